// Build-time helper (test infrastructure): links the REFERENCE's own kernel-registration translation units
// (operators/cl_kernels/*.cpp, compiled in place from the reference tree) and writes the OpenCL C text of the
// quantized kernels on the hot path, with the private headers the reference prepends (CLRuntime.cpp:764-779),
// to a generated include file.  oracle/ref_kernels_shim.cpp compiles that text as C++ behind a small
// OpenCL-compatibility prelude, so the CPU oracle can be compared with the reference's own kernel bodies.
#include <cstdio>
#include <regex>
#include <string>
#include <vector>

#include "userdriver/gpu/common/CLKernels.hpp"

using namespace enn::ud::gpu;

int main(int argc, char **argv) {
    if (argc < 2) return 2;
    const std::vector<std::string> names = {
        "conv_per_channel_quantized_INT8", "depthwise_conv_INT8", "depthwise_conv_per_channel_INT8", "depthwise_conv_unequal_INT8",
        "matrixTrans_INT8", "weightAlign_INT8", "convBackGemmRXR_INT8", "convertBottomDiff2_INT8",
        "PERCHANNELconvBackGemmRXR_INT8", "convertBottomDiff2_per_channel_INT8", "avepooling_tflite_INT8",
        "eltwiseAddQuantized_opt_INT8",
        // per-tensor GEMM convolution (CLGEMMConvolutionQuantized + CLPadConvert)
        "pad_opt_INT8", "convert_optimized_INT8", "convertBlocked2_INT8", "alignQuantizedWeight_gemm_INT8", "quantizedGemmBlocked_INT8",
        // remaining quantized graph operators
        "maxpooling_INT8", "mean_feature_opt_INT8", "sum_axis_INT8", "mean_INT8", "concat_axis1_INT8", "resize_bilinear_INT8",
    };
    FILE *f = std::fopen(argv[1], "w");
    if (!f) return 3;
    std::fprintf(f, "// GENERATED at build time from the reference tree by oracle/ref_dump_kernels.cpp - not committed.\n");
    std::vector<bool> header_done(NUM_OF_PRIVATE_KERNEL_HEADER, false);
    int missing = 0;
    for (const auto &n : names) {
        auto hit = Kernels::KernelHeaderMap().find(n);
        if (hit != Kernels::KernelHeaderMap().end())
            for (auto h : hit->second)
                if (!header_done[h]) {
                    header_done[h] = true;
                    std::fprintf(f, "%s\n", private_kernel_header[h]);
                }
        auto kit = Kernels::KernelMap().find(n);
        if (kit == Kernels::KernelMap().end()) {
            std::fprintf(stderr, "kernel %s not found in the reference registry\n", n.c_str());
            ++missing;
            continue;
        }
        // OpenCL multi-component swizzles (.s0123, .s89ab ...) are no C++ member names: every one the hot-path kernels
        // use is a run of consecutive components, written out as .sub<length>(first) for the shim's vector types.
        std::string text = kit->second;
        static const std::regex swz("\\.s([0-9a-f]{2,})\\b");
        std::string outp;
        auto it = std::sregex_iterator(text.begin(), text.end(), swz);
        size_t pos = 0;
        for (; it != std::sregex_iterator(); ++it) {
            const std::string comps = (*it)[1].str();
            auto val = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
            bool run = true;
            for (size_t i = 1; i < comps.size(); ++i) run = run && val(comps[i]) == val(comps[i - 1]) + 1;
            if (!run) {
                std::fprintf(stderr, "kernel %s: swizzle .s%s is not a run of consecutive components\n", n.c_str(), comps.c_str());
                ++missing;
            }
            outp += text.substr(pos, it->position() - pos);
            outp += ".sub<" + std::to_string(comps.size()) + ">(" + std::to_string(val(comps[0])) + ")";
            pos = it->position() + it->length();
        }
        outp += text.substr(pos);
        std::fprintf(f, "%s\n\n", outp.c_str());
    }
    std::fclose(f);
    return missing ? 4 : 0;
}
