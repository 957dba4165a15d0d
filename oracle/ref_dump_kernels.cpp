// Build-time helper (test infrastructure): links the REFERENCE's own kernel-registration translation units
// (operators/cl_kernels/*.cpp, compiled in place from the reference tree) and writes the OpenCL C text of the
// quantized kernels on the hot path, with the private headers the reference prepends (CLRuntime.cpp:764-779),
// to a generated include file.  oracle/ref_kernels_shim.cpp compiles that text as C++ behind a small
// OpenCL-compatibility prelude, so the CPU oracle can be compared with the reference's own kernel bodies.
#include <cstdio>
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
        std::fprintf(f, "%s\n\n", kit->second.c_str());
    }
    std::fclose(f);
    return missing ? 4 : 0;
}
