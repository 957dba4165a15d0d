// Drives the operators through the C++ adapter classes exactly as OperationConstructor / EnnUDOperator drive the
// OpenCL ones: create tensors, fill *Parameters, initialize(), execute(), read back.  Checks
//   1. the reference known-answer test gpu_userdriver_test.cc:474-575 (ANDROID_NN, NCHW, per-channel int8 weights);
//   2. a seeded NHWC per-tensor 3x3 convolution and a per-channel depthwise convolution against the CPU oracle.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "../cl-eden-kernel_b200/adapter/b200_operators.hpp"

extern "C" {
int32_t orc_conv2d(const enn_b200_conv_desc *, const void *, const void *, const int32_t *, const float *, void *);
int32_t orc_depthwise(const enn_b200_conv_desc *, const void *, const void *, const int32_t *, const float *, void *);
}

using namespace enn::ud::b200;

static int fails = 0;
#define CHECK(c)                                                  \
    do {                                                          \
        if (!(c)) {                                               \
            std::printf("FAILED %s:%d %s\n", __FILE__, __LINE__, #c); \
            ++fails;                                              \
        }                                                         \
    } while (0)

int main() {
    B200ComputeLibrary lib(0);
    if (lib.runtime()->status() != Status::SUCCESS) {
        std::printf("no device\n");
        return 2;
    }
    {   // 1. reference KAT
        uint8_t input_data[] = {138, 138, 138, 108, 108, 108};
        int8_t weight_data[] = {1, 2, 1, 2, 1, 2};
        int bias_data[] = {4, 4, 4};
        uint8_t expect[] = {121, 121, 121, 118, 118, 118, 115, 115, 115};
        auto ifm = lib.create_and_copy_tensor(DataType::UINT8, input_data, Dim4{1, 2, 3, 1}, DataOrder::NCHW, 0.5f, 128);
        auto w = lib.create_and_copy_tensor(DataType::INT8, weight_data, Dim4{3, 1, 1, 2}, DataOrder::NCHW, 0.0f, 0);
        auto b = lib.create_and_copy_tensor(DataType::INT32, bias_data, Dim4{3, 1, 1, 1}, DataOrder::NCHW, 1.0f, 0);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{1, 3, 3, 1}, DataOrder::NCHW, 1.0f, 128);
        auto p = std::make_shared<ConvolutionParameters>();
        p->per_channel_quant = true;
        p->androidNN = true;
        p->isNCHW = true;
        p->scales = {0.5f, 0.75f, 1.0f};
        auto conv = lib.createConvolution(PrecisionType::UINT8);
        CHECK(conv->initialize({ifm, w, b}, {ofm}, p) == Status::SUCCESS);
        CHECK(conv->execute() == Status::SUCCESS);
        uint8_t out[9] = {0};
        CHECK(ofm->readData(out) == Status::SUCCESS);
        for (int i = 0; i < 9; ++i) CHECK(out[i] == expect[i]);
        CHECK(conv->release() == Status::SUCCESS);
    }
    std::mt19937 rng(7);
    {   // 2a. NHWC per-tensor 3x3 convolution, RELU6
        const uint32_t N = 2, H = 14, W = 15, CI = 16, CO = 24;
        std::vector<uint8_t> x(N * H * W * CI), wt(CO * 3 * 3 * CI), y(N * H * W * CO), y_ref(y.size());
        std::vector<int32_t> bias(CO);
        for (auto &v : x) v = rng() & 255;
        for (auto &v : wt) v = rng() & 255;
        for (auto &v : bias) v = static_cast<int32_t>(rng() % 2001) - 1000;
        // NHWC tensors carry {n, h, w, c} in the (n, c, h, w) slots
        auto ifm = lib.create_and_copy_tensor(DataType::UINT8, x.data(), Dim4{N, H, W, CI}, DataOrder::NHWC, 0.02f, 128);
        auto w = lib.create_and_copy_tensor(DataType::UINT8, wt.data(), Dim4{CO, 3, 3, CI}, DataOrder::NHWC, 0.005f, 127);
        auto b = lib.create_and_copy_tensor(DataType::INT32, bias.data(), Dim4{CO, 1, 1, 1}, DataOrder::NHWC, 0.02f * 0.005f, 0);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{N, H, W, CO}, DataOrder::NHWC, 0.05f, 128);
        auto p = std::make_shared<ConvolutionParameters>();
        p->padding = {1, 1, 1, 1};
        p->androidNN = true;
        p->isNCHW = false;
        p->activation_info = std::make_shared<ActivationInfo>(ActivationInfo::ActivationType::RELU6, true);
        auto conv = lib.createConvolution(PrecisionType::UINT8);
        CHECK(conv->initialize({ifm, w, b}, {ofm}, p) == Status::SUCCESS);
        CHECK(conv->execute() == Status::SUCCESS);
        CHECK(ofm->readData(y.data()) == Status::SUCCESS);
        enn_b200_conv_desc d{};
        d.n = N; d.h = H; d.w = W; d.cin = CI; d.cout = CO; d.kh = d.kw = 3; d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1;
        d.pad_t = d.pad_r = d.pad_b = d.pad_l = 1; d.groups = 1; d.activation = ENN_B200_ACT_RELU6; d.weight_layout = ENN_B200_W_OHWI;
        d.in_scale = 0.02f; d.in_zp = 128; d.w_scale = 0.005f; d.w_zp = 127; d.bias_scale = 0.02f * 0.005f; d.out_scale = 0.05f; d.out_zp = 128;
        orc_conv2d(&d, x.data(), wt.data(), bias.data(), nullptr, y_ref.data());
        size_t bad = 0;
        for (size_t i = 0; i < y.size(); ++i) bad += y[i] != y_ref[i];
        CHECK(bad == 0);
    }
    {   // 2b. NHWC per-channel depthwise 3x3 stride 2, weights [C][1][3][3]
        const uint32_t N = 2, H = 12, W = 12, C = 8;
        std::vector<uint8_t> x(N * H * W * C), y(N * 6 * 6 * C), y_ref(y.size());
        std::vector<int8_t> wt(C * 9);
        std::vector<int32_t> bias(C);
        std::vector<float> scales(C);
        for (auto &v : x) v = rng() & 255;
        for (auto &v : wt) v = static_cast<int8_t>(static_cast<int>(rng() % 255) - 127);
        for (auto &v : bias) v = static_cast<int32_t>(rng() % 1001) - 500;
        for (auto &v : scales) v = 0.001f + 0.0001f * (rng() % 500);
        auto ifm = lib.create_and_copy_tensor(DataType::UINT8, x.data(), Dim4{N, H, W, C}, DataOrder::NHWC, 0.02f, 128);
        auto w = lib.create_and_copy_tensor(DataType::INT8, wt.data(), Dim4{C, 1, 3, 3}, DataOrder::NCHW, 0.0f, 0);
        auto b = lib.create_and_copy_tensor(DataType::INT32, bias.data(), Dim4{C, 1, 1, 1}, DataOrder::NCHW, 1.0f, 0);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{N, 6, 6, C}, DataOrder::NHWC, 0.04f, 0);
        auto p = std::make_shared<DepthwiseConvolutionParameters>();
        p->padding = {0, 1, 1, 0};
        p->stride = {2, 2};
        p->per_channel_quant = true;
        p->isNCHW = false;
        p->scales = scales;
        p->activation_info = std::make_shared<ActivationInfo>(ActivationInfo::ActivationType::RELU6, true);
        auto dw = lib.createDepthwiseConvolution(PrecisionType::UINT8);
        CHECK(dw->initialize({ifm, w, b}, {ofm}, p) == Status::SUCCESS);
        CHECK(dw->execute() == Status::SUCCESS);
        CHECK(ofm->readData(y.data()) == Status::SUCCESS);
        enn_b200_conv_desc d{};
        d.n = N; d.h = H; d.w = W; d.cin = C; d.cout = C; d.kh = d.kw = 3; d.stride_h = d.stride_w = 2; d.dil_h = d.dil_w = 1;
        d.pad_t = 0; d.pad_r = 1; d.pad_b = 1; d.pad_l = 0; d.groups = 1; d.activation = ENN_B200_ACT_RELU6; d.weight_layout = ENN_B200_W_OIHW;
        d.weight_dtype = ENN_B200_S8; d.per_channel = 1;
        d.in_scale = 0.02f; d.in_zp = 128; d.out_scale = 0.04f; d.out_zp = 0;
        orc_depthwise(&d, x.data(), wt.data(), bias.data(), scales.data(), y_ref.data());
        size_t bad = 0;
        for (size_t i = 0; i < y.size(); ++i) bad += y[i] != y_ref[i];
        CHECK(bad == 0);
    }
    {   // 3. error convention: wrong parameter type -> INVALID_PARAMS, no exception crosses the interface
        auto conv = lib.createConvolution(PrecisionType::UINT8);
        CHECK(conv->initialize({}, {}, std::make_shared<FullyConnectedParameters>()) == Status::INVALID_PARAMS);
        CHECK(conv->execute() == Status::FAILURE);
    }
    std::printf(fails ? "adapter test: %d failures\n" : "adapter test: OK\n", fails);
    return fails ? 1 : 0;
}
