// Drives the operators through the C++ adapter classes exactly as OperationConstructor / EnnUDOperator drive the
// OpenCL ones: create tensors, fill *Parameters, initialize(), execute(), read back.  Checks
//   1. the reference known-answer test gpu_userdriver_test.cc:474-575 (ANDROID_NN, NCHW, per-channel int8 weights);
//   2. seeded convolution, depthwise convolution, deconvolution, fully connected, add and average pool against the
//      CPU oracle, a convolution whose filter and bias are runtime tensors, and the ITensor members the executor uses.
// Builds against the stand-in declarations or, with -DENN_B200_WITH_REFERENCE_HEADERS, against the reference's own.
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "../cl-eden-kernel_b200/adapter/b200_operators.hpp"

extern "C" {
int32_t orc_conv2d(const enn_b200_conv_desc *, const void *, const void *, const int32_t *, const float *, void *);
int32_t orc_depthwise(const enn_b200_conv_desc *, const void *, const void *, const int32_t *, const float *, void *);
int32_t orc_deconv(const enn_b200_conv_desc *, const void *, const void *, const int32_t *, const float *, void *);
int32_t orc_fc(const enn_b200_fc_desc *, const void *, const void *, const int32_t *, const float *, void *);
int32_t orc_add(const enn_b200_add_desc *, const void *, const void *, void *);
int32_t orc_avgpool(const enn_b200_pool_desc *, const void *, void *);
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
    {   // 2c. deconvolution, Caffe-style [Cin][Cout][Kh][Kw] filter, NCHW tensors, 4x4 stride 2 pad 1
        const uint32_t N = 1, H = 6, W = 7, CI = 16, CO = 8, K = 4;
        const uint32_t OH = H * 2 + K - 2 - 2, OW = W * 2 + K - 2 - 2;
        std::vector<uint8_t> x_nhwc(N * H * W * CI), x(x_nhwc.size()), wt(CI * CO * K * K), y(N * CO * OH * OW), y_ref(y.size());
        std::vector<int32_t> bias(CO);
        for (auto &v : x_nhwc) v = rng() & 255;
        for (auto &v : wt) v = rng() & 255;
        for (auto &v : bias) v = static_cast<int32_t>(rng() % 2001) - 1000;
        for (uint32_t h = 0; h < H; ++h)
            for (uint32_t w = 0; w < W; ++w)
                for (uint32_t c = 0; c < CI; ++c) x[(c * H + h) * W + w] = x_nhwc[(h * W + w) * CI + c];
        auto ifm = lib.create_and_copy_tensor(DataType::UINT8, x.data(), Dim4{N, CI, H, W}, DataOrder::NCHW, 0.02f, 128);
        auto w = lib.create_and_copy_tensor(DataType::UINT8, wt.data(), Dim4{CI, CO, K, K}, DataOrder::NCHW, 0.004f, 120);
        auto b = lib.create_and_copy_tensor(DataType::INT32, bias.data(), Dim4{CO, 1, 1, 1}, DataOrder::NCHW, 0.02f * 0.004f, 0);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{N, CO, OH, OW}, DataOrder::NCHW, 0.05f, 128);
        auto p = std::make_shared<DeconvolutionParameters>();
        p->padding = {1, 1, 1, 1};
        p->stride = {2, 2};
        p->isNCHW = true;
        auto dc = lib.createDeconvolution(PrecisionType::UINT8);
        CHECK(dc->initialize({ifm, w, b}, {ofm}, p) == Status::SUCCESS);
        CHECK(dc->execute() == Status::SUCCESS);
        CHECK(ofm->readData(y.data()) == Status::SUCCESS);
        enn_b200_conv_desc d{};
        d.n = N; d.h = H; d.w = W; d.cin = CI; d.cout = CO; d.kh = d.kw = K; d.stride_h = d.stride_w = 2; d.dil_h = d.dil_w = 1;
        d.pad_t = d.pad_r = d.pad_b = d.pad_l = 1; d.groups = 1; d.weight_layout = ENN_B200_W_IOHW;
        d.in_scale = 0.02f; d.in_zp = 128; d.w_scale = 0.004f; d.w_zp = 120; d.bias_scale = 0.02f * 0.004f; d.out_scale = 0.05f; d.out_zp = 128;
        orc_deconv(&d, x_nhwc.data(), wt.data(), bias.data(), nullptr, y_ref.data());      // NHWC out
        size_t bad = 0;
        for (uint32_t h = 0; h < OH; ++h)
            for (uint32_t w2 = 0; w2 < OW; ++w2)
                for (uint32_t c = 0; c < CO; ++c) bad += y[(c * OH + h) * OW + w2] != y_ref[(h * OW + w2) * CO + c];
        CHECK(bad == 0);
    }
    {   // 2d. fully connected, [Nout][K] filter, batch 3
        const uint32_t M = 3, K = 192, NO = 40;
        std::vector<uint8_t> x(M * K), wt(NO * K), y(M * NO), y_ref(y.size());
        std::vector<int32_t> bias(NO);
        for (auto &v : x) v = rng() & 255;
        for (auto &v : wt) v = rng() & 255;
        for (auto &v : bias) v = static_cast<int32_t>(rng() % 4001) - 2000;
        auto ifm = lib.create_and_copy_tensor(DataType::UINT8, x.data(), Dim4{M, K, 1, 1}, DataOrder::NCHW, 0.03f, 127);
        auto w = lib.create_and_copy_tensor(DataType::UINT8, wt.data(), Dim4{NO, K, 1, 1}, DataOrder::NCHW, 0.006f, 131);
        auto b = lib.create_and_copy_tensor(DataType::INT32, bias.data(), Dim4{NO, 1, 1, 1}, DataOrder::NCHW, 0.03f * 0.006f, 0);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{M, NO, 1, 1}, DataOrder::NCHW, 0.09f, 120);
        auto p = std::make_shared<FullyConnectedParameters>();
        p->activation_info = std::make_shared<ActivationInfo>(ActivationInfo::ActivationType::RELU, true);
        auto fc = lib.createFullyConnected(PrecisionType::UINT8);
        CHECK(fc->initialize({ifm, w, b}, {ofm}, p) == Status::SUCCESS);
        float us = -1.f;
        CHECK(fc->lastExecuteMicroseconds(&us) == Status::INVALID_PARAMS);      // profiling is off by default
        CHECK(fc->setProfiling(true) == Status::SUCCESS);
        CHECK(fc->execute() == Status::SUCCESS);
        CHECK(fc->lastExecuteMicroseconds(&us) == Status::SUCCESS && us > 0.f && us < 1e5f);
        CHECK(ofm->readData(y.data()) == Status::SUCCESS);
        enn_b200_fc_desc d{};
        d.m = M; d.k = K; d.n = NO; d.activation = ENN_B200_ACT_RELU;
        d.in_scale = 0.03f; d.in_zp = 127; d.w_scale = 0.006f; d.w_zp = 131; d.bias_scale = 0.03f * 0.006f; d.out_scale = 0.09f; d.out_zp = 120;
        orc_fc(&d, x.data(), wt.data(), bias.data(), nullptr, y_ref.data());
        size_t bad = 0;
        for (size_t i = 0; i < y.size(); ++i) bad += y[i] != y_ref[i];
        CHECK(bad == 0);
    }
    {   // 2e. quantized add of two tensors with different scales
        const uint32_t N = 2, H = 9, W = 11, C = 24;
        std::vector<uint8_t> a(N * H * W * C), c2(a.size()), y(a.size()), y_ref(a.size());
        for (auto &v : a) v = rng() & 255;
        for (auto &v : c2) v = rng() & 255;
        auto t0 = lib.create_and_copy_tensor(DataType::UINT8, a.data(), Dim4{N, H, W, C}, DataOrder::NHWC, 0.021f, 120);
        auto t1 = lib.create_and_copy_tensor(DataType::UINT8, c2.data(), Dim4{N, H, W, C}, DataOrder::NHWC, 0.034f, 131);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{N, H, W, C}, DataOrder::NHWC, 0.05f, 126);
        auto p = std::make_shared<AddParameters>();
        auto add = lib.createAdd(PrecisionType::UINT8);
        CHECK(add->initialize({t0, t1}, {ofm}, p) == Status::SUCCESS);
        CHECK(add->execute() == Status::SUCCESS);
        CHECK(ofm->readData(y.data()) == Status::SUCCESS);
        enn_b200_add_desc d{};
        d.count = static_cast<int64_t>(a.size());
        d.in0_scale = 0.021f; d.in0_zp = 120; d.in1_scale = 0.034f; d.in1_zp = 131; d.out_scale = 0.05f; d.out_zp = 126;
        orc_add(&d, a.data(), c2.data(), y_ref.data());
        size_t bad = 0;
        for (size_t i = 0; i < y.size(); ++i) bad += y[i] != y_ref[i];
        CHECK(bad == 0);
    }
    {   // 2f. average pool 7x7 -> 1x1 (the network head) and 3x3 stride 2 with padding
        for (int variant = 0; variant < 2; ++variant) {
            const uint32_t N = 2, H = variant ? 10 : 7, W = H, C = 32;
            const uint32_t K = variant ? 3 : 7, S = variant ? 2 : 1, P = variant ? 1 : 0;
            const uint32_t OH = (H + 2 * P - K) / S + 1;
            std::vector<uint8_t> x(N * H * W * C), y(N * OH * OH * C), y_ref(y.size());
            for (auto &v : x) v = rng() & 255;
            auto ifm = lib.create_and_copy_tensor(DataType::UINT8, x.data(), Dim4{N, H, W, C}, DataOrder::NHWC, 0.02f, 3);
            auto ofm = lib.create_tensor(DataType::UINT8, Dim4{N, OH, OH, C}, DataOrder::NHWC, 0.02f, 3);
            auto p = std::make_shared<Pool2DParameters>();
            p->filter = {K, K};
            p->stride = {S, S};
            p->padding = {P, P, P, P};
            p->isNCHW = false;
            auto pool = lib.createAveragepool(PrecisionType::UINT8);
            CHECK(pool->initialize({ifm}, {ofm}, p) == Status::SUCCESS);
            CHECK(pool->execute() == Status::SUCCESS);
            CHECK(ofm->readData(y.data()) == Status::SUCCESS);
            enn_b200_pool_desc d{};
            d.n = N; d.h = H; d.w = W; d.c = C; d.kh = d.kw = K; d.stride_h = d.stride_w = S; d.pad_t = d.pad_l = P; d.out_h = d.out_w = OH;
            d.out_scale = 0.02f; d.out_zp = 3;
            orc_avgpool(&d, x.data(), y_ref.data());
            size_t bad = 0;
            for (size_t i = 0; i < y.size(); ++i) bad += y[i] != y_ref[i];
            CHECK(bad == 0);
        }
    }
    {   // 2g. filter and bias that are not constant tensors: read from their device buffers at every execute()
        const uint32_t N = 1, H = 10, W = 10, CI = 16, CO = 16;
        std::vector<uint8_t> x(N * H * W * CI), wt(CO * CI), y(N * H * W * CO), y_ref(y.size());
        std::vector<int32_t> bias(CO);
        for (auto &v : x) v = rng() & 255;
        auto ifm = lib.create_and_copy_tensor(DataType::UINT8, x.data(), Dim4{N, H, W, CI}, DataOrder::NHWC, 0.02f, 128);
        auto w = lib.create_tensor(DataType::UINT8, Dim4{CO, 1, 1, CI}, DataOrder::NHWC, 0.005f, 127);
        auto b = lib.create_tensor(DataType::INT32, Dim4{CO, 1, 1, 1}, DataOrder::NHWC, 0.02f * 0.005f, 0);
        auto ofm = lib.create_tensor(DataType::UINT8, Dim4{N, H, W, CO}, DataOrder::NHWC, 0.03f, 100);
        CHECK(!w->is_const() && !b->is_const());
        auto p = std::make_shared<ConvolutionParameters>();
        p->androidNN = true;
        p->isNCHW = false;
        auto conv = lib.createConvolution(PrecisionType::UINT8);
        CHECK(conv->initialize({ifm, w, b}, {ofm}, p) == Status::SUCCESS);
        enn_b200_conv_desc d{};
        d.n = N; d.h = H; d.w = W; d.cin = CI; d.cout = CO; d.kh = d.kw = 1; d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1;
        d.groups = 1; d.weight_layout = ENN_B200_W_OHWI;
        d.in_scale = 0.02f; d.in_zp = 128; d.w_scale = 0.005f; d.w_zp = 127; d.bias_scale = 0.02f * 0.005f; d.out_scale = 0.03f; d.out_zp = 100;
        for (int round = 0; round < 2; ++round) {
            for (auto &v : wt) v = rng() & 255;
            for (auto &v : bias) v = static_cast<int32_t>(rng() % 2001) - 1000;
            CHECK(w->writeData(wt.data()) == Status::SUCCESS);
            CHECK(b->writeData(bias.data()) == Status::SUCCESS);
            CHECK(conv->execute() == Status::SUCCESS);
            CHECK(ofm->readData(y.data()) == Status::SUCCESS);
            orc_conv2d(&d, x.data(), wt.data(), bias.data(), nullptr, y_ref.data());
            size_t bad = 0;
            for (size_t i = 0; i < y.size(); ++i) bad += y[i] != y_ref[i];
            CHECK(bad == 0);
        }
    }
    {   // 2h. the ITensor members the executor and the operator constructor use
        uint8_t data[24];
        for (int i = 0; i < 24; ++i) data[i] = static_cast<uint8_t>(i);
        auto t = std::make_shared<B200Tensor>(lib.runtime(), DataType::UINT8, Dim4{1, 2, 3, 4}, DataOrder::NCHW, 0.5f, 7);
        CHECK(t->getNumOfDims() == 4 && t->getDims(1) == 2 && t->getDims(-1) == 4 && t->getTotalSizeFromDims() == 24);
        CHECK(t->getPrecisionType() == PrecisionType::UINT8);
        CHECK(t->writeData(data) == Status::SUCCESS);
        uint8_t nhwc[24], back[24];
        CHECK(t->readData(nhwc, true, DataOrderChangeType::NCHW2NHWC) == Status::SUCCESS);
        CHECK(nhwc[1] == 12 && nhwc[2] == 1);                       // (h0, w0, c1) = NCHW element 12
        CHECK(t->reorder(DataOrder::NHWC) == Status::SUCCESS);      // on the device
        CHECK(t->getDataOrder() == DataOrder::NHWC && t->getDim().c == 3 && t->getDim().w == 2);
        CHECK(t->readData(back) == Status::SUCCESS);
        for (int i = 0; i < 24; ++i) CHECK(back[i] == nhwc[i]);
        CHECK(t->reorder(DataOrder::NCHW) == Status::SUCCESS);
        CHECK(t->readData(back) == Status::SUCCESS);
        for (int i = 0; i < 24; ++i) CHECK(back[i] == data[i]);
        t->setScale(0.25f);
        t->setZeroPoint(9);
        t->set_buffer_index(5);
        t->set_buffer_type(2);
        CHECK(t->getScale() == 0.25f && t->getZeroPoint() == 9 && t->get_buffer_index() == 5 && t->get_buffer_type() == 2);
        CHECK(t->reconfigureDimAndBuffer(Dim4{2, 2, 3, 4}) == Status::SUCCESS && t->getNumOfBytes() == 48);
        CHECK(t->reconfigureDim(Dim4{1, 1, 3, 4}) == Status::SUCCESS && t->getNumOfBytes() == 12);
        // pooled memory assigned by the executor
        void *pool = nullptr;
        CHECK(enn_b200_malloc(lib.runtime()->context(), 64, &pool) == ENN_B200_SUCCESS);
        t->set_buffer_ptr(pool);
        CHECK(t->getDataPtr() == pool);
        CHECK(t->writeData(data) == Status::SUCCESS && t->readData(back) == Status::SUCCESS && back[11] == 11);
        t.reset();                                                   // does not free memory it does not own
        CHECK(enn_b200_free(lib.runtime()->context(), pool) == ENN_B200_SUCCESS);
    }
    {   // 3. error convention: wrong parameter type -> INVALID_PARAMS, no exception crosses the interface
        auto conv = lib.createConvolution(PrecisionType::UINT8);
        CHECK(conv->initialize({}, {}, std::make_shared<FullyConnectedParameters>()) == Status::INVALID_PARAMS);
        CHECK(conv->execute() == Status::FAILURE);
    }
    std::printf(fails ? "adapter test: %d failures\n" : "adapter test: OK\n", fails);
    return fails ? 1 : 0;
}
