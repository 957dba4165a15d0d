#include "b200_operators.hpp"

#include <cstring>

namespace enn {
namespace ud {
namespace b200 {

namespace {

int32_t act_code(const ActivationInfo &a) {
    if (!a.isEnabled()) return ENN_B200_ACT_NONE;
    switch (a.activation()) {
        case ActivationInfo::ActivationType::RELU: return ENN_B200_ACT_RELU;
        case ActivationInfo::ActivationType::RELU1: return ENN_B200_ACT_RELU1;
        case ActivationInfo::ActivationType::RELU6: return ENN_B200_ACT_RELU6;
        default: return ENN_B200_ACT_NONE;
    }
}

// Tensors report NCHW-named dims; an NHWC tensor of an ANDROID_NN / TFLite model stores {n, h, w, c} in the
// same four slots (Common.hpp convertDimToNCHW), so normalise to logical (n, c, h, w).
Dim4 logical_dim(const std::shared_ptr<ITensor> &t, bool nchw) {
    const Dim4 d = t->getDim();
    if (nchw) return d;
    return Dim4{d.n, d.w, d.c, d.h};
}

const void *host_bytes(const std::shared_ptr<ITensor> &t, std::vector<uint8_t> *tmp) {
    auto bt = std::dynamic_pointer_cast<B200Tensor>(t);
    if (bt && !bt->hostCopy().empty()) return bt->hostCopy().data();
    tmp->resize(t->getNumOfBytes());
    t->readData(tmp->data());
    return tmp->data();
}

}  // namespace

Status B200OperatorBase::ensure_nhwc_staging(bool nchw) {
    nchw_ = nchw;
    if (!nchw) return Status::SUCCESS;
    // NCHW models: the kernels are NHWC-native, so convert in and out (the reference does the opposite around
    // its NCHW kernels, CLConvolution.cpp:468-483).
    if (enn_b200_malloc(runtime_->context(), inputs_[0]->getNumOfBytes(), &in_nhwc_) != ENN_B200_SUCCESS) return Status::CL_FAILURE;
    if (enn_b200_malloc(runtime_->context(), outputs_[0]->getNumOfBytes(), &out_nhwc_) != ENN_B200_SUCCESS) return Status::CL_FAILURE;
    return Status::SUCCESS;
}

Status B200OperatorBase::prepare_conv_like(int kind, const enn_b200_conv_desc &desc, const std::shared_ptr<ITensor> &weight,
                                           const std::shared_ptr<ITensor> &bias, const std::vector<float> &scales) {
    // A filter or bias that is not a constant tensor is read from its device buffer at every execute()
    // (CLConvolution.cpp:75-76, CLDepthwiseConvolution.cpp:121; the deconvolution says so in its parameters).
    enn_b200_conv_desc d = desc;
    runtime_weights_ = d.weights_as_input != 0 || !weight->is_const();
    runtime_bias_ = !bias->is_const();
    d.weights_as_input = runtime_weights_;
    d.bias_as_input = runtime_bias_;
    std::vector<uint8_t> wt, bt;
    const void *w = runtime_weights_ ? nullptr : host_bytes(weight, &wt);
    const int32_t *b = runtime_bias_ ? nullptr : static_cast<const int32_t *>(host_bytes(bias, &bt));
    const float *sc = d.per_channel ? scales.data() : nullptr;
    if (d.per_channel && static_cast<int64_t>(scales.size()) < d.cout) return Status::INVALID_PARAMS;
    int32_t st;
    if (kind == 0) st = enn_b200_conv2d_prepare(runtime_->context(), &d, w, b, sc, &op_);
    else if (kind == 1) st = enn_b200_depthwise_prepare(runtime_->context(), &d, w, b, sc, &op_);
    else st = enn_b200_deconv_prepare(runtime_->context(), &d, w, b, sc, &op_);
    return to_status(st);
}

Status B200OperatorBase::setProfiling(bool on) {
    if (on && !timer_) return to_status(enn_b200_timer_create(runtime_->context(), &timer_));
    if (!on && timer_) {
        enn_b200_timer_destroy(timer_);
        timer_ = nullptr;
    }
    return Status::SUCCESS;
}

Status B200OperatorBase::lastExecuteMicroseconds(float *us) {
    if (!timer_ || !us) return Status::INVALID_PARAMS;
    return to_status(enn_b200_timer_elapsed_us(timer_, us));
}

Status B200OperatorBase::execute() {
    if (!timer_) return run();
    enn_b200_timer_start(timer_);
    const Status s = run();
    enn_b200_timer_stop(timer_);
    return s;
}

Status B200OperatorBase::run() {
    if (!op_) return Status::FAILURE;
    enn_b200_context *ctx = runtime_->context();
    const void *in = device_ptr(inputs_[0]);
    void *out = device_ptr(outputs_[0]);
    if (!in || !out) return Status::INVALID_PARAMS;      // not a tensor of this driver, or no buffer assigned yet
    int32_t st;
    if (runtime_weights_ || runtime_bias_) {
        st = enn_b200_op_rebind_constants(op_, device_ptr(inputs_[1]), static_cast<const int32_t *>(device_ptr(inputs_[2])));
        if (st != ENN_B200_SUCCESS) return to_status(st);
    }
    if (nchw_) {
        st = enn_b200_nchw_to_nhwc(ctx, in, in_nhwc_, in_dim_.n, in_dim_.c, in_dim_.h, in_dim_.w);
        if (st != ENN_B200_SUCCESS) return to_status(st);
        st = enn_b200_op_execute(op_, in_nhwc_, out_nhwc_);
        if (st != ENN_B200_SUCCESS) return to_status(st);
        return to_status(enn_b200_nhwc_to_nchw(ctx, out_nhwc_, out, out_dim_.n, out_dim_.c, out_dim_.h, out_dim_.w));
    }
    if (two_inputs_) return to_status(enn_b200_op_execute2(op_, in, device_ptr(inputs_[1]), out));
    return to_status(enn_b200_op_execute(op_, in, out));
}

Status B200OperatorBase::release() {
    if (op_) enn_b200_op_release(op_);
    op_ = nullptr;
    if (in_nhwc_) enn_b200_free(runtime_->context(), in_nhwc_);
    if (out_nhwc_) enn_b200_free(runtime_->context(), out_nhwc_);
    in_nhwc_ = out_nhwc_ = nullptr;
    if (timer_) enn_b200_timer_destroy(timer_);
    timer_ = nullptr;
    return Status::SUCCESS;
}

static void fill_common(enn_b200_conv_desc *d, const Dim4 &in, const Dim4 &out, PrecisionType precision, const std::shared_ptr<ITensor> &ifm,
                        const std::shared_ptr<ITensor> &w, const std::shared_ptr<ITensor> &bias, const std::shared_ptr<ITensor> &ofm,
                        bool per_channel) {
    std::memset(d, 0, sizeof(*d));
    d->n = in.n; d->h = in.h; d->w = in.w; d->cin = in.c;
    d->cout = out.c;
    d->out_h = out.h; d->out_w = out.w;
    d->dil_h = d->dil_w = 1;
    d->act_dtype = precision == PrecisionType::INT8 ? ENN_B200_S8 : ENN_B200_U8;
    // Per-channel filters are int8 ("char" in the kernels); per-tensor filters share the activation type.
    d->weight_dtype = per_channel ? ENN_B200_S8 : (w->getDataType() == DataType::INT8 ? ENN_B200_S8 : ENN_B200_U8);
    d->per_channel = per_channel;
    d->in_scale = ifm->getScale(); d->in_zp = ifm->getZeroPoint();
    d->w_scale = w->getScale(); d->w_zp = w->getZeroPoint();
    d->bias_scale = bias->getScale();
    d->out_scale = ofm->getScale(); d->out_zp = ofm->getZeroPoint();
}

Status B200Convolution::initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                                   std::shared_ptr<Parameters> parameters) {
    auto p = std::dynamic_pointer_cast<ConvolutionParameters>(parameters);
    if (!p || inputs.size() < 3 || outputs.empty()) return Status::INVALID_PARAMS;
    inputs_ = inputs; outputs_ = outputs;
    const bool nchw = p->isNCHW;
    in_dim_ = logical_dim(inputs[0], nchw);
    out_dim_ = logical_dim(outputs[0], nchw);
    enn_b200_conv_desc d;
    fill_common(&d, in_dim_, out_dim_, precision_, inputs[0], inputs[1], inputs[2], outputs[0], p->per_channel_quant);
    const Dim4 wd = inputs[1]->getDim();
    // ANDROID_NN kernels are [Cout][Kh][Kw][Cin] stored in the (n, c, h, w) slots; others are OIHW (CLConvolution.cpp:97-98).
    d.kh = p->androidNN ? wd.c : wd.h;
    d.kw = p->androidNN ? wd.h : wd.w;
    d.weight_layout = p->androidNN ? ENN_B200_W_OHWI : ENN_B200_W_OIHW;
    d.stride_h = p->stride.h; d.stride_w = p->stride.w;
    d.dil_h = p->dilation.h; d.dil_w = p->dilation.w;
    d.pad_t = p->padding.t; d.pad_r = p->padding.r; d.pad_b = p->padding.b; d.pad_l = p->padding.l;
    d.groups = p->group_size;
    d.activation = act_code(*p->activation_info);
    Status s = ensure_nhwc_staging(nchw);
    if (s != Status::SUCCESS) return s;
    return prepare_conv_like(0, d, inputs[1], inputs[2], p->scales);
}

Status B200DepthwiseConvolution::initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                                            std::shared_ptr<Parameters> parameters) {
    auto p = std::dynamic_pointer_cast<DepthwiseConvolutionParameters>(parameters);
    if (!p || inputs.size() < 3 || outputs.empty()) return Status::INVALID_PARAMS;
    inputs_ = inputs; outputs_ = outputs;
    const bool nchw = p->isNCHW;
    in_dim_ = logical_dim(inputs[0], nchw);
    out_dim_ = logical_dim(outputs[0], nchw);
    enn_b200_conv_desc d;
    fill_common(&d, in_dim_, out_dim_, precision_, inputs[0], inputs[1], inputs[2], outputs[0], p->per_channel_quant);
    const Dim4 wd = inputs[1]->getDim();
    // [Cout][1][Kh][Kw], or [1][Kh][Kw][Cout] for ANDROID_NN (CLDepthwiseConvolution.cpp:126-143).
    d.kh = p->androidNN ? wd.c : wd.h;
    d.kw = p->androidNN ? wd.h : wd.w;
    d.weight_layout = p->androidNN ? ENN_B200_W_OHWI : ENN_B200_W_OIHW;
    d.stride_h = p->stride.h; d.stride_w = p->stride.w;
    d.dil_h = p->dilation.h; d.dil_w = p->dilation.w;
    d.pad_t = p->padding.t; d.pad_r = p->padding.r; d.pad_b = p->padding.b; d.pad_l = p->padding.l;
    d.groups = p->depth_multiplier;
    d.activation = act_code(*p->activation_info);
    Status s = ensure_nhwc_staging(nchw);
    if (s != Status::SUCCESS) return s;
    return prepare_conv_like(1, d, inputs[1], inputs[2], p->scales);
}

Status B200Deconvolution::initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                                     std::shared_ptr<Parameters> parameters) {
    auto p = std::dynamic_pointer_cast<DeconvolutionParameters>(parameters);
    if (!p || inputs.size() < 3 || outputs.empty()) return Status::INVALID_PARAMS;
    inputs_ = inputs; outputs_ = outputs;
    const bool nchw = p->isNCHW;
    in_dim_ = logical_dim(inputs[0], nchw);
    out_dim_ = logical_dim(outputs[0], nchw);
    enn_b200_conv_desc d;
    fill_common(&d, in_dim_, out_dim_, precision_, inputs[0], inputs[1], inputs[2], outputs[0], p->per_channel_quant);
    const Dim4 wd = inputs[1]->getDim();
    // Caffe layout [Cin][Cout][Kh][Kw]; ANDROID_NN [Cout][Kh][Kw][Cin] (CLDeconvolutionQuantized.cpp:39-46).
    d.kh = p->androidNN ? wd.c : wd.h;
    d.kw = p->androidNN ? wd.h : wd.w;
    d.weight_layout = p->androidNN ? ENN_B200_W_OHWI : ENN_B200_W_IOHW;
    d.stride_h = p->stride.h; d.stride_w = p->stride.w;
    d.pad_t = p->padding.t; d.pad_r = p->padding.r; d.pad_b = p->padding.b; d.pad_l = p->padding.l;
    d.groups = p->group_size;
    d.weights_as_input = p->weights_as_input;
    d.activation = act_code(*p->activation_info);
    Status s = ensure_nhwc_staging(nchw);
    if (s != Status::SUCCESS) return s;
    return prepare_conv_like(2, d, inputs[1], inputs[2], p->scales);
}

Status B200FullyConnected::initialize(const std::vector<std::shared_ptr<ITensor>> &input_tensors,
                                      const std::vector<std::shared_ptr<ITensor>> &output_tensors, const std::shared_ptr<Parameters> parameters) {
    auto p = std::dynamic_pointer_cast<FullyConnectedParameters>(parameters);
    if (!p || input_tensors.size() < 3 || output_tensors.empty()) return Status::INVALID_PARAMS;
    inputs_ = input_tensors; outputs_ = output_tensors;
    const Dim4 id = input_tensors[0]->getDim(), wd = input_tensors[1]->getDim();
    enn_b200_fc_desc d;
    std::memset(&d, 0, sizeof(d));
    // weights are [Nout][K]; the input is flattened to [batch][K] (CLFullyConnected.cpp:46-57)
    d.n = wd.n;
    d.k = wd.c * wd.h * wd.w;
    d.m = static_cast<int32_t>((static_cast<int64_t>(id.n) * id.c * id.h * id.w) / d.k);
    d.activation = act_code(*p->activation_info);
    d.act_dtype = precision_ == PrecisionType::INT8 ? ENN_B200_S8 : ENN_B200_U8;
    d.weight_dtype = input_tensors[1]->getDataType() == DataType::INT8 ? ENN_B200_S8 : ENN_B200_U8;
    d.per_channel = 0;
    d.in_scale = input_tensors[0]->getScale(); d.in_zp = input_tensors[0]->getZeroPoint();
    d.w_scale = input_tensors[1]->getScale(); d.w_zp = input_tensors[1]->getZeroPoint();
    d.bias_scale = input_tensors[2]->getScale();
    d.out_scale = output_tensors[0]->getScale(); d.out_zp = output_tensors[0]->getZeroPoint();
    runtime_weights_ = !input_tensors[1]->is_const();     // CLFullyConnected.cpp:36
    runtime_bias_ = !input_tensors[2]->is_const();
    d.weights_as_input = runtime_weights_;
    d.bias_as_input = runtime_bias_;
    std::vector<uint8_t> wt, bt;
    const void *w = runtime_weights_ ? nullptr : host_bytes(input_tensors[1], &wt);
    const int32_t *b = runtime_bias_ ? nullptr : static_cast<const int32_t *>(host_bytes(input_tensors[2], &bt));
    return to_status(enn_b200_fc_prepare(runtime_->context(), &d, w, b, nullptr, &op_));
}

Status B200Add::initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                           std::shared_ptr<Parameters> parameters) {
    auto p = std::dynamic_pointer_cast<AddParameters>(parameters);
    if (!p || inputs.size() < 2 || outputs.empty()) return Status::INVALID_PARAMS;
    inputs_ = inputs; outputs_ = outputs;
    two_inputs_ = true;
    enn_b200_add_desc d;
    std::memset(&d, 0, sizeof(d));
    d.count = static_cast<int64_t>(outputs[0]->getNumOfBytes());
    d.activation = act_code(p->activation_info);
    d.act_dtype = precision_ == PrecisionType::INT8 ? ENN_B200_S8 : ENN_B200_U8;
    d.in0_scale = inputs[0]->getScale(); d.in0_zp = inputs[0]->getZeroPoint();
    d.in1_scale = inputs[1]->getScale(); d.in1_zp = inputs[1]->getZeroPoint();
    d.out_scale = outputs[0]->getScale(); d.out_zp = outputs[0]->getZeroPoint();
    return to_status(enn_b200_add_prepare(runtime_->context(), &d, &op_));
}

Status B200Averagepool::initialize(std::vector<std::shared_ptr<ITensor>> inputs, std::vector<std::shared_ptr<ITensor>> outputs,
                                   std::shared_ptr<Parameters> parameters) {
    auto p = std::dynamic_pointer_cast<Pool2DParameters>(parameters);
    if (!p || inputs.empty() || outputs.empty()) return Status::INVALID_PARAMS;
    inputs_ = inputs; outputs_ = outputs;
    const bool nchw = inputs[0]->getDataOrder() == DataOrder::NCHW;
    in_dim_ = logical_dim(inputs[0], nchw);
    out_dim_ = logical_dim(outputs[0], nchw);
    enn_b200_pool_desc d;
    std::memset(&d, 0, sizeof(d));
    d.n = in_dim_.n; d.h = in_dim_.h; d.w = in_dim_.w; d.c = in_dim_.c;
    d.kh = p->filter.h; d.kw = p->filter.w; d.stride_h = p->stride.h; d.stride_w = p->stride.w;
    d.pad_t = p->padding.t; d.pad_l = p->padding.l;
    d.out_h = out_dim_.h; d.out_w = out_dim_.w;
    d.activation = act_code(p->activation_info);
    d.act_dtype = precision_ == PrecisionType::INT8 ? ENN_B200_S8 : ENN_B200_U8;
    d.out_scale = outputs[0]->getScale(); d.out_zp = outputs[0]->getZeroPoint();
    Status s = ensure_nhwc_staging(nchw);
    if (s != Status::SUCCESS) return s;
    return to_status(enn_b200_avgpool_prepare(runtime_->context(), &d, &op_));
}

}  // namespace b200
}  // namespace ud
}  // namespace enn
