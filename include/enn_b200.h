/*
 * enn_b200.h - C ABI of the B200 (sm_100a) quantized-operator library that stands in for the
 * OpenCL operator path of the ENN GPU userdriver (reference project: src/userdriver/gpu).
 *
 * Every entry point is extern "C", takes plain pointers / sizes / POD descriptors, and returns an
 * int32_t status that mirrors the reference's `enum class Status`
 * (src/userdriver/common/operator_interfaces/common/Common.hpp:113-119).
 *
 * Lifecycle mirrors the reference operator interface
 *   initialize(inputs, outputs, parameters)  ->  enn_b200_<op>_prepare(ctx, desc, weights, bias, ..., &op)
 *   execute()                                ->  enn_b200_op_execute(op, in_dev, out_dev)   (enqueue only, no host sync)
 *   release()                                ->  enn_b200_op_release(op)
 * and the reference runtime shim (CLRuntime / CLTensor / CLBuffer) becomes
 *   enn_b200_context_create / _malloc / _upload / _download / _stream_sync.
 *
 * Activation tensors are NHWC, channel innermost.  All arithmetic is integer and reproduces the
 * reference's fixed-point requantisation bit for bit.
 */
#ifndef ENN_B200_H_
#define ENN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: same values as enn::ud::Status (Common.hpp:113-119); CL_FAILURE becomes CUDA_FAILURE. */
enum {
    ENN_B200_SUCCESS = 0,
    ENN_B200_FAILURE = 1,
    ENN_B200_CUDA_FAILURE = 2,
    ENN_B200_INVALID_PARAMS = 3
};

/* ActivationInfo::ActivationType (common/ActivationInfo.hpp:5-12); only the quantized clamps exist here. */
enum { ENN_B200_ACT_NONE = 0, ENN_B200_ACT_RELU = 1, ENN_B200_ACT_RELU1 = 2, ENN_B200_ACT_RELU6 = 3 };

/* Element types of activations / weights (PrecisionType::UINT8 / INT8, Common.hpp:96-104). */
enum { ENN_B200_U8 = 0, ENN_B200_S8 = 1 };

/* Weight memory layouts accepted at prepare time (they are re-packed once on the device):
 *   OIHW  [Cout][Cin/g][Kh][Kw]   reference NCHW models (CLConvolution.cpp:97-98)
 *   OHWI  [Cout][Kh][Kw][Cin/g]   ANDROID_NN models (CLGEMMConvolutionQuantized.cpp:59-72)
 *   IOHW  [Cin][Cout/g][Kh][Kw]   Caffe deconvolution (CLDeconvolutionQuantized.cpp:39-46)
 * Depthwise: OIHW means [Cout][1][Kh][Kw], OHWI means [1][Kh][Kw][Cout]
 * (CLDepthwiseConvolution.cpp:126-143).  FullyConnected weights are [Nout][K] (OI) in both. */
enum { ENN_B200_W_OIHW = 0, ENN_B200_W_OHWI = 1, ENN_B200_W_IOHW = 2 };

/* Which kernel family an op handle was bound to (reported by enn_b200_op_info). */
enum {
    ENN_B200_IMPL_DIRECT = 0,    /* CUDA-core dp4a direct kernel (any geometry) */
    ENN_B200_IMPL_TCGEN05 = 1,   /* TMA + tcgen05.mma kind::i8 implicit GEMM */
    ENN_B200_IMPL_GEMV = 2,      /* HBM-bound small-M FullyConnected */
    ENN_B200_IMPL_DEPTHWISE = 3,
    ENN_B200_IMPL_ELTWISE = 4
};

typedef struct enn_b200_context enn_b200_context; /* one device + one in-order stream (CLRuntime's queue) */
typedef struct enn_b200_op enn_b200_op;           /* one prepared operator (CLConvolution etc.) */

/* Conv2D / DepthwiseConv2D / Deconvolution geometry + quantisation.
 * Fields are what ConvolutionParameters (CLConvolution.hpp:31-44), DepthwiseConvolutionParameters
 * (CLDepthwiseConvolution.hpp:18-29), DeconvolutionParameters (CLDeconvolution.hpp:20-31) and the
 * three CLTensors (scale, zero point, dims) carry into initialize(). */
typedef struct enn_b200_conv_desc {
    int32_t n, h, w, cin;           /* input NHWC */
    int32_t cout, kh, kw;           /* depthwise: cout = cin * depth_multiplier */
    int32_t stride_h, stride_w;
    int32_t dil_h, dil_w;           /* ignored by deconvolution */
    int32_t pad_t, pad_r, pad_b, pad_l;  /* Pad4 order (Common.hpp:152-154) */
    int32_t groups;                 /* conv/deconv group_size; depthwise: depth_multiplier */
    int32_t activation;             /* ENN_B200_ACT_* */
    int32_t act_dtype;              /* ENN_B200_U8 | ENN_B200_S8: type of input and output bytes */
    int32_t weight_dtype;           /* ENN_B200_U8 | ENN_B200_S8 */
    int32_t weight_layout;          /* ENN_B200_W_* */
    int32_t per_channel;            /* 1: per_channel_scales[cout] given, weight zero point is 0 */
    float in_scale;   int32_t in_zp;
    float w_scale;    int32_t w_zp;     /* per-tensor weights */
    float bias_scale;                    /* must equal in_scale*w_scale (KernelUtil.cpp:14-16) or multiplier is 0 */
    float out_scale;  int32_t out_zp;
    int32_t out_h, out_w;           /* 0 = derive; deconvolution may pass explicit output size */
    int32_t weights_as_input;       /* 1: the filter is a runtime tensor (CLConvolution.cpp:75 !weight->is_const()) */
    int32_t bias_as_input;          /* 1: the bias is a runtime tensor (CLConvolution.cpp:76, :496-501) */
} enn_b200_conv_desc;

/* FullyConnected: out[m][n] = requant(bias[n] + sum_k (a[m][k]-in_zp)(w[n][k]-w_zp)), the integer
 * contraction the reference computes for the same shape expressed as a 1x1 CONV_2D. */
typedef struct enn_b200_fc_desc {
    int32_t m, k, n;
    int32_t activation, act_dtype, weight_dtype, per_channel;
    float in_scale;   int32_t in_zp;
    float w_scale;    int32_t w_zp;
    float bias_scale;
    float out_scale;  int32_t out_zp;
    int32_t weights_as_input;       /* CLFullyConnected.cpp:36 */
    int32_t bias_as_input;
} enn_b200_fc_desc;

/* Quantized elementwise add (CLAddQuantized.cpp:70-165) and average pool (CLAveragepool.cpp:175-224). */
typedef struct enn_b200_add_desc {
    int64_t count;                  /* number of elements */
    int32_t activation, act_dtype;
    float in0_scale;  int32_t in0_zp;
    float in1_scale;  int32_t in1_zp;
    float out_scale;  int32_t out_zp;
} enn_b200_add_desc;

typedef struct enn_b200_pool_desc {
    int32_t n, h, w, c;
    int32_t kh, kw, stride_h, stride_w, pad_t, pad_l;
    int32_t out_h, out_w;
    int32_t activation, act_dtype;
    float out_scale;  int32_t out_zp;
} enn_b200_pool_desc;

/* Remaining quantized graph operators of the reference's u8 models.  Tensors are described by their memory order, so
 * the same descriptors serve NHWC and NCHW callers.
 * Mean (CLMean.cpp:72-297, MeanKernels.cpp): integer sum over the axes in axis_mask (bit i = dims[i]) divided by the
 * element count with C truncation; no rescaling (the reference assumes equal input and output quantisation). */
typedef struct enn_b200_mean_desc {
    int32_t dims[4];                /* in memory order, outermost first (NHWC: n, h, w, c) */
    int32_t axis_mask;
    int32_t act_dtype;
} enn_b200_mean_desc;

/* Concatenation (CLConcat.cpp:224-256, ConcatKernels.cpp:399-470): input i is viewed as [outer][inner[i]] and lands at
 * column offset sum(inner[0..i)) of the output [outer][sum inner]; an input whose scale differs from the output's is
 * requantised in float, round((x - zp_i) * s_i / s_o) + zp_o, one whose scale is equal is copied as it is. */
#define ENN_B200_CONCAT_MAX_INPUTS 8
typedef struct enn_b200_concat_desc {
    int32_t n_inputs;
    int32_t act_dtype;
    int64_t outer;
    int64_t inner[ENN_B200_CONCAT_MAX_INPUTS];
    float in_scale[ENN_B200_CONCAT_MAX_INPUTS];
    int32_t in_zp[ENN_B200_CONCAT_MAX_INPUTS];
    float out_scale;
    int32_t out_zp;
} enn_b200_concat_desc;

/* Softmax over `channels` of a tensor viewed as [outer][channels][inner] (CLSoftmax.cpp:81-150: dequantise, float
 * softmax_axis2 with beta, quantise with round(x / s_o + zp_o) and saturation). */
typedef struct enn_b200_softmax_desc {
    int64_t outer;
    int32_t channels;
    int64_t inner;
    float beta;
    int32_t act_dtype;
    float in_scale;   int32_t in_zp;
    float out_scale;  int32_t out_zp;
} enn_b200_softmax_desc;

/* Bilinear resize of NHWC bytes (CLResizeBilinear.cpp, ResizeBilinearKernels.cpp:41-83): float interpolation of the raw
 * bytes, truncated; no rescaling. */
typedef struct enn_b200_resize_desc {
    int32_t n, h, w, c;
    int32_t out_h, out_w;
    int32_t align_corners, half_pixel_centers;
    int32_t act_dtype;
} enn_b200_resize_desc;

/* Derived per-op facts, for callers that size buffers or report work. */
typedef struct enn_b200_op_info_t {
    int32_t impl;                   /* ENN_B200_IMPL_* */
    int32_t out_n, out_h, out_w, out_c;
    int64_t in_bytes, out_bytes;
    int64_t macs;                   /* multiply-accumulates of one execute */
    int64_t algorithmic_bytes;      /* input + weights + bias/params + output, each once */
    int32_t act_min, act_max;       /* clamp derived as KernelUtil.cpp:27-71 */
    int32_t kernel_launches;        /* kernels one execute enqueues */
} enn_b200_op_info_t;

/* ---- runtime shim: replaces CLRuntime / CLBuffer / CLTensor::readData,writeData
 *      (gpu/common/CLRuntime.cpp:34-157, CLTensor.hpp:39-331, CLComputeLibrary.cpp:15-186) ---- */
int32_t enn_b200_context_create(int32_t device, enn_b200_context **ctx);
int32_t enn_b200_context_destroy(enn_b200_context *ctx);
int32_t enn_b200_malloc(enn_b200_context *ctx, size_t bytes, void **dev_ptr);
int32_t enn_b200_free(enn_b200_context *ctx, void *dev_ptr);
/* Asynchronous on the context stream, like the reference's non-blocking writeData
 * (gpu_userdriver.cc set_input_data); host memory should be pinned for overlap. */
int32_t enn_b200_upload(enn_b200_context *ctx, void *dev_dst, const void *host_src, size_t bytes);
/* Copies device->host on the stream and blocks until done, like the blocking readData in set_output_data. */
int32_t enn_b200_download(enn_b200_context *ctx, void *host_dst, const void *dev_src, size_t bytes);
/* Device->device on the stream (CLRuntime::copyBuffer, as used by CLConvolution.cpp:151 for the bias). */
int32_t enn_b200_copy_device(enn_b200_context *ctx, void *dev_dst, const void *dev_src, size_t bytes);
int32_t enn_b200_stream_sync(enn_b200_context *ctx);            /* CLComputeLibrary::synchronize */
/* Device timer on the context's stream: start / stop enqueue an event each, elapsed_us waits for the stop event.  What
 * EnnUDOperator<T>::execute brackets every operator with (PROFILE_FROM / PROFILE_UNTIL, userdriver_operator.h:35-42),
 * in device time. */
typedef struct enn_b200_timer enn_b200_timer;
int32_t enn_b200_timer_create(enn_b200_context *ctx, enn_b200_timer **timer);
int32_t enn_b200_timer_start(enn_b200_timer *timer);
int32_t enn_b200_timer_stop(enn_b200_timer *timer);
int32_t enn_b200_timer_elapsed_us(enn_b200_timer *timer, float *microseconds);
int32_t enn_b200_timer_destroy(enn_b200_timer *timer);
int32_t enn_b200_host_alloc(size_t bytes, void **host_ptr);      /* pinned host staging */
int32_t enn_b200_host_free(void *host_ptr);
/* Last error text of this context (empty string if none); never fails. */
int32_t enn_b200_last_error(enn_b200_context *ctx, char *buf, size_t buf_len);
/* cudaStream_t of the context, as void*, so a caller can order its own work against it. */
void *enn_b200_stream(enn_b200_context *ctx);
/* Planner overrides for tests and tuning, read when an operator is prepared (the library reads no environment
 * variable).  Names: no_pdl, no_relu_mode, no_relu_hi, no_relu_sat, no_wide_store, no_grouped_tc, no_first_layer, no_implicit, no_gemv, no_narrow_span, no_pack,
 * pack_wide, no_bres, no_bres_k1, no_fan_out, tc_bn (>= 96), tc_pair, tc_raster, epi_g, dw_legacy, dw_rows, no_fuse, fuse_all, no_out_stream, no_narrow_n.
 * grid_cap = G: operators prepared afterwards launch at most G CTAs of their persistent kernels (tensor-core GEMM /
 * convolution, row-ring depthwise), i.e. occupy at most G SMs.  Meant for several contexts that share one GPU, each
 * running its own operator list: with G = SMs / 4 their kernels run side by side in four shares instead of taking
 * the whole GPU in turn, which hides the latency of the small layers (MobileNetV2-u8, 256 images: 1.25 ms per step
 * with eight lists of 37 SMs against 1.43 ms with three uncapped lists; 32 images: 0.22 against 0.34 ms).
 * Stands where the reference reads its build-time device switches (CLRuntime.cpp:174-213).  Unknown names are
 * rejected with INVALID_PARAMS; none of them changes a result. */
int32_t enn_b200_context_set_option(enn_b200_context *ctx, const char *name, int32_t value);

/* ---- operators.  *_prepare uploads + re-packs constant tensors once (the reference does this in
 *      initialize(): alignQuantizedWeightGEMM, align_weight_direct, matrixTrans ...) and derives the
 *      requantisation parameters the reference recomputes on every execute.  Host pointers are not
 *      retained (gpu_op_constructor.cc:2130-2147). ---- */

/* CLConvolution::initialize (CLConvolution.cpp:34-456) -> per-tensor CLGEMMConvolutionQuantized /
 * CLQuantizedDirectConvolution / CLGEMM1xXConvolutionQuantized or CLConvolutionPerChannelQuantized. */
int32_t enn_b200_conv2d_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *desc, const void *weights_host,
                                const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op);
/* CLDepthwiseConvolution::initialize (CLDepthwiseConvolution.cpp:88-215). */
int32_t enn_b200_depthwise_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *desc, const void *weights_host,
                                   const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op);
/* CLDeconvolution::initialize (CLDeconvolution.cpp:36-215). */
int32_t enn_b200_deconv_prepare(enn_b200_context *ctx, const enn_b200_conv_desc *desc, const void *weights_host,
                                const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op);
/* CLFullyConnected::initialize (CLFullyConnected.cpp:22-102). */
int32_t enn_b200_fc_prepare(enn_b200_context *ctx, const enn_b200_fc_desc *desc, const void *weights_host,
                            const int32_t *bias_host, const float *per_channel_scales, enn_b200_op **op);
/* CLAdd::initialize -> CLAddQuantized (CLAddQuantized.cpp:20-68). */
int32_t enn_b200_add_prepare(enn_b200_context *ctx, const enn_b200_add_desc *desc, enn_b200_op **op);
/* CLAveragepool::initialize (CLAveragepool.cpp). */
int32_t enn_b200_avgpool_prepare(enn_b200_context *ctx, const enn_b200_pool_desc *desc, enn_b200_op **op);

/* CLMaxpool::initialize (CLMaxpool.cpp:21-118; kernel MaxpoolKernels.cpp:33-58: window clipped to the image, clamp). */
int32_t enn_b200_maxpool_prepare(enn_b200_context *ctx, const enn_b200_pool_desc *desc, enn_b200_op **op);
/* CLMean::initialize (CLMean.cpp:30-107). */
int32_t enn_b200_mean_prepare(enn_b200_context *ctx, const enn_b200_mean_desc *desc, enn_b200_op **op);
/* CLConcat::initialize (CLConcat.cpp:126-205); executed with enn_b200_op_execute_n. */
int32_t enn_b200_concat_prepare(enn_b200_context *ctx, const enn_b200_concat_desc *desc, enn_b200_op **op);
/* CLSoftmax::initialize (CLSoftmax.cpp:28-121). */
int32_t enn_b200_softmax_prepare(enn_b200_context *ctx, const enn_b200_softmax_desc *desc, enn_b200_op **op);
/* CLResizeBilinear::initialize (CLResizeBilinear.cpp:120-218). */
int32_t enn_b200_resize_bilinear_prepare(enn_b200_context *ctx, const enn_b200_resize_desc *desc, enn_b200_op **op);

/* Force the kernel family of a prepared conv / fc / deconv handle (ENN_B200_IMPL_DIRECT or
 * ENN_B200_IMPL_TCGEN05 ...); INVALID_PARAMS if that family cannot run the geometry.  For tests and benches. */
int32_t enn_b200_op_set_impl(enn_b200_op *op, int32_t impl);

/* EnnUDOperator<T>::execute -> op_->execute() (userdriver_operator.h:32-44): enqueue on the context
 * stream, no host synchronisation.  Device pointers are read at call time because the reference only
 * assigns pooled activation buffers after every initialize() has run (gpu_op_constructor.cc:1839-1843). */
int32_t enn_b200_op_execute(enn_b200_op *op, const void *in_dev, void *out_dev);
/* Two-input form for the quantized add (inputs = {a, b}). */
int32_t enn_b200_op_execute2(enn_b200_op *op, const void *in0_dev, const void *in1_dev, void *out_dev);
/* n-input form (concatenation; also accepts the one- and two-input operators). */
int32_t enn_b200_op_execute_n(enn_b200_op *op, const void *const *ins_dev, int32_t n_in, void *out_dev);
/* Fuses a quantized add into the epilogue of the convolution that produces one of its inputs (the MobileNetV2
 * residual pattern: CONV_2D -> ADD, `CLAddQuantized.cpp:70-165` applied to every output byte before it is stored).
 * `add` is a prepared add over exactly the convolution's output; on success the convolution owns it, takes two inputs
 * (enn_b200_op_execute2 / _n: in0 feeds the convolution, in1 is the add's other input, same layout as the output) and
 * writes the add's result.  INVALID_PARAMS, with both operators unchanged, when the convolution's plan cannot take it
 * (not on the tensor-core path, ReLU-merged epilogue, output rows not multiples of 16 bytes, no shared memory left for
 * the add's tables); the caller then runs the two operators one after the other.  Results are those of the two
 * operators run separately, bit for bit. */
int32_t enn_b200_op_fuse_add(enn_b200_op *conv, enn_b200_op *add, int32_t conv_is_second_input);
/* Operators prepared with weights_as_input / bias_as_input take those tensors at run time.  The reference re-runs
 * its weight conversion and bias copy inside every execute() of such an operator
 * (CLGEMMConvolutionQuantized.cpp:142-160, CLConvolution.cpp:496-501); here the caller states when the tensors have
 * changed: rebind reads the flagged tensor(s) from device memory in the layout the descriptor names (the other one,
 * if constant, is the copy kept from prepare), re-derives every packed constant of the operator in place and returns
 * when they are on the device.  execute() of such an operator fails with FAILURE until the first rebind.  A pointer
 * whose tensor is not flagged is ignored (may be NULL).  Such operators cannot be added to an operator list, whose
 * captured launch sequence holds the constants' addresses. */
int32_t enn_b200_op_rebind_constants(enn_b200_op *op, const void *weights_dev, const int32_t *bias_dev);
/* No counterpart in the reference.  Runs a prepared Conv2D / Deconvolution whose input is gathered into a scratch
 * matrix without allocating anything: the matrix goes into a 32 MiB device array that is part of the library image.
 * For callers that may not call cudaMalloc at run time.  Limits: the operator must be on the tensor-core path and
 * need between 1 byte and 32 MiB of scratch (INVALID_PARAMS otherwise); calls that overlap on one GPU race on the
 * shared array; the first call per device does a one-time address lookup and should precede any stream capture. */
int32_t enn_b200_op_execute_noalloc(enn_b200_op *op, const void *in_dev, void *out_dev);
int32_t enn_b200_op_info(const enn_b200_op *op, enn_b200_op_info_t *info);
/* Failure handling (Common.hpp:113-119 CL_FAILURE; the reference has no device-side waits to bound).  A kernel whose
 * bounded barrier wait ran out leaves a code in host-visible memory and every later execute of that operator returns
 * CUDA_FAILURE until enn_b200_op_clear_error.  enn_b200_op_test_starve_next arms a self-test of exactly that path for
 * a tensor-core operator: its next execute issues no operand copy and uses a wait limit of under a millisecond, so the
 * kernel gives up with nothing in flight, releases its tensor memory and returns; outputs of that execute are
 * undefined. */
int32_t enn_b200_op_test_starve_next(enn_b200_op *op);
int32_t enn_b200_op_clear_error(enn_b200_op *op);
int32_t enn_b200_op_release(enn_b200_op *op);

/* ---- operator list: GpuUserDriver::OpenSubGraph / ExecuteSubGraph / CloseSubGraph (gpu_userdriver.cc) and
 *      OperationExecutor::execute (gpu_op_executor.cc).  Tensors are numbered like BufferTable indices. ---- */
typedef struct enn_b200_oplist enn_b200_oplist;
int32_t enn_b200_oplist_create(enn_b200_context *ctx, enn_b200_oplist **list);
int32_t enn_b200_oplist_add_tensor(enn_b200_oplist *list, int64_t bytes, int32_t *tensor_id);
/* Appends a prepared operator reading tensors in_ids[0..n_in) and writing out_id; the list owns the op from here on. */
int32_t enn_b200_oplist_add_op(enn_b200_oplist *list, enn_b200_op *op, const int32_t *in_ids, int32_t n_in, int32_t out_id);
int32_t enn_b200_oplist_set_io(enn_b200_oplist *list, const int32_t *input_ids, int32_t n_inputs, const int32_t *output_ids,
                               int32_t n_outputs);
/* assignBuffers (gpu_op_constructor.cc:1839-1843, CLRuntime.cpp:34-157): liveness-based device buffer assignment,
 * then one eager pass and capture of the operator sequence into a CUDA graph. */
int32_t enn_b200_oplist_finalize(enn_b200_oplist *list);
/* ExecuteSubGraph: host_inputs[i] / host_outputs[i] follow the order given to set_io; copies in, runs, copies out, blocks. */
int32_t enn_b200_oplist_execute(enn_b200_oplist *list, const void *const *host_inputs, void *const *host_outputs);
/* Pipelined ExecuteSubGraph (the async H2D / D2H overlap the reference's set_input_data / set_output_data do not have):
 * queues copy-in, graph and copy-out and returns; the copy-in of one submission overlaps the operators of the previous
 * one.  Outputs are valid after enn_b200_oplist_wait.  Host buffers must stay untouched until then (pin them). */
int32_t enn_b200_oplist_submit(enn_b200_oplist *list, const void *const *host_inputs, void *const *host_outputs);
/* One pipelined submission on each of `n` lists of one device (each in its own context, normally prepared with option
 * grid_cap = SMs / n) whose operators start together: all inputs are copied first and every list's graph waits for all
 * of them.  Lists that share a GPU run fastest when they execute the same layer at the same time (kernels of one kind
 * fill every SM; a mix of kinds leaves SMs that hold a small CTA closed to a large one): MobileNetV2-u8, 256 images per
 * list, four lists of 37 SMs: 1.33 ms per step in rounds against 2.1 ms when each list starts as its own input lands.
 * host_inputs[k] / host_outputs[k] are the buffer tables of lists[k]; results are valid after enn_b200_oplist_wait on
 * each list.  The reference has one command queue per device and no counterpart (CLRuntime.cpp:214-247). */
int32_t enn_b200_oplist_submit_round(enn_b200_oplist *const *lists, int32_t n, const void *const *const *host_inputs,
                                     void *const *const *host_outputs);
int32_t enn_b200_oplist_wait(enn_b200_oplist *list);
/* Operators only, on device-resident tensors, asynchronous on the context stream. */
int32_t enn_b200_oplist_execute_device(enn_b200_oplist *list);
int32_t enn_b200_oplist_tensor_ptr(enn_b200_oplist *list, int32_t tensor_id, void **dev_ptr);
/* The list's nodes after finalize (a fused CONV_2D -> ADD pair is one node): count, and per node the operator's info,
 * its kind (0 conv, 1 depthwise, 2 deconvolution, 3 fully connected, 4 add, 5 average pool, 6 max pool, 7 mean,
 * 8 concat, 9 softmax, 10 resize) and its number of inputs. */
int32_t enn_b200_oplist_node_count(const enn_b200_oplist *list, int32_t *n_nodes);
int32_t enn_b200_oplist_node_info(const enn_b200_oplist *list, int32_t index, enn_b200_op_info_t *info, int32_t *kind, int32_t *n_inputs);
/* Per-operator device time in microseconds (average over `repeats` eager passes over the list's own tensors, one
 * event between consecutive nodes): the per-operator bracket of userdriver_operator.h:35-42 for a whole list. */
int32_t enn_b200_oplist_profile(enn_b200_oplist *list, int32_t repeats, float *node_us, int32_t capacity);
/* Device address of graph output `output_index` as written by the latest enn_b200_oplist_submit (submissions alternate
 * between two device copies of every graph input / output), for callers that pass results on device-side
 * (CLTensor::getDataPtr on an output tensor). */
int32_t enn_b200_oplist_last_output_ptr(enn_b200_oplist *list, int32_t output_index, void **dev_ptr);
int32_t enn_b200_oplist_stats(enn_b200_oplist *list, int64_t *device_bytes, int32_t *n_buffers, int32_t *kernel_launches);
/* CloseSubGraph: releases the operators, the buffers and the graph. */
int32_t enn_b200_oplist_destroy(enn_b200_oplist *list);

/* ---- operator-list group: one ExecuteSubGraph call (gpu_userdriver.cc, whole batch per call) spread over several
 *      devices.  Every member is a finalized list built for its slice of the batch, on its own context (one per device,
 *      or several per device).  A call splits each graph input along its outermost dimension into contiguous slices in
 *      member order (member i takes as many bytes as its own input tensor holds), runs the members side by side with one
 *      host worker thread each, and writes each member's outputs at the matching offsets of host_outputs.  No collective
 *      is involved: the slices are independent and only the results meet again, in host memory.  submit / wait are the
 *      pipelined forms (enn_b200_oplist_submit / _wait on every member).  destroy_lists != 0 also destroys the lists. ---- */
typedef struct enn_b200_group enn_b200_group;
int32_t enn_b200_group_create(enn_b200_oplist *const *lists, int32_t n_lists, enn_b200_group **group);
int32_t enn_b200_group_execute(enn_b200_group *group, const void *const *host_inputs, void *const *host_outputs);
int32_t enn_b200_group_submit(enn_b200_group *group, const void *const *host_inputs, void *const *host_outputs);
int32_t enn_b200_group_wait(enn_b200_group *group);
int32_t enn_b200_group_last_error(enn_b200_group *group, char *buf, size_t buf_len);
int32_t enn_b200_group_destroy(enn_b200_group *group, int32_t destroy_lists);

/* ---- NNC model front end: the model-to-operators half of GpuUserDriver::OpenSubGraph (OperationConstructor::open_oplist
 *      and create_ud_operator<...>, gpu_op_constructor.cc:63-383, 789-863, 1797-2046) over the NNC v2 flatbuffer
 *      (src/model/schema/nnc/v2/schema.fbs).  Parses the first subgraph, derives padding / precision / per-channel
 *      information with the reference's rules, prepares every operator and finalizes an operator list.  `batch` > 0
 *      replaces the outermost dimension of every activation tensor.  Models whose activations are NHWC in memory only
 *      (TENSORFLOW_NHWC, CAFFE_NHWC, ANDROID_NN without use_nchw); UINT8 / INT8 tensors only. ---- */
typedef struct enn_b200_model enn_b200_model;
int32_t enn_b200_model_open(enn_b200_context *ctx, const void *nnc_bytes, size_t nbytes, int32_t batch, enn_b200_model **model);
int32_t enn_b200_model_info(enn_b200_model *model, int32_t *n_inputs, int32_t *n_outputs, int32_t *n_operators);
int32_t enn_b200_model_io_bytes(enn_b200_model *model, int32_t is_output, int32_t index, int64_t *bytes);
/* The model's operator list (owned by the model), for the pipelined / device-resident calls. */
int32_t enn_b200_model_oplist(enn_b200_model *model, enn_b200_oplist **list);
/* ExecuteSubGraph on the model: host buffers in graph input / output order. */
int32_t enn_b200_model_execute(enn_b200_model *model, const void *const *host_inputs, void *const *host_outputs);
int32_t enn_b200_model_close(enn_b200_model *model);

/* Layout converters for NCHW models (CLRuntime.cpp:1477-1620 NHWC2NCHW_* / NCHW2NHWC_*), 1-byte elements. */
int32_t enn_b200_nchw_to_nhwc(enn_b200_context *ctx, const void *src_dev, void *dst_dev, int32_t n, int32_t c,
                              int32_t h, int32_t w);
int32_t enn_b200_nhwc_to_nchw(enn_b200_context *ctx, const void *src_dev, void *dst_dev, int32_t n, int32_t c,
                              int32_t h, int32_t w);

/* Host-side quantisation helpers (cl_quantized_utils/QuantizationUtil.cpp:8-35, KernelUtil.cpp:7-71),
 * exported so a caller can inspect what prepare derived. */
void enn_b200_quantize_multiplier(double real_multiplier, int32_t *quantized_multiplier, int32_t *shift);
int32_t enn_b200_conv_multiplier(double in_scale, double w_scale, double bias_scale, double out_scale,
                                 double *multiplier);
void enn_b200_activation_range(int32_t activation, int32_t act_dtype, float scale, int32_t zero_point,
                               int32_t *act_min, int32_t *act_max);

/* The kernels' requantisation tail evaluated on the host with the same inline code the device uses
 * (CLKernels.hpp:121-168: left shift, SaturatingRoundingDoublingHighMul, RoundingDivideByPOT, + zero point, clamp). */
int32_t enn_b200_requant_host(int32_t acc, int32_t multiplier, int32_t shift, int32_t out_zp, int32_t act_min,
                              int32_t act_max);

/* Measures the sustained tcgen05.mma rate of the device (no reference counterpart: it provides the measured
 * tensor-pipe ceiling that GEMM-shaped operators are reported against).  kind 0: kind::i8 (u8 x s8 -> s32),
 * kind 1: kind::f16 with bf16 operands; kinds 2 and 3: the same on pseudo-random operand bytes.  n: MMA N (16..256, multiple of 16); iters: MMA groups of 4 per SM.
 * Writes tera-operations (2 x MAC) per second summed over all SMs. */
int32_t enn_b200_measure_mma_peak(enn_b200_context *ctx, int32_t kind, int32_t n, int32_t iters, double *tera_ops);

/* Library identification: returns a static string naming the build (arch, version). */
const char *enn_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ENN_B200_H_ */
