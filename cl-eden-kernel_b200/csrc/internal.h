// Internal structures shared by the C-ABI translation units.  Not part of the public interface.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/enn_b200.h"

struct enn_b200_context {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    std::string last_error;
    void *encode_tiled = nullptr;   // cuTensorMapEncodeTiled, resolved through the runtime
    // Side streams for operators made of independent launches (the parity classes of a transposed convolution): forked
    // from and joined back into `stream` with events, created on first use.
    static constexpr int kAuxStreams = 8;
    cudaStream_t aux_streams[kAuxStreams] = {};
    cudaEvent_t ev_fork = nullptr, ev_join[kAuxStreams] = {};
    bool aux_ready = false;
    // Planner overrides set with enn_b200_context_set_option (tests and tuning).  They are read when an operator is
    // prepared, never on the execute path, and never from the environment.
    std::map<std::string, int> options;
    bool has_opt(const char *name) const { return options.find(name) != options.end(); }
    int opt(const char *name, int dflt = 0) const {
        auto it = options.find(name);
        return it == options.end() ? dflt : it->second;
    }
    // SMs one launch of a persistent kernel may occupy: option grid_cap (several operator lists that share the GPU each
    // take a share of it, so that their kernels run side by side instead of one after another), else all of them.
    int launch_sms() const {
        const int cap = opt("grid_cap");
        return cap > 0 && cap < sm_count ? cap : sm_count;
    }
};

namespace enn_b200 {

enum OpKind { OP_CONV = 0, OP_DEPTHWISE = 1, OP_DECONV = 2, OP_FC = 3, OP_ADD = 4, OP_AVGPOOL = 5, OP_MAXPOOL = 6, OP_MEAN = 7, OP_CONCAT = 8, OP_SOFTMAX = 9, OP_RESIZE = 10 };

// Geometry + quantisation handed to kernels by value.
struct ConvGeom {
    int32_t n, h, w, cin;
    int32_t cout, kh, kw;
    int32_t sh, sw, dh, dw;
    int32_t pt, pl;
    int32_t oh, ow;
    int32_t groups, cin_g, cout_g;   // depthwise: groups = depth multiplier
    int32_t in_zp, w_zp, out_zp;
    int32_t act_min, act_max;
    int32_t a_signed, w_signed;
};

struct Requant {
    const int32_t *mult;    // [cout] Q0.31 multipliers
    const int32_t *shift;   // [cout] signed exponents (>0 left, <=0 right)
    const int32_t *bias;    // [cout]
};

struct AddParams {
    int32_t in0_off, in1_off, out_off;
    int32_t m0, s0, m1, s1, mo, so;   // multipliers and (non-positive) shifts
    int32_t act_min, act_max;
    int32_t is_signed;
    // Stage-1 values of both inputs by input byte (device array of 2 x 256 words: in0 table, in1 table), so that the
    // vector kernel spends its instructions on the last stage only.  Built at prepare time with the same functions.
    const int32_t *lut;
    // The whole operator as one table: output byte for every pair of input bytes, at index
    // add_lut2_index(a, b) (65536 bytes, built from the same three stages at prepare time).  Large tensors use it
    // from shared memory: a lookup replaces the 64-bit multiply and both rounding shifts of the last stage.
    const uint8_t *lut2;
};

// Position of pair (a, b) in the 64 KB table: row a, column b with the low bits of a folded into the word index, so
// that lanes whose b bytes agree (flat image regions) still spread over the shared-memory banks.
__host__ __device__ inline uint32_t add_lut2_index(uint32_t a, uint32_t b) {
    const uint32_t idx = (a << 8) | b;
    return idx ^ ((idx >> 6) & 0x7cu);
}

struct PoolGeom {
    int32_t n, h, w, c, kh, kw, sh, sw, pt, pl, oh, ow;
    int32_t act_min, act_max, is_signed;
};

}  // namespace enn_b200

// Operators whose filter and / or bias are runtime tensors: what prepare needs again at every rebind.
struct RuntimeConstants {
    bool weights = false, bias = false, bound = false;
    enn_b200_conv_desc desc{};         // flags cleared
    int prepare_kind = 0;              // OP_CONV / OP_DEPTHWISE / OP_DECONV handed to the prepare routine
    std::vector<float> scales;
    std::vector<uint8_t> w_host;       // caller's layout
    std::vector<int32_t> b_host;
};

struct enn_b200_op {
    enn_b200_context *ctx = nullptr;
    int kind = 0;
    int impl = 0;
    enn_b200::ConvGeom g{};
    enn_b200::Requant rq{};
    enn_b200::AddParams add{};
    enn_b200::PoolGeom pool{};
    int64_t count = 0;                 // add: element count
    void *w_direct = nullptr;          // weights in the direct kernels' layout
    std::vector<void *> owned;         // device allocations released with the op
    enn_b200_op_info_t info{};
    void *dw_chan = nullptr;           // depthwise 3x3 fast path: per-channel constants (in `owned`)
    bool dw_relu = false;              // dw_chan holds the merged ReLU form {C low, C high, M0, e - 1}
    void *dw_w = nullptr;              // depthwise 3x3 fast path: packed 3-tap weight words (in `owned`)
    void *dw_ring = nullptr;           // depthwise row-ring plan (depthwise.cu), owned
    void *tc = nullptr;                // tensor-core plan (gemm_tc.cu), owned
    void *graph_state = nullptr;       // state of Mean / Concat / Softmax / Resize (graph_ops.cu), owned
    std::unique_ptr<RuntimeConstants> dyn;   // set when the descriptor said weights_as_input / bias_as_input
    enn_b200_op *fused_add = nullptr;  // convolution + quantized add: the add operator whose table the epilogue uses (owned)
};

namespace enn_b200 {

bool pdl_enabled();     // abi.cu: false once option no_pdl has been set on any context

// kernels_direct.cu
cudaError_t launch_conv_direct(const ConvGeom &g, const Requant &rq, const void *in, const void *w, void *out,
                               cudaStream_t s);
cudaError_t launch_deconv_direct(const ConvGeom &g, const Requant &rq, const void *in, const void *w, void *out,
                                 cudaStream_t s);
cudaError_t launch_depthwise(const ConvGeom &g, const Requant &rq, const void *in, const void *w, void *out,
                             int sm_count, cudaStream_t s);
bool dw3x3_eligible(const ConvGeom &g);
cudaError_t launch_dw3x3(const ConvGeom &g, const void *chan, bool relu_form, const void *w_packed, const void *in, void *out,
                         int sm_count, cudaStream_t s);
bool dw_ring_plan(enn_b200_op *op);
cudaError_t dw_ring_launch(enn_b200_op *op, const void *in, void *out);
void dw_ring_release(enn_b200_op *op);
void dw_ring_clear_error(enn_b200_op *op);
cudaError_t add_kernel_init();
cudaError_t launch_add(const AddParams &p, int64_t count, const void *a, const void *b, void *out, int sm_count,
                       cudaStream_t s);
cudaError_t launch_avgpool(const PoolGeom &p, const void *in, void *out, cudaStream_t s);
cudaError_t launch_maxpool(const PoolGeom &p, const void *in, void *out, cudaStream_t s);
cudaError_t launch_graph_op(enn_b200_op *op, const void *const *ins, int n_in, void *out);     // Mean, Concat, Softmax, Resize
void graph_op_release(enn_b200_op *op);
cudaError_t launch_transpose_nchw_nhwc(const void *src, void *dst, int n, int c, int h, int w, bool to_nhwc,
                                       cudaStream_t s);


// ---- programmatic dependent launch ------------------------------------------------------------------------
// Kernels launched with launch_pdl may start (block scheduling, their own set-up code) while the kernel before them in
// the stream is still draining; they call pdl_wait() before they read or write any tensor, which blocks until that
// kernel has completed and its writes are visible, and pdl_trigger() to let their own successor start early.  A kernel
// that is launched the ordinary way keeps the ordinary stream order, whatever its neighbours do.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

}  // namespace enn_b200
