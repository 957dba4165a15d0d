// Operator-list executor: the part of GpuUserDriver that sits directly around the operators
// (gpu_userdriver.cc OpenSubGraph / ExecuteSubGraph / CloseSubGraph, OperationExecutor::execute).
//
//   OpenSubGraph   -> enn_b200_oplist_create + add_tensor/add_op + finalize
//                     (finalize = CLRuntime::assignBufferPool: inter-operator buffers are assigned after all
//                      operators are prepared, with liveness-based reuse, CLRuntime.cpp:34-157)
//   ExecuteSubGraph-> enn_b200_oplist_execute: async H2D of every graph input from the caller's host
//                     buffers (set_input_data), all operators in order, blocking D2H of every output
//                     (set_output_data)
//   CloseSubGraph  -> enn_b200_oplist_destroy
//
// The operator sequence is captured once into a CUDA graph, so an inference is one graph launch instead of
// one enqueue per operator.
#include <algorithm>
#include <cstdio>
#include <new>

#include "internal.h"

struct enn_b200_oplist {
    enn_b200_context *ctx = nullptr;
    struct Tensor {
        int64_t bytes = 0;
        void *dev = nullptr;
        void *dev_alt = nullptr;       // second copy of a graph input / output, for pipelined submission
        int first_def = -1, last_use = -1;
        bool is_input = false, is_output = false;
        int pool_slot = -1;
    };
    struct Node {
        enn_b200_op *op = nullptr;
        std::vector<int> ins;
        int out = -1;
    };
    std::vector<Tensor> tensors;
    std::vector<Node> nodes;
    std::vector<int> inputs, outputs;
    std::vector<void *> pool;          // device allocations backing the tensors
    std::vector<int64_t> pool_bytes;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    // Pipelined submission (enn_b200_oplist_submit): a second graph bound to the alternate input / output buffers,
    // a copy stream for the host-to-device transfers, and events that hand the two buffer sets back and forth.
    cudaGraph_t graph_alt = nullptr;
    cudaGraphExec_t exec_alt = nullptr;
    cudaStream_t copy_stream = nullptr;
    cudaStream_t out_stream = nullptr;      // device-to-host copies of the results: the operators' stream never waits for a copy engine
    cudaEvent_t ev_in_ready[2] = {nullptr, nullptr}, ev_slot_free[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr};
    bool slot_used[2] = {false, false};
    uint64_t seq = 0;
    bool finalized = false;
    int64_t device_bytes = 0;
    int32_t kernel_launches = 0;
};

namespace {
constexpr int64_t kFuseAddMaxCount = 1 << 21;
int32_t lfail(enn_b200_oplist *l, int32_t st, const char *msg) {
    if (l && l->ctx) l->ctx->last_error = msg;
    return st;
}
int32_t run_nodes(enn_b200_oplist *l, int slot = 0) {
    auto ptr = [&](int t) {
        auto &T = l->tensors[t];
        return (slot == 1 && T.dev_alt) ? T.dev_alt : T.dev;
    };
    for (auto &n : l->nodes) {
        const void *ins[ENN_B200_CONCAT_MAX_INPUTS];
        for (size_t i = 0; i < n.ins.size(); ++i) ins[i] = ptr(n.ins[i]);
        const int32_t st = enn_b200_op_execute_n(n.op, ins, static_cast<int32_t>(n.ins.size()), ptr(n.out));
        if (st != ENN_B200_SUCCESS) return st;
    }
    return ENN_B200_SUCCESS;
}
}  // namespace

extern "C" {

int32_t enn_b200_oplist_create(enn_b200_context *ctx, enn_b200_oplist **out) {
    if (!ctx || !out) return ENN_B200_INVALID_PARAMS;
    enn_b200_oplist *l = new (std::nothrow) enn_b200_oplist();
    if (!l) return ENN_B200_FAILURE;
    l->ctx = ctx;
    *out = l;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_add_tensor(enn_b200_oplist *l, int64_t bytes, int32_t *tensor_id) {
    if (!l || !tensor_id || bytes < 0) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_tensor: bad argument");
    if (l->finalized) return lfail(l, ENN_B200_FAILURE, "oplist already finalized");
    enn_b200_oplist::Tensor t;
    t.bytes = bytes;
    l->tensors.push_back(t);
    *tensor_id = static_cast<int32_t>(l->tensors.size()) - 1;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_add_op(enn_b200_oplist *l, enn_b200_op *op, const int32_t *in_ids, int32_t n_in, int32_t out_id) {
    if (!l || !op || !in_ids || n_in < 1 || n_in > ENN_B200_CONCAT_MAX_INPUTS) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: bad argument");
    if (l->finalized) return lfail(l, ENN_B200_FAILURE, "oplist already finalized");
    if (op->dyn) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: operators with runtime filter / bias run outside operator lists");
    const int nt = static_cast<int>(l->tensors.size());
    if (out_id < 0 || out_id >= nt) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: bad output tensor id");
    for (int i = 0; i < n_in; ++i)
        if (in_ids[i] < 0 || in_ids[i] >= nt) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: bad input tensor id");
    const int want_in = op->kind == enn_b200::OP_ADD ? 2 : (op->kind == enn_b200::OP_CONCAT ? n_in : 1);
    if (n_in != want_in) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: wrong input count for this operator");
    if (l->tensors[out_id].bytes < op->info.out_bytes) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: output tensor too small");
    if (op->kind == enn_b200::OP_CONCAT) {
        int64_t have = 0;
        for (int i = 0; i < n_in; ++i) have += l->tensors[in_ids[i]].bytes;
        if (have < op->info.in_bytes) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: input tensors too small");
    } else {
        const int64_t need_in = n_in == 2 ? op->info.in_bytes / 2 : op->info.in_bytes;
        for (int i = 0; i < n_in; ++i)
            if (l->tensors[in_ids[i]].bytes < need_in) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_add_op: input tensor too small");
    }
    enn_b200_oplist::Node n;
    n.op = op;
    n.ins.assign(in_ids, in_ids + n_in);
    n.out = out_id;
    l->nodes.push_back(n);
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_set_io(enn_b200_oplist *l, const int32_t *input_ids, int32_t n_inputs, const int32_t *output_ids,
                               int32_t n_outputs) {
    if (!l || n_inputs < 0 || n_outputs < 0 || (n_inputs && !input_ids) || (n_outputs && !output_ids))
        return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_set_io: bad argument");
    if (l->finalized) return lfail(l, ENN_B200_FAILURE, "oplist already finalized");
    const int nt = static_cast<int>(l->tensors.size());
    l->inputs.assign(input_ids, input_ids + n_inputs);
    l->outputs.assign(output_ids, output_ids + n_outputs);
    for (int id : l->inputs)
        if (id < 0 || id >= nt) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_set_io: bad input id");
    for (int id : l->outputs)
        if (id < 0 || id >= nt) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_set_io: bad output id");
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_finalize(enn_b200_oplist *l) {
    if (!l) return ENN_B200_INVALID_PARAMS;
    if (l->finalized) return ENN_B200_SUCCESS;
    enn_b200_context *ctx = l->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "cudaSetDevice failed");
    for (int id : l->inputs) l->tensors[id].is_input = true;
    for (int id : l->outputs) l->tensors[id].is_output = true;
    // Convolution -> add (the residual blocks): where the convolution's result is read by that add only and its plan can
    // take it, the add moves into the convolution's epilogue and its node and the tensor between them disappear.
    if (!ctx->opt("no_fuse")) {
        std::vector<int> readers(l->tensors.size(), 0);
        for (auto &n : l->nodes)
            for (int t : n.ins) ++readers[t];
        for (size_t a = 0; a < l->nodes.size(); ++a) {
            auto &add = l->nodes[a];
            if (add.op->kind != enn_b200::OP_ADD || add.ins.size() != 2 || add.ins[0] == add.ins[1]) continue;
            // Large adds stay on their own: the stand-alone kernel runs them from the 64 KB pair table at HBM speed, while
            // the epilogue computes the last stage (about 20 integer instructions per output); below about two million
            // elements the add kernel is all launch latency and the fused form wins (measured on the MobileNetV2 graph:
            // fusing every add costs 2 % at 256 images per list, fusing the small ones gains at 32).
            if (add.op->count > kFuseAddMaxCount && !ctx->opt("fuse_all")) continue;
            for (int side = 0; side < 2; ++side) {
                const int mid = add.ins[side];
                const auto &M = l->tensors[mid];
                if (M.is_input || M.is_output || readers[mid] != 1) continue;
                int prod = -1;
                for (size_t c = 0; c < a; ++c)
                    if (l->nodes[c].out == mid) prod = static_cast<int>(c);      // the last writer before the add
                if (prod < 0 || l->nodes[prod].op->kind != enn_b200::OP_CONV || l->nodes[prod].ins.size() != 1) continue;
                // The other addend must exist before the convolution runs.
                const int other = add.ins[1 - side];
                bool other_ready = l->tensors[other].is_input;
                for (int c = 0; c < prod; ++c)
                    if (l->nodes[c].out == other) other_ready = true;
                for (size_t c = prod; c < a; ++c)
                    if (l->nodes[c].out == other) other_ready = false;            // rewritten in between
                if (!other_ready) continue;
                bool touched = false;      // nothing between the two may read or write the add's output tensor
                for (size_t c = prod; c < a && !touched; ++c) {
                    touched = l->nodes[c].out == add.out;
                    for (int t : l->nodes[c].ins) touched = touched || t == add.out;
                }
                if (touched) continue;
                if (enn_b200_op_fuse_add(l->nodes[prod].op, add.op, side) != ENN_B200_SUCCESS) continue;
                l->nodes[prod].ins.push_back(other);
                l->nodes[prod].out = add.out;
                // the convolution now runs where it did, but the other addend must stay alive until then and the add's
                // output is written earlier: both follow from the node order, which the liveness pass below reads
                l->nodes.erase(l->nodes.begin() + static_cast<long>(a));
                --a;
                break;
            }
        }
    }
    const int n_nodes = static_cast<int>(l->nodes.size());
    for (int i = 0; i < n_nodes; ++i) {
        auto &n = l->nodes[i];
        for (int t : n.ins) {
            auto &T = l->tensors[t];
            if (T.first_def < 0 && !T.is_input) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist: tensor read before it is written");
            T.last_use = i;
        }
        auto &O = l->tensors[n.out];
        if (O.first_def < 0) O.first_def = i;
        O.last_use = std::max(O.last_use, i);
    }
    // Liveness-based assignment: graph inputs/outputs get dedicated buffers (the caller's copies land there);
    // an intermediate takes the smallest free pool buffer that fits, and returns it after its last reader.
    std::vector<int> free_slots;
    std::vector<std::vector<int>> expiring(n_nodes + 1);
    auto new_slot = [&](int64_t bytes) {
        l->pool.push_back(nullptr);
        l->pool_bytes.push_back(bytes);
        return static_cast<int>(l->pool.size()) - 1;
    };
    for (auto &T : l->tensors)
        if (T.is_input || T.is_output || T.first_def < 0) T.pool_slot = new_slot(T.bytes);
    for (int i = 0; i < n_nodes; ++i) {
        auto &T = l->tensors[l->nodes[i].out];
        if (T.pool_slot < 0) {
            int best = -1;
            for (size_t k = 0; k < free_slots.size(); ++k) {
                const int s = free_slots[k];
                if (l->pool_bytes[s] >= T.bytes && (best < 0 || l->pool_bytes[s] < l->pool_bytes[free_slots[best]])) best = static_cast<int>(k);
            }
            if (best >= 0) {
                T.pool_slot = free_slots[best];
                free_slots.erase(free_slots.begin() + best);
            } else {
                T.pool_slot = new_slot(T.bytes);
            }
            expiring[T.last_use].push_back(T.pool_slot);
        }
        // Buffers whose last reader is this node become free for the NEXT node (never for this node's output).
        for (int s : expiring[i]) free_slots.push_back(s);
    }
    l->device_bytes = 0;
    for (size_t s = 0; s < l->pool.size(); ++s) {
        const size_t bytes = static_cast<size_t>(l->pool_bytes[s] > 0 ? l->pool_bytes[s] : 1);
        if (cudaMalloc(&l->pool[s], (bytes + 255) & ~static_cast<size_t>(255)) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: device allocation failed");
        l->device_bytes += static_cast<int64_t>(bytes);
    }
    for (auto &T : l->tensors) T.dev = T.pool_slot >= 0 ? l->pool[T.pool_slot] : nullptr;
    l->kernel_launches = 0;
    for (auto &n : l->nodes) l->kernel_launches += n.op->info.kernel_launches;

    // One eager pass (lets every operator build the state it creates lazily for fixed pointers), then capture.
    int32_t st = run_nodes(l);
    if (st != ENN_B200_SUCCESS) return st;
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: warm-up pass failed");
    if (n_nodes > 0) {
        if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: stream capture could not start");
        st = run_nodes(l);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &l->graph);
        if (st != ENN_B200_SUCCESS) return st;
        if (e != cudaSuccess || !l->graph) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: stream capture failed");
        if (cudaGraphInstantiate(&l->exec, l->graph, 0) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: graph instantiation failed");
        // Second buffer set + graph for pipelined submission.
        for (auto &T : l->tensors)
            if (T.is_input || T.is_output) {
                const size_t bytes = static_cast<size_t>(T.bytes > 0 ? T.bytes : 1);
                if (cudaMalloc(&T.dev_alt, (bytes + 255) & ~static_cast<size_t>(255)) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: device allocation failed");
                l->device_bytes += static_cast<int64_t>(bytes);
            }
        st = run_nodes(l, 1);      // eager pass on the alternate pointers (operators cache per-pointer state)
        if (st != ENN_B200_SUCCESS) return st;
        if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: warm-up pass failed");
        if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: stream capture could not start");
        st = run_nodes(l, 1);
        e = cudaStreamEndCapture(ctx->stream, &l->graph_alt);
        if (st != ENN_B200_SUCCESS) return st;
        if (e != cudaSuccess || !l->graph_alt) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: stream capture failed");
        if (cudaGraphInstantiate(&l->exec_alt, l->graph_alt, 0) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: graph instantiation failed");
        if (cudaStreamCreateWithFlags(&l->copy_stream, cudaStreamNonBlocking) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: copy stream creation failed");
        if (!ctx->opt("no_out_stream") && cudaStreamCreateWithFlags(&l->out_stream, cudaStreamNonBlocking) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: output stream creation failed");
        for (int i = 0; i < 2; ++i)
            if (cudaEventCreateWithFlags(&l->ev_in_ready[i], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&l->ev_done[i], cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&l->ev_slot_free[i], cudaEventDisableTiming) != cudaSuccess)
                return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: event creation failed");
    }
    l->finalized = true;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_execute_device(enn_b200_oplist *l) {
    if (!l || !l->finalized) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist not finalized");
    if (!l->exec) return ENN_B200_SUCCESS;
    if (cudaGraphLaunch(l->exec, l->ctx->stream) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist: graph launch failed");
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_execute(enn_b200_oplist *l, const void *const *host_inputs, void *const *host_outputs) {
    if (!l || !l->finalized) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist not finalized");
    if ((!l->inputs.empty() && !host_inputs) || (!l->outputs.empty() && !host_outputs)) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_execute: null buffer table");
    cudaStream_t s = l->ctx->stream;
    for (size_t i = 0; i < l->inputs.size(); ++i) {
        auto &T = l->tensors[l->inputs[i]];
        if (!host_inputs[i]) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_execute: null input buffer");
        if (T.bytes && cudaMemcpyAsync(T.dev, host_inputs[i], static_cast<size_t>(T.bytes), cudaMemcpyHostToDevice, s) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_execute: input copy failed");
    }
    int32_t st = enn_b200_oplist_execute_device(l);
    if (st != ENN_B200_SUCCESS) return st;
    for (size_t i = 0; i < l->outputs.size(); ++i) {
        auto &T = l->tensors[l->outputs[i]];
        if (!host_outputs[i]) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_execute: null output buffer");
        if (T.bytes && cudaMemcpyAsync(host_outputs[i], T.dev, static_cast<size_t>(T.bytes), cudaMemcpyDeviceToHost, s) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_execute: output copy failed");
    }
    if (cudaStreamSynchronize(s) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_execute: stream synchronisation failed");
    return ENN_B200_SUCCESS;
}

// Pipelined ExecuteSubGraph: returns as soon as the work is queued.  The host-to-device copy of this submission runs
// on a copy stream and overlaps the operators of the previous one (two device copies of every graph input / output
// alternate); results are valid in host_outputs after enn_b200_oplist_wait.  Host buffers must stay alive and untouched
// until then and should be pinned.
namespace {
// First half of a pipelined submission: this step's inputs travel to the free buffer set on the list's copy stream.
int32_t submit_inputs(enn_b200_oplist *l, const void *const *host_inputs, int slot, enn_b200_oplist *const *others = nullptr,
                      int32_t n_others = 0) {
    cudaStream_t cs = l->copy_stream;
    // A round's inputs travel after those of the round before: the copy engine serves the lists' copy streams in no
    // particular order, and a copy of the next round that overtakes one of this round delays all graphs of this round
    // (four lists, 38.5 MB inputs: the first round started 2.1 ms late).
    for (int32_t j = 0; j < n_others; ++j)
        if (others[j]->seq > 0 && cudaStreamWaitEvent(cs, others[j]->ev_in_ready[(others[j]->seq & 1) ^ 1], 0) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event wait failed");
    // the previous user of this buffer set must have finished reading its inputs and copying out its outputs
    if (l->slot_used[slot] && cudaStreamWaitEvent(cs, l->ev_slot_free[slot], 0) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event wait failed");
    for (size_t i = 0; i < l->inputs.size(); ++i) {
        auto &T = l->tensors[l->inputs[i]];
        if (!host_inputs[i]) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit: null input buffer");
        void *dst = slot ? T.dev_alt : T.dev;
        if (T.bytes && cudaMemcpyAsync(dst, host_inputs[i], static_cast<size_t>(T.bytes), cudaMemcpyHostToDevice, cs) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: input copy failed");
    }
    if (cudaEventRecord(l->ev_in_ready[slot], cs) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event record failed");
    return ENN_B200_SUCCESS;
}
// Second half: the graph on the list's stream once its inputs (and those of `others`, the lists of the same round)
// have landed, then the results on the output stream.
int32_t submit_run(enn_b200_oplist *l, void *const *host_outputs, int slot, enn_b200_oplist *const *others, int32_t n_others) {
    cudaStream_t s = l->ctx->stream;
    if (cudaStreamWaitEvent(s, l->ev_in_ready[slot], 0) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event hand-over failed");
    for (int32_t j = 0; j < n_others; ++j)
        if (others[j] != l && cudaStreamWaitEvent(s, others[j]->ev_in_ready[others[j]->seq & 1], 0) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event hand-over failed");
    if (cudaGraphLaunch(slot ? l->exec_alt : l->exec, s) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: graph launch failed");
    // The results leave on a stream of their own: the next graph of this list starts when this one ends, not when the
    // copy engine (busy with the other lists' inputs) has served the result copy.
    cudaStream_t os = l->out_stream ? l->out_stream : s;
    if (os != s && (cudaEventRecord(l->ev_done[slot], s) != cudaSuccess || cudaStreamWaitEvent(os, l->ev_done[slot], 0) != cudaSuccess))
        return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event hand-over failed");
    for (size_t i = 0; i < l->outputs.size(); ++i) {
        auto &T = l->tensors[l->outputs[i]];
        if (!host_outputs[i]) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit: null output buffer");
        const void *src = slot ? T.dev_alt : T.dev;
        if (T.bytes && cudaMemcpyAsync(host_outputs[i], src, static_cast<size_t>(T.bytes), cudaMemcpyDeviceToHost, os) != cudaSuccess)
            return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: output copy failed");
    }
    if (cudaEventRecord(l->ev_slot_free[slot], os) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_submit: event record failed");
    return ENN_B200_SUCCESS;
}
}  // namespace

int32_t enn_b200_oplist_submit(enn_b200_oplist *l, const void *const *host_inputs, void *const *host_outputs) {
    if (!l || !l->finalized) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist not finalized");
    if ((!l->inputs.empty() && !host_inputs) || (!l->outputs.empty() && !host_outputs)) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit: null buffer table");
    if (!l->exec || !l->exec_alt) return enn_b200_oplist_execute(l, host_inputs, host_outputs);
    const int slot = static_cast<int>(l->seq & 1);
    int32_t st = submit_inputs(l, host_inputs, slot);
    if (st == ENN_B200_SUCCESS) st = submit_run(l, host_outputs, slot, nullptr, 0);
    if (st != ENN_B200_SUCCESS) return st;
    l->slot_used[slot] = true;
    ++l->seq;
    return ENN_B200_SUCCESS;
}

// One step on each of `n` lists of the same device whose operators start together: every list's inputs are copied
// first, and every list's graph waits for all of them.  Lists that share a GPU (each prepared with option grid_cap, so
// that their kernels fit side by side) run fastest when they execute the same layer at the same time: kernels of
// one kind fill every SM, while a mix of kinds leaves SMs that hold a small CTA closed to a large one.
// host_inputs[k] / host_outputs[k] are the buffer tables of lists[k], as for enn_b200_oplist_submit.
int32_t enn_b200_oplist_submit_round(enn_b200_oplist *const *lists, int32_t n, const void *const *const *host_inputs,
                                     void *const *const *host_outputs) {
    if (!lists || n < 1 || n > 64 || !host_inputs || !host_outputs) return ENN_B200_INVALID_PARAMS;
    for (int32_t k = 0; k < n; ++k) {
        enn_b200_oplist *l = lists[k];
        if (!l || !l->finalized) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist not finalized");
        if (!l->exec || !l->exec_alt) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit_round: a list without operators");
        if ((!l->inputs.empty() && !host_inputs[k]) || (!l->outputs.empty() && !host_outputs[k])) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit_round: null buffer table");
        if (l->ctx->device != lists[0]->ctx->device) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit_round: lists of different devices");
        for (int32_t j = 0; j < k; ++j)
            if (lists[j] == l) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_submit_round: a list named twice");
    }
    for (int32_t k = 0; k < n; ++k) {
        const int32_t st = submit_inputs(lists[k], host_inputs[k], static_cast<int>(lists[k]->seq & 1), lists, n);
        if (st != ENN_B200_SUCCESS) return st;
    }
    for (int32_t k = 0; k < n; ++k) {
        const int32_t st = submit_run(lists[k], host_outputs[k], static_cast<int>(lists[k]->seq & 1), lists, n);
        if (st != ENN_B200_SUCCESS) return st;
    }
    for (int32_t k = 0; k < n; ++k) {
        lists[k]->slot_used[lists[k]->seq & 1] = true;
        ++lists[k]->seq;
    }
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_wait(enn_b200_oplist *l) {
    if (!l || !l->finalized) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist not finalized");
    if (l->copy_stream && cudaStreamSynchronize(l->copy_stream) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_wait: copy stream failed");
    if (cudaStreamSynchronize(l->ctx->stream) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_wait: stream synchronisation failed");
    if (l->out_stream && cudaStreamSynchronize(l->out_stream) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "oplist_wait: output stream failed");
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_tensor_ptr(enn_b200_oplist *l, int32_t tensor_id, void **dev_ptr) {
    if (!l || !dev_ptr || tensor_id < 0 || tensor_id >= static_cast<int32_t>(l->tensors.size())) return ENN_B200_INVALID_PARAMS;
    if (!l->finalized) return lfail(l, ENN_B200_FAILURE, "oplist not finalized");
    *dev_ptr = l->tensors[tensor_id].dev;
    return ENN_B200_SUCCESS;
}

// Device address of graph output `output_index` as written by the most recent submit / execute (pipelined submissions
// alternate between two device copies of every graph input and output).
int32_t enn_b200_oplist_last_output_ptr(enn_b200_oplist *l, int32_t output_index, void **dev_ptr) {
    if (!l || !dev_ptr || output_index < 0 || output_index >= static_cast<int32_t>(l->outputs.size())) return ENN_B200_INVALID_PARAMS;
    if (!l->finalized) return lfail(l, ENN_B200_FAILURE, "oplist not finalized");
    auto &T = l->tensors[l->outputs[output_index]];
    const bool alt = l->seq > 0 && ((l->seq - 1) & 1) && T.dev_alt;
    *dev_ptr = alt ? T.dev_alt : T.dev;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_node_count(const enn_b200_oplist *l, int32_t *n_nodes) {
    if (!l || !n_nodes) return ENN_B200_INVALID_PARAMS;
    *n_nodes = static_cast<int32_t>(l->nodes.size());
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_node_info(const enn_b200_oplist *l, int32_t index, enn_b200_op_info_t *info, int32_t *kind, int32_t *n_inputs) {
    if (!l || index < 0 || index >= static_cast<int32_t>(l->nodes.size())) return ENN_B200_INVALID_PARAMS;
    const auto &n = l->nodes[index];
    if (info) *info = n.op->info;
    if (kind) *kind = n.op->kind;
    if (n_inputs) *n_inputs = static_cast<int32_t>(n.ins.size());
    return ENN_B200_SUCCESS;
}

// Device time of every node: the nodes are launched one by one on the list's own tensors with an event between them
// (the role of the PROFILE_FROM / PROFILE_UNTIL pair around every operator, userdriver_operator.h:35-42).
int32_t enn_b200_oplist_profile(enn_b200_oplist *l, int32_t repeats, float *node_us, int32_t capacity) {
    if (!l || !l->finalized) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist not finalized");
    const int n = static_cast<int>(l->nodes.size());
    if (!node_us || capacity < n || repeats < 1 || repeats > 1000) return lfail(l, ENN_B200_INVALID_PARAMS, "oplist_profile: bad argument");
    enn_b200_context *ctx = l->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return lfail(l, ENN_B200_CUDA_FAILURE, "cudaSetDevice failed");
    std::vector<cudaEvent_t> ev(n + 1, nullptr);
    int32_t st = ENN_B200_SUCCESS;
    for (auto &e : ev)
        if (cudaEventCreate(&e) != cudaSuccess) st = lfail(l, ENN_B200_CUDA_FAILURE, "oplist_profile: event creation failed");
    for (int i = 0; i < n; ++i) node_us[i] = 0.f;
    for (int rep = -1; rep < repeats && st == ENN_B200_SUCCESS; ++rep) {      // pass -1 warms up
        cudaEventRecord(ev[0], ctx->stream);
        for (int i = 0; i < n && st == ENN_B200_SUCCESS; ++i) {
            const auto &nd = l->nodes[i];
            const void *ins[ENN_B200_CONCAT_MAX_INPUTS];
            for (size_t k = 0; k < nd.ins.size(); ++k) ins[k] = l->tensors[nd.ins[k]].dev;
            st = enn_b200_op_execute_n(nd.op, ins, static_cast<int32_t>(nd.ins.size()), l->tensors[nd.out].dev);
            cudaEventRecord(ev[i + 1], ctx->stream);
        }
        if (st == ENN_B200_SUCCESS && cudaStreamSynchronize(ctx->stream) != cudaSuccess) st = lfail(l, ENN_B200_CUDA_FAILURE, "oplist_profile: execution failed");
        for (int i = 0; i < n && st == ENN_B200_SUCCESS && rep >= 0; ++i) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, ev[i], ev[i + 1]);
            node_us[i] += ms * 1000.f / static_cast<float>(repeats);
        }
    }
    for (auto &e : ev)
        if (e) cudaEventDestroy(e);
    return st;
}

int32_t enn_b200_oplist_stats(enn_b200_oplist *l, int64_t *device_bytes, int32_t *n_buffers, int32_t *kernel_launches) {
    if (!l || !l->finalized) return ENN_B200_INVALID_PARAMS;
    if (device_bytes) *device_bytes = l->device_bytes;
    if (n_buffers) *n_buffers = static_cast<int32_t>(l->pool.size());
    if (kernel_launches) *kernel_launches = l->kernel_launches;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_oplist_destroy(enn_b200_oplist *l) {
    if (!l) return ENN_B200_INVALID_PARAMS;
    if (l->ctx) {
        cudaSetDevice(l->ctx->device);
        cudaStreamSynchronize(l->ctx->stream);
    }
    if (l->copy_stream) {
        cudaStreamSynchronize(l->copy_stream);
        cudaStreamDestroy(l->copy_stream);
    }
    if (l->out_stream) {
        cudaStreamSynchronize(l->out_stream);
        cudaStreamDestroy(l->out_stream);
    }
    for (int i = 0; i < 2; ++i) {
        if (l->ev_done[i]) cudaEventDestroy(l->ev_done[i]);
        if (l->ev_in_ready[i]) cudaEventDestroy(l->ev_in_ready[i]);
        if (l->ev_slot_free[i]) cudaEventDestroy(l->ev_slot_free[i]);
    }
    if (l->exec) cudaGraphExecDestroy(l->exec);
    if (l->graph) cudaGraphDestroy(l->graph);
    if (l->exec_alt) cudaGraphExecDestroy(l->exec_alt);
    if (l->graph_alt) cudaGraphDestroy(l->graph_alt);
    for (auto &T : l->tensors)
        if (T.dev_alt) cudaFree(T.dev_alt);
    for (auto &n : l->nodes) enn_b200_op_release(n.op);
    for (void *p : l->pool)
        if (p) cudaFree(p);
    delete l;
    return ENN_B200_SUCCESS;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------------
// Operator-list group: one ExecuteSubGraph call over several devices.
//
// The reference's GpuUserDriver::ExecuteSubGraph (gpu_userdriver.cc) takes the whole batch in one call.  A group holds
// one finalized operator list per device (or several per device), each built for its share of the batch; one call
// splits every graph input along its outermost dimension into contiguous slices (member i takes the next
// bytes-of-its-input-tensor bytes), runs the members side by side, one host worker thread per member, and lands every
// member's outputs at the matching offsets of the caller's output buffers.  There is no collective: batch slices are
// independent, only the results meet again, in host memory.
// ------------------------------------------------------------------------------------------------------
#include <condition_variable>
#include <mutex>
#include <thread>

struct enn_b200_group {
    struct Member {
        enn_b200_oplist *list = nullptr;
        std::thread worker;
        std::vector<const void *> ins;
        std::vector<void *> outs;
        int job = 0;            // 0 idle, 1 execute (blocking), 2 submit, 3 wait, -1 quit
        int32_t status = ENN_B200_SUCCESS;
        bool done = true;
    };
    std::vector<Member> members;
    std::mutex m;
    std::condition_variable cv_job, cv_done;
    std::string last_error;
};

namespace {
void group_worker(enn_b200_group *g, int idx) {
    enn_b200_group::Member &me = g->members[idx];
    cudaSetDevice(me.list->ctx->device);       // the worker's current device for its whole life
    for (;;) {
        int job;
        {
            std::unique_lock<std::mutex> lk(g->m);
            g->cv_job.wait(lk, [&] { return me.job != 0; });
            job = me.job;
        }
        int32_t st = ENN_B200_SUCCESS;
        if (job == 1) st = enn_b200_oplist_execute(me.list, me.ins.data(), me.outs.data());
        else if (job == 2) st = enn_b200_oplist_submit(me.list, me.ins.data(), me.outs.data());
        else if (job == 3) st = enn_b200_oplist_wait(me.list);
        {
            std::lock_guard<std::mutex> lk(g->m);
            me.status = st;
            me.job = 0;
            me.done = true;
        }
        g->cv_done.notify_all();
        if (job < 0) return;
    }
}

// Hands `job` to every member (with its slices of the caller's buffers for jobs 1 and 2) and waits for all of them.
int32_t group_run(enn_b200_group *g, int job, const void *const *host_inputs, void *const *host_outputs) {
    if (!g) return ENN_B200_INVALID_PARAMS;
    if (job == 1 || job == 2) {
        const size_t n_in = g->members[0].list->inputs.size(), n_out = g->members[0].list->outputs.size();
        if ((n_in && !host_inputs) || (n_out && !host_outputs)) return ENN_B200_INVALID_PARAMS;
        std::vector<size_t> in_off(n_in, 0), out_off(n_out, 0);
        for (auto &me : g->members) {
            me.ins.resize(n_in);
            me.outs.resize(n_out);
            for (size_t i = 0; i < n_in; ++i) {
                if (!host_inputs[i]) return ENN_B200_INVALID_PARAMS;
                me.ins[i] = static_cast<const uint8_t *>(host_inputs[i]) + in_off[i];
                in_off[i] += static_cast<size_t>(me.list->tensors[me.list->inputs[i]].bytes);
            }
            for (size_t i = 0; i < n_out; ++i) {
                if (!host_outputs[i]) return ENN_B200_INVALID_PARAMS;
                me.outs[i] = static_cast<uint8_t *>(host_outputs[i]) + out_off[i];
                out_off[i] += static_cast<size_t>(me.list->tensors[me.list->outputs[i]].bytes);
            }
        }
    }
    {
        std::lock_guard<std::mutex> lk(g->m);
        for (auto &me : g->members) {
            me.done = false;
            me.job = job;
        }
    }
    g->cv_job.notify_all();
    int32_t st = ENN_B200_SUCCESS;
    {
        std::unique_lock<std::mutex> lk(g->m);
        g->cv_done.wait(lk, [&] {
            for (auto &me : g->members)
                if (!me.done) return false;
            return true;
        });
        for (auto &me : g->members)
            if (me.status != ENN_B200_SUCCESS && st == ENN_B200_SUCCESS) {
                st = me.status;
                g->last_error = me.list->ctx->last_error;
            }
    }
    return st;
}
}  // namespace

extern "C" {

int32_t enn_b200_group_create(enn_b200_oplist *const *lists, int32_t n_lists, enn_b200_group **out) {
    if (!lists || n_lists < 1 || !out) return ENN_B200_INVALID_PARAMS;
    *out = nullptr;
    for (int i = 0; i < n_lists; ++i) {
        if (!lists[i] || !lists[i]->finalized) return ENN_B200_INVALID_PARAMS;
        if (lists[i]->inputs.size() != lists[0]->inputs.size() || lists[i]->outputs.size() != lists[0]->outputs.size())
            return lfail(lists[i], ENN_B200_INVALID_PARAMS, "group: members differ in their number of graph inputs / outputs");
        for (int k = 0; k < i; ++k)
            if (lists[k] == lists[i] || lists[k]->ctx == lists[i]->ctx)
                return lfail(lists[i], ENN_B200_INVALID_PARAMS, "group: every member needs its own list and context");
    }
    enn_b200_group *g = new (std::nothrow) enn_b200_group();
    if (!g) return ENN_B200_FAILURE;
    g->members.resize(n_lists);
    for (int i = 0; i < n_lists; ++i) g->members[i].list = lists[i];
    for (int i = 0; i < n_lists; ++i) g->members[i].worker = std::thread(group_worker, g, i);
    *out = g;
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_group_execute(enn_b200_group *g, const void *const *host_inputs, void *const *host_outputs) {
    return group_run(g, 1, host_inputs, host_outputs);
}

int32_t enn_b200_group_submit(enn_b200_group *g, const void *const *host_inputs, void *const *host_outputs) {
    return group_run(g, 2, host_inputs, host_outputs);
}

int32_t enn_b200_group_wait(enn_b200_group *g) { return group_run(g, 3, nullptr, nullptr); }

int32_t enn_b200_group_last_error(enn_b200_group *g, char *buf, size_t buf_len) {
    if (!buf || !buf_len) return ENN_B200_SUCCESS;
    std::snprintf(buf, buf_len, "%s", g ? g->last_error.c_str() : "null group");
    return ENN_B200_SUCCESS;
}

int32_t enn_b200_group_destroy(enn_b200_group *g, int32_t destroy_lists) {
    if (!g) return ENN_B200_INVALID_PARAMS;
    group_run(g, -1, nullptr, nullptr);
    for (auto &me : g->members)
        if (me.worker.joinable()) me.worker.join();
    if (destroy_lists)
        for (auto &me : g->members) enn_b200_oplist_destroy(me.list);
    delete g;
    return ENN_B200_SUCCESS;
}

}  // extern "C"
