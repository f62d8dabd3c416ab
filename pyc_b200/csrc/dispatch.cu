// pyc_cuda_dispatch: run one compiled PyC IR module on the GPU.
//
// Replaces src/compiler/runtime/cuda_backend.c:2495-2928 of PyC
// (execute_native_cuda_graph_cuda + pyc_cuda_dispatch_impl) and its graph parser
// (parse_matmul_chain_graph, cuda_backend.c:1232-1390).  Differences by design:
//   * any topologically ordered sequence of INPUT / MATMUL / ADD / RELU / GELU /
//     REDUCE_SUM / LAYERNORM / OUTPUT ops is accepted, not just one matmul chain;
//   * matmul -> add(bias) -> relu|gelu is re-fused here from the UNFUSED chain
//     (PyC switches its own lossy fusion pass off for this backend,
//     src/compiler/compiler_api.c:2484-2488) into the GEMM kernel's epilogue;
//   * intermediates live in ONE device arena at offsets from a first-fit
//     lifetime plan (the algorithm of src/compiler/runtime/runtime_allocator.c:
//     123-187, fed with real def/last-use steps instead of PyC's [i, i+2]);
//   * the whole step list (H2D copies, kernels, D2H copies) is captured once per
//     (module, tensor descriptors) as a CUDA graph and replayed afterwards;
//   * tensors may be device pointers (zero copy) or host pointers (pinned
//     staging, as PyC does at cuda_backend.c:1766-1853).
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <map>
#include <memory>
#include <mutex>
#include <algorithm>
#include <string>
#include <vector>

#include "internal.h"
#include "runtime.h"

namespace b200 {
int run_simulated_device(const pyc_ir_module* module, const pyc_tensor* inputs, size_t input_count,
                         pyc_tensor* outputs, size_t output_count);
}

using namespace b200;

namespace {

double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Same truthiness rules as PyC's env_true / env_default_true (cuda_backend.c:653-670).
bool env_true(const char* name) {
    const char* v = getenv(name);
    return v && (!strcmp(v, "1") || !strcmp(v, "true") || !strcmp(v, "TRUE"));
}
bool env_is_false_value(const char* name) {
    const char* v = getenv(name);
    return v && (!strcmp(v, "0") || !strcmp(v, "false") || !strcmp(v, "FALSE"));
}
bool env_default_true(const char* name) {
    const char* v = getenv(name);
    if (!v || !v[0]) return true;
    return !(!strcmp(v, "0") || !strcmp(v, "false") || !strcmp(v, "FALSE"));
}

void set_reason(pyc_cuda_dispatch_trace* t, const char* s) {
    if (!t) return;
    strncpy(t->reason, s, PYC_CUDA_REASON_MAX - 1);
    t->reason[PYC_CUDA_REASON_MAX - 1] = '\0';
}

enum MemKind { MEM_PAGEABLE = 0, MEM_PINNED = 1, MEM_DEVICE = 2 };
MemKind classify_pointer(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return MEM_PAGEABLE; }
    if (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) return MEM_DEVICE;
    if (a.type == cudaMemoryTypeHost) return MEM_PINNED;
    return MEM_PAGEABLE;
}

enum ValueKind { V_NONE = 0, V_INPUT_DIRECT, V_TEMP, V_OUTPUT_DIRECT, V_ALIAS };
struct Value {
    ValueKind kind = V_NONE;
    int ext = -1;            // index into inputs[] / outputs[]
    int alias_of = -1;
    pyc_dtype dtype = PYC_DTYPE_UNKNOWN;
    size_t rank = 0;
    int64_t dims[PYC_IR_MAX_DIMS] = {0};
    size_t elems = 0, bytes = 0;
    size_t arena_off = 0;
    int def_step = -1, last_step = -1;
    int consumers = 0;
};

enum StepKind { S_H2D = 0, S_GEMM, S_ADD, S_BIAS_ACT, S_LAYERNORM, S_REDUCE_SUM, S_COPY, S_D2H, S_SOFTMAX, S_ATTENTION, S_CONV2D, S_FFN_FP8 };
struct Step {
    StepKind kind;
    int out = -1;            // value id written (temps) or -1
    int in0 = -1, in1 = -1, in2 = -1, in3 = -1, in4 = -1;
    int scratch = -1;        // value id of a step-private workspace in the arena (extended ops)
    int xp[12] = {0};        // parameters of an extended op (see parse_extended_op)
    int ext = -1;            // inputs[]/outputs[] index for copies
    int add_mode = 0, act = 0;
    size_t rows = 0, cols = 0, bytes = 0;
    int M = 0, N = 0, K = 0;
    size_t stage_off = 0;    // offset in the pinned staging buffer (pageable host tensors)
    bool via_stage = false;
    int op_main = -1, op_add = -1, op_act = -1;   // IR op ids this step stands for (the fused add / activation when absorbed)
    std::string symbol, chosen_by;                // kernel that ran the step and who picked it (GEMM steps), set at enqueue
};

struct Plan {
    std::vector<Value> values;   // one per IR op, then extra temps
    std::vector<Step> steps;
    size_t arena_peak = 0, arena_total = 0, stage_bytes = 0;
    std::string symbol;          // GEMM configuration of the first matmul (for the reason string)
    std::string description;     // one line per step: kernel symbol and the IR ops it absorbed (pyc_b200_last_plan)
    uint64_t module_hash = 0;    // content hash of the IR ops alone (no tensor addresses)
    bool all_device = true;
    // Host-tensor pipeline (see plan_pipeline): index of the GEMM step, rows per chunk, chunk count.
    int pipe_gemm = -1, pipe_rows = 0, pipe_chunks = 0;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int resolve(const std::vector<Value>& vals, int id) {
    while (id >= 0 && vals[id].kind == V_ALIAS) id = vals[id].alias_of;
    return id;
}

uint64_t fnv1a(uint64_t h, const void* data, size_t n) {
    const unsigned char* p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}

// ---- ops PyC's IR cannot name: the side table is the op NAME ---------------------------------------------------------
// PyC's op kinds stop at matmul / add / relu / gelu / reduce_sum / layernorm (include/pyc/ir.h:16-40) and its ops carry no
// attributes.  Without touching a PyC header, an op of kind REDUCE_SUM (the one kind whose declared shape PyC's shape
// inference leaves alone, src/compiler/passes/pass_manager.c:171-203) whose NAME starts with "b200." is read as:
//   b200.softmax                        softmax over the last axis of input 0
//   b200.attention[.causal]             inputs Q, K, V of shape [..., S, D]: softmax(Q K^T / sqrt(D)) V per leading index
//   b200.conv2d.p<ph>x<pw>.s<sh>x<sw>[.relu]   inputs X [N,H,W,C], W [K,R,S,C] and optionally bias [K]; NHWC forward convolution
//   b200.ffn_fp8                        inputs x [T,H] bf16, W1 [H,I] and W2 [I,H] as I8 (e4m3 codes), s1 [I], s2 [H] f32:
//                                       gelu(layernorm(x) W1) W2 with per-token activation quantisation (bf16 out)
// The op's declared shape is its output shape.  Names survive PyC's compile step unchanged and are part of its module
// fingerprint, so PyC's caches tell such modules apart.  PyC's CPU executor does not know these ops (it rejects REDUCE_SUM):
// such a module has no CPU fallback, by construction.
enum ExtOp { EXT_NONE = 0, EXT_SOFTMAX, EXT_ATTENTION, EXT_CONV2D, EXT_FFN_FP8, EXT_BAD };
ExtOp parse_extended_op(const char* name, int* xp) {
    if (strncmp(name, "b200.", 5) != 0) return EXT_NONE;
    const char* r = name + 5;
    if (!strcmp(r, "softmax")) return EXT_SOFTMAX;
    if (!strcmp(r, "attention")) { xp[0] = 0; return EXT_ATTENTION; }
    if (!strcmp(r, "attention.causal")) { xp[0] = 1; return EXT_ATTENTION; }
    if (!strcmp(r, "ffn_fp8")) return EXT_FFN_FP8;
    if (!strncmp(r, "conv2d.", 7)) {
        int ph = 0, pw = 0, sh = 1, sw = 1, used = 0;
        if (sscanf(r + 7, "p%dx%d.s%dx%d%n", &ph, &pw, &sh, &sw, &used) != 4) return EXT_BAD;
        const char* tail = r + 7 + used;
        if (tail[0] && strcmp(tail, ".relu") != 0) return EXT_BAD;
        xp[0] = ph; xp[1] = pw; xp[2] = sh; xp[3] = sw; xp[4] = tail[0] ? 1 : 0;
        return EXT_CONV2D;
    }
    return EXT_BAD;
}

// Build the step list.  Returns 0, 1 (module uses something the GPU path does not
// know: caller falls back) or -1 (malformed call).
int build_plan(const pyc_ir_module* m, const pyc_tensor* inputs, size_t n_in, pyc_tensor* outputs, size_t n_out,
               const std::vector<MemKind>& in_mem, const std::vector<MemKind>& out_mem, bool skip_out_copy,
               unsigned static_mask, Plan* plan) {
    const size_t n = m->op_count;
    std::vector<Value>& V = plan->values;
    V.assign(n, Value());
    V.reserve(n + 64);        // step-private workspaces are appended behind the ops' values without moving them
    size_t in_i = 0, out_i = 0;

    // Pass 1: shapes, dtypes, consumer counts.
    for (size_t i = 0; i < n; ++i) {
        const pyc_ir_op& op = m->ops[i];
        Value& v = V[i];
        for (size_t j = 0; j < op.input_count; ++j) {
            if (op.input_ids[j] < 0 || static_cast<size_t>(op.input_ids[j]) >= i) return -1;
            V[op.input_ids[j]].consumers++;
        }
        auto copy_shape = [&](const Value& s) { v.rank = s.rank; memcpy(v.dims, s.dims, sizeof(v.dims)); v.dtype = s.dtype; };
        switch (op.kind) {
            case PYC_IR_OP_INPUT: {
                if (in_i >= n_in || !inputs[in_i].data) return -1;
                const pyc_shape& s = op.shape.rank ? op.shape : inputs[in_i].shape;
                v.rank = s.rank; memcpy(v.dims, s.dims, sizeof(v.dims));
                v.dtype = op.dtype != PYC_DTYPE_UNKNOWN ? op.dtype : inputs[in_i].dtype;
                if (inputs[in_i].dtype != v.dtype) return -1;
                v.ext = static_cast<int>(in_i++);
                break;
            }
            case PYC_IR_OP_MATMUL: {
                if (op.input_count < 2) return -1;
                const Value &a = V[op.input_ids[0]], &b = V[op.input_ids[1]];
                if (a.rank != 2 || b.rank != 2 || a.dims[1] != b.dims[0] || a.dtype != b.dtype) return 1;
                v.rank = 2; v.dims[0] = a.dims[0]; v.dims[1] = b.dims[1]; v.dtype = a.dtype;
                break;
            }
            case PYC_IR_OP_ADD: {
                if (op.input_count < 2) return -1;
                const Value &a = V[op.input_ids[0]], &b = V[op.input_ids[1]];
                copy_shape(a.elems >= b.elems ? a : b);
                if (a.dtype != b.dtype) return 1;
                break;
            }
            case PYC_IR_OP_RELU: case PYC_IR_OP_GELU: case PYC_IR_OP_LAYERNORM: case PYC_IR_OP_OUTPUT:
                if (op.input_count < 1) return -1;
                copy_shape(V[op.input_ids[0]]);
                break;
            case PYC_IR_OP_REDUCE_SUM: {
                if (op.input_count < 1) return -1;
                const Value& a = V[op.input_ids[0]];
                int xp[12] = {0};
                const ExtOp ext = parse_extended_op(op.name, xp);
                if (ext == EXT_BAD) return 1;
                if (ext != EXT_NONE) {
                    if (ext == EXT_SOFTMAX && !op.shape.rank) { copy_shape(a); break; }
                    if (!op.shape.rank) return -1;          // the declared shape IS the output shape
                    v.rank = op.shape.rank; memcpy(v.dims, op.shape.dims, sizeof(v.dims));
                    v.dtype = ext == EXT_FFN_FP8 ? PYC_DTYPE_BF16 : a.dtype;
                    break;
                }
                if (op.shape.rank) { v.rank = op.shape.rank; memcpy(v.dims, op.shape.dims, sizeof(v.dims)); }
                else if (a.rank > 1) { v.rank = a.rank - 1; memcpy(v.dims, a.dims, sizeof(v.dims)); v.dims[a.rank - 1] = 0; }
                else { v.rank = 1; v.dims[0] = 1; }
                v.dtype = a.dtype;
                break;
            }
            default:
                return 1;  // CONST carries no payload in PyC's IR; PyC's executors reject it too
        }
        if (v.dtype != PYC_DTYPE_F32 && v.dtype != PYC_DTYPE_BF16 && v.dtype != PYC_DTYPE_F16) {
            // Other dtypes are only moved, never computed on (INPUT -> OUTPUT).
            if (op.kind != PYC_IR_OP_INPUT && op.kind != PYC_IR_OP_OUTPUT) return 1;
            if (dtype_size(v.dtype) == 0) return 1;
        }
        v.elems = v.rank ? 1 : 0;
        for (size_t d = 0; d < v.rank; ++d) { if (v.dims[d] <= 0) return -1; v.elems *= static_cast<size_t>(v.dims[d]); }
        v.bytes = v.elems * dtype_size(v.dtype);
        if (v.elems == 0) return -1;
        if (op.kind == PYC_IR_OP_INPUT && inputs[v.ext].size_bytes < v.bytes) return -1;
    }

    // Pass 2: steps.  Host inputs are staged into arena temps first.
    std::vector<Step>& S = plan->steps;
    plan->all_device = true;
    for (size_t i = 0; i < n; ++i) {
        if (m->ops[i].kind != PYC_IR_OP_INPUT) continue;
        Value& v = V[i];
        if (in_mem[v.ext] == MEM_DEVICE) { v.kind = V_INPUT_DIRECT; continue; }
        plan->all_device = false;
        v.kind = V_TEMP;
        // static_mask only pins lifetimes (pass 3); whether an upload is dropped is decided by the caller per run.
        Step s; s.kind = S_H2D; s.out = static_cast<int>(i); s.ext = v.ext; s.bytes = v.bytes; s.op_main = static_cast<int>(i);
        s.via_stage = in_mem[v.ext] == MEM_PAGEABLE;
        if (s.via_stage) { s.stage_off = plan->stage_bytes; plan->stage_bytes = align_up(plan->stage_bytes + v.bytes, 256); }
        S.push_back(s);
    }
    std::vector<char> done(n, 0);
    for (size_t i = 0; i < n; ++i) {
        const pyc_ir_op& op = m->ops[i];
        if (done[i] || op.kind == PYC_IR_OP_INPUT) continue;
        // Follow a single-consumer chain: returns the consumer op id or -1.
        auto sole_consumer = [&](int id) -> int {
            if (V[id].consumers != 1) return -1;
            for (size_t c = id + 1; c < n; ++c)
                for (size_t j = 0; j < m->ops[c].input_count; ++j)
                    if (m->ops[c].input_ids[j] == id) return static_cast<int>(c);
            return -1;
        };
        auto try_fuse_act = [&](int cur, Step& s) -> int {
            const int c = sole_consumer(cur);
            if (c >= 0 && (m->ops[c].kind == PYC_IR_OP_RELU || m->ops[c].kind == PYC_IR_OP_GELU)) {
                s.act = m->ops[c].kind == PYC_IR_OP_RELU ? PYC_B200_ACT_RELU : PYC_B200_ACT_GELU;
                s.op_act = c;
                V[cur].kind = V_ALIAS; V[cur].alias_of = c; done[c] = 1;
                return c;
            }
            return cur;
        };
        auto classify_add = [&](const Value& big, const Value& small) -> int {
            if (small.elems == big.elems) return PYC_B200_ADD_MATRIX;
            if (small.elems == 1) return PYC_B200_ADD_SCALAR;
            if (big.rank >= 1 && small.elems == static_cast<size_t>(big.dims[big.rank - 1])) return PYC_B200_ADD_ROW_BIAS;
            return -1;
        };
        switch (op.kind) {
            case PYC_IR_OP_MATMUL: {
                Step s; s.kind = S_GEMM; s.in0 = op.input_ids[0]; s.in1 = op.input_ids[1]; s.op_main = static_cast<int>(i);
                s.M = static_cast<int>(V[i].dims[0]); s.N = static_cast<int>(V[i].dims[1]); s.K = static_cast<int>(V[s.in0].dims[1]);
                int cur = static_cast<int>(i);
                const int c = sole_consumer(cur);
                if (c >= 0 && m->ops[c].kind == PYC_IR_OP_ADD) {
                    const int other = m->ops[c].input_ids[0] == cur ? m->ops[c].input_ids[1] : m->ops[c].input_ids[0];
                    const bool ready = other != cur && (m->ops[other].kind == PYC_IR_OP_INPUT || static_cast<size_t>(other) < i);
                    const int mode = ready ? classify_add(V[cur], V[other]) : -1;
                    if (mode > 0 && V[other].elems <= V[cur].elems) {
                        s.add_mode = mode; s.in2 = other; s.op_add = c;
                        V[cur].kind = V_ALIAS; V[cur].alias_of = c; done[c] = 1;
                        cur = c;
                    }
                }
                cur = try_fuse_act(cur, s);
                s.out = cur; V[cur].kind = V_TEMP;
                S.push_back(s);
                break;
            }
            case PYC_IR_OP_ADD: {
                const int a = op.input_ids[0], b = op.input_ids[1];
                const int big = V[a].elems >= V[b].elems ? a : b, small = big == a ? b : a;
                const int mode = classify_add(V[big], V[small]);
                if (mode < 0) return 1;
                Step s; s.in0 = big; s.in1 = small; s.op_main = static_cast<int>(i);
                int cur = static_cast<int>(i);
                s.cols = static_cast<size_t>(V[big].dims[V[big].rank - 1]); s.rows = V[big].elems / s.cols;
                s.kind = S_BIAS_ACT; s.add_mode = mode;
                cur = try_fuse_act(cur, s);
                if (mode == PYC_B200_ADD_MATRIX && s.act == PYC_B200_ACT_NONE) s.kind = S_ADD;
                s.out = cur; V[cur].kind = V_TEMP;
                S.push_back(s);
                break;
            }
            case PYC_IR_OP_RELU: case PYC_IR_OP_GELU: {
                Step s; s.kind = S_BIAS_ACT; s.in0 = op.input_ids[0]; s.add_mode = PYC_B200_ADD_NONE; s.op_main = static_cast<int>(i);
                s.act = op.kind == PYC_IR_OP_RELU ? PYC_B200_ACT_RELU : PYC_B200_ACT_GELU;
                s.cols = static_cast<size_t>(V[i].dims[V[i].rank - 1]); s.rows = V[i].elems / s.cols;
                s.out = static_cast<int>(i); V[i].kind = V_TEMP;
                S.push_back(s);
                break;
            }
            case PYC_IR_OP_LAYERNORM: {
                Step s; s.kind = S_LAYERNORM; s.in0 = op.input_ids[0]; s.op_main = static_cast<int>(i);
                s.in1 = op.input_count > 1 ? op.input_ids[1] : -1; s.in2 = op.input_count > 2 ? op.input_ids[2] : -1;
                s.cols = static_cast<size_t>(V[i].dims[V[i].rank - 1]); s.rows = V[i].elems / s.cols;
                if (s.in1 >= 0 && V[s.in1].elems != s.cols) return 1;
                if (s.in2 >= 0 && V[s.in2].elems != s.cols) return 1;
                s.out = static_cast<int>(i); V[i].kind = V_TEMP;
                S.push_back(s);
                break;
            }
            case PYC_IR_OP_REDUCE_SUM: {
                const Value& a = V[op.input_ids[0]];
                Step xs;
                const ExtOp ext = parse_extended_op(op.name, xs.xp);
                if (ext != EXT_NONE) {
                    xs.op_main = static_cast<int>(i); xs.out = static_cast<int>(i); V[i].kind = V_TEMP;
                    xs.in0 = op.input_ids[0];
                    xs.in1 = op.input_count > 1 ? op.input_ids[1] : -1; xs.in2 = op.input_count > 2 ? op.input_ids[2] : -1;
                    xs.in3 = op.input_count > 3 ? op.input_ids[3] : -1; xs.in4 = op.input_count > 4 ? op.input_ids[4] : -1;
                    const Value& o = V[i];
                    if (ext == EXT_SOFTMAX) {
                        if (o.elems != a.elems || a.rank < 1) return 1;
                        xs.kind = S_SOFTMAX; xs.cols = static_cast<size_t>(a.dims[a.rank - 1]); xs.rows = a.elems / xs.cols;
                    } else if (ext == EXT_ATTENTION) {
                        if (op.input_count < 3 || a.rank < 2) return -1;
                        const Value &kk = V[xs.in1], &vv = V[xs.in2];
                        if (kk.elems != a.elems || vv.elems != a.elems || o.elems != a.elems || kk.dtype != a.dtype || vv.dtype != a.dtype) return 1;
                        xs.kind = S_ATTENTION;
                        xs.xp[1] = static_cast<int>(a.dims[a.rank - 2]); xs.xp[2] = static_cast<int>(a.dims[a.rank - 1]);
                        xs.xp[3] = static_cast<int>(a.elems / (static_cast<size_t>(xs.xp[1]) * xs.xp[2]));     // batch * heads
                    } else if (ext == EXT_CONV2D) {
                        if (op.input_count < 2 || a.rank != 4 || V[xs.in1].rank != 4 || o.rank != 4) return -1;
                        const Value& w = V[xs.in1];
                        if (w.dims[3] != a.dims[3] || w.dtype != a.dtype) return 1;
                        const int P = (static_cast<int>(a.dims[1]) - static_cast<int>(w.dims[1]) + 2 * xs.xp[0]) / xs.xp[2] + 1;
                        const int Q = (static_cast<int>(a.dims[2]) - static_cast<int>(w.dims[2]) + 2 * xs.xp[1]) / xs.xp[3] + 1;
                        if (o.dims[0] != a.dims[0] || o.dims[1] != P || o.dims[2] != Q || o.dims[3] != w.dims[0]) return -1;
                        if (xs.in2 >= 0 && V[xs.in2].elems != static_cast<size_t>(w.dims[0])) return 1;
                        xs.kind = S_CONV2D;
                        xs.xp[5] = static_cast<int>(a.dims[0]); xs.xp[6] = static_cast<int>(a.dims[1]); xs.xp[7] = static_cast<int>(a.dims[2]);
                        xs.xp[8] = static_cast<int>(a.dims[3]); xs.xp[9] = static_cast<int>(w.dims[0]); xs.xp[10] = static_cast<int>(w.dims[1]);
                        xs.xp[11] = static_cast<int>(w.dims[2]);
                    } else {   // EXT_FFN_FP8
                        if (op.input_count < 5 || a.rank != 2 || a.dtype != PYC_DTYPE_BF16) return 1;
                        const Value &w1 = V[xs.in1], &s1 = V[xs.in2], &w2 = V[xs.in3], &s2 = V[xs.in4];
                        if (w1.rank != 2 || w2.rank != 2 || w1.dtype != PYC_DTYPE_I8 || w2.dtype != PYC_DTYPE_I8 || s1.dtype != PYC_DTYPE_F32 ||
                            s2.dtype != PYC_DTYPE_F32 || w1.dims[0] != a.dims[1] || w2.dims[0] != w1.dims[1] || w2.dims[1] != a.dims[1] ||
                            s1.elems != static_cast<size_t>(w1.dims[1]) || s2.elems != static_cast<size_t>(a.dims[1]) || o.elems != a.elems) return 1;
                        xs.kind = S_FFN_FP8;
                        xs.xp[0] = static_cast<int>(a.dims[0]); xs.xp[1] = static_cast<int>(a.dims[1]); xs.xp[2] = static_cast<int>(w1.dims[1]);
                        Value ws; ws.kind = V_TEMP; ws.dtype = PYC_DTYPE_I8; ws.rank = 1;
                        ws.bytes = pyc_b200_ffn_workspace_bytes(xs.xp[0], xs.xp[1], xs.xp[2]); ws.elems = ws.bytes; ws.dims[0] = static_cast<int64_t>(ws.bytes);
                        xs.scratch = static_cast<int>(V.size());
                        V.push_back(ws);                      // invalidates references into V: none is used below
                    }
                    S.push_back(xs);
                    break;
                }
                if (a.elems % V[i].elems) return 1;
                Step s; s.kind = S_REDUCE_SUM; s.in0 = op.input_ids[0]; s.rows = V[i].elems; s.cols = a.elems / V[i].elems; s.op_main = static_cast<int>(i);
                s.out = static_cast<int>(i); V[i].kind = V_TEMP;
                S.push_back(s);
                break;
            }
            case PYC_IR_OP_OUTPUT: {
                if (out_i >= n_out || !outputs[out_i].data) return -1;
                const int o = static_cast<int>(out_i++);
                const int src = resolve(V, op.input_ids[0]);
                if (outputs[o].size_bytes < V[src].bytes) return -1;
                V[i].kind = V_ALIAS; V[i].alias_of = src; V[i].ext = o;
                if (out_mem[o] != MEM_DEVICE) plan->all_device = false;
                if (V[src].kind == V_TEMP && V[src].consumers == 1 && out_mem[o] == MEM_DEVICE && m->ops[src].kind != PYC_IR_OP_INPUT) {
                    V[src].kind = V_OUTPUT_DIRECT; V[src].ext = o;  // the producing kernel writes the caller's buffer
                } else if (out_mem[o] == MEM_DEVICE) {
                    Step s; s.kind = S_COPY; s.in0 = src; s.ext = o; s.bytes = V[src].bytes; s.op_main = static_cast<int>(i);
                    S.push_back(s);
                } else if (!skip_out_copy) {
                    Step s; s.kind = S_D2H; s.in0 = src; s.ext = o; s.bytes = V[src].bytes; s.op_main = static_cast<int>(i);
                    s.via_stage = out_mem[o] == MEM_PAGEABLE;
                    if (s.via_stage) { s.stage_off = plan->stage_bytes; plan->stage_bytes = align_up(plan->stage_bytes + s.bytes, 256); }
                    S.push_back(s);
                }
                break;
            }
            default:
                return 1;
        }
        done[i] = 1;
    }
    if (out_i != n_out && n_out > out_i) { /* extra caller outputs are left untouched */ }

    // Pass 3: lifetimes over step indices, then first-fit placement in request order
    // (runtime_allocator.c:123-187: reuse the first earlier slot that is large enough and
    // has no live tenant; otherwise bump the peak).
    for (size_t si = 0; si < S.size(); ++si) {
        const Step& s = S[si];
        const int ids[7] = {s.out, s.in0 >= 0 ? resolve(V, s.in0) : -1, s.in1 >= 0 ? resolve(V, s.in1) : -1, s.in2 >= 0 ? resolve(V, s.in2) : -1,
                            s.in3 >= 0 ? resolve(V, s.in3) : -1, s.in4 >= 0 ? resolve(V, s.in4) : -1, s.scratch};
        for (int id : ids) {
            if (id < 0 || V[id].kind != V_TEMP) continue;
            if (V[id].def_step < 0) V[id].def_step = static_cast<int>(si);
            V[id].last_step = static_cast<int>(si);
        }
    }
    struct Req { int id; size_t bytes, off; int a, b; };
    std::vector<Req> reqs;
    for (size_t i = 0; i < V.size(); ++i) {       // the IR ops' values, then the step-private workspaces
        Value& v = V[i];
        if (v.kind != V_TEMP) continue;
        if (v.def_step < 0) { v.def_step = 0; v.last_step = static_cast<int>(S.size()); }
        // Inputs whose upload is skipped (assume-static) must survive between runs: pin them for the whole plan.
        if (i < n && m->ops[i].kind == PYC_IR_OP_INPUT && static_mask) { v.def_step = 0; v.last_step = static_cast<int>(S.size()); }
        reqs.push_back({static_cast<int>(i), v.bytes, 0, v.def_step, v.last_step});
    }
    size_t peak = 0, total = 0;
    for (size_t i = 0; i < reqs.size(); ++i) {
        Req& cur = reqs[i];
        total += cur.bytes;
        bool placed = false;
        for (size_t j = 0; j < i && !placed; ++j) {
            if (reqs[j].bytes < cur.bytes) continue;
            bool conflict = false;
            for (size_t k = 0; k < i; ++k)
                if (reqs[k].off == reqs[j].off && !(reqs[k].b < cur.a || cur.b < reqs[k].a)) { conflict = true; break; }
            if (!conflict) { cur.off = reqs[j].off; placed = true; }
        }
        if (!placed) { cur.off = align_up(peak, 1024); peak = cur.off + cur.bytes; }
        V[cur.id].arena_off = cur.off;
    }
    plan->arena_peak = peak;
    plan->arena_total = total;
    return 0;
}

// A call whose tensors live in pinned host memory is bound by the PCIe copies, not by the kernel: for the
// common shape "upload operands, one (fused) GEMM, download the result" the rows of A are uploaded in chunks,
// each chunk's GEMM starts as soon as its rows have landed, and its rows of the result go back while the next
// chunk is still arriving.  Uploads, kernels and downloads sit on three streams joined by events, so the same
// enqueue works under stream capture (the graph gets three parallel branches) and on a plain stream.
// Recognised here; anything else keeps the serial order.
void plan_pipeline(Plan* plan) {
    plan->pipe_gemm = -1;
    const std::vector<Step>& S = plan->steps;
    int g = -1;
    for (size_t i = 0; i < S.size(); ++i)
        if (S[i].kind == S_GEMM) { if (g >= 0) return; g = static_cast<int>(i); }
    if (g < 0 || g + 2 != static_cast<int>(S.size())) return;
    const Step& gemm = S[g];
    const Step& down = S[g + 1];
    const int a = resolve(plan->values, gemm.in0), d = resolve(plan->values, gemm.out);
    if (down.kind != S_D2H || down.via_stage || resolve(plan->values, down.in0) != d) return;
    if (resolve(plan->values, gemm.in1) == a || (gemm.in2 >= 0 && resolve(plan->values, gemm.in2) == a)) return;
    bool a_uploaded = false;
    for (int i = 0; i < g; ++i) {
        if (S[i].kind != S_H2D) return;
        if (resolve(plan->values, S[i].out) == a) { if (S[i].via_stage) return; a_uploaded = true; }
    }
    if (!a_uploaded) return;
    const size_t moved = plan->values[a].bytes + plan->values[d].bytes;
    if (gemm.M < 1024 || moved < (size_t(32) << 20)) return;
    // Whole 256-row tiles, about eight chunks; PYC_B200_PIPELINE_CHUNKS asks for another count (2..64): more, smaller
    // chunks help when several processes share one host's PCIe root and memory system.
    int want_chunks = 8;
    if (const char* e = getenv("PYC_B200_PIPELINE_CHUNKS")) { const int v = atoi(e); if (v >= 2 && v <= 64) want_chunks = v; }
    int rows = (gemm.M / want_chunks + 255) / 256 * 256;
    plan->pipe_gemm = g;
    plan->pipe_rows = rows;
    plan->pipe_chunks = (gemm.M + rows - 1) / rows;
}

void* value_ptr(const Plan& plan, const DeviceContext* ctx, const pyc_tensor* inputs, pyc_tensor* outputs, int id) {
    id = resolve(plan.values, id);
    const Value& v = plan.values[id];
    switch (v.kind) {
        case V_INPUT_DIRECT: return inputs[v.ext].data;
        case V_OUTPUT_DIRECT: return outputs[v.ext].data;
        case V_TEMP: return static_cast<char*>(ctx->arena) + v.arena_off;
        default: return nullptr;
    }
}

// The pipelined order of plan_pipeline().  Every side stream is forked from and joined back into `stream`.
int enqueue_pipelined(Plan& plan, DeviceContext* ctx, const pyc_tensor* inputs, pyc_tensor* outputs, cudaStream_t stream, size_t* kernels) {
    const Step& gemm = plan.steps[plan.pipe_gemm];
    const Step& down = plan.steps[plan.pipe_gemm + 1];
    const int chunks = plan.pipe_chunks, rows = plan.pipe_rows;
    if (ctx->ensure_pipeline(static_cast<size_t>(2 * chunks + 3)) != 0) return -1;
    cudaEvent_t* ev = ctx->events.data();   // 0 fork, 1 shared operands landed, 2 downloads done, 3.. A chunks, 3+chunks.. D chunks
    const int a_id = resolve(plan.values, gemm.in0);
    const pyc_dtype dt = plan.values[resolve(plan.values, gemm.out)].dtype;
    const size_t es = dtype_size(dt);
    B200_CUDA_OK(cudaEventRecord(ev[0], stream));
    B200_CUDA_OK(cudaStreamWaitEvent(ctx->copy_in, ev[0], 0));
    B200_CUDA_OK(cudaStreamWaitEvent(ctx->copy_out, ev[0], 0));
    const char* a_host = nullptr;
    for (int i = 0; i < plan.pipe_gemm; ++i) {
        const Step& s = plan.steps[i];
        if (resolve(plan.values, s.out) == a_id) { a_host = static_cast<const char*>(inputs[s.ext].data); continue; }
        const void* src = s.via_stage ? static_cast<const void*>(static_cast<char*>(ctx->pinned) + s.stage_off) : inputs[s.ext].data;
        B200_CUDA_OK(cudaMemcpyAsync(value_ptr(plan, ctx, inputs, outputs, s.out), src, s.bytes, cudaMemcpyHostToDevice, ctx->copy_in));
    }
    B200_CUDA_OK(cudaEventRecord(ev[1], ctx->copy_in));
    B200_CUDA_OK(cudaStreamWaitEvent(stream, ev[1], 0));
    char* a_dev = static_cast<char*>(value_ptr(plan, ctx, inputs, outputs, gemm.in0));
    char* d_dev = static_cast<char*>(value_ptr(plan, ctx, inputs, outputs, gemm.out));
    char* d_host = static_cast<char*>(outputs[down.ext].data);
    const char* add = gemm.in2 >= 0 ? static_cast<const char*>(value_ptr(plan, ctx, inputs, outputs, gemm.in2)) : nullptr;
    for (int c = 0; c < chunks; ++c) {
        const size_t r0 = static_cast<size_t>(c) * rows;
        const size_t rc = std::min<size_t>(rows, gemm.M - r0);
        const size_t a_off = r0 * gemm.K * es, d_off = r0 * gemm.N * es;
        B200_CUDA_OK(cudaMemcpyAsync(a_dev + a_off, a_host + a_off, rc * gemm.K * es, cudaMemcpyHostToDevice, ctx->copy_in));
        B200_CUDA_OK(cudaEventRecord(ev[3 + c], ctx->copy_in));
        B200_CUDA_OK(cudaStreamWaitEvent(stream, ev[3 + c], 0));
        GemmProblem p;
        p.dtype = dt;
        p.M = static_cast<int>(rc); p.N = gemm.N; p.K = gemm.K;
        p.A = a_dev + a_off; p.B = value_ptr(plan, ctx, inputs, outputs, gemm.in1); p.D = d_dev + d_off;
        p.add_mode = gemm.add_mode; p.act = gemm.act;
        p.add = add ? (gemm.add_mode == PYC_B200_ADD_MATRIX ? add + d_off : add) : nullptr;
        const GemmConfig* cfg = choose_gemm_config(p);
        if (!cfg) { set_error("no GEMM configuration for %zux%dx%d", rc, gemm.N, gemm.K); return -1; }
        if (plan.symbol.empty()) plan.symbol = gemm_symbol(dt, *cfg);
        if (c == 0) { plan.steps[plan.pipe_gemm].symbol = gemm_symbol(dt, *cfg); plan.steps[plan.pipe_gemm].chosen_by = last_selection_source(); }
        if (launch_gemm(*cfg, p, stream) != 0) return -1;
        ++*kernels;
        B200_CUDA_OK(cudaEventRecord(ev[3 + chunks + c], stream));
        B200_CUDA_OK(cudaStreamWaitEvent(ctx->copy_out, ev[3 + chunks + c], 0));
        B200_CUDA_OK(cudaMemcpyAsync(d_host + d_off, d_dev + d_off, rc * gemm.N * es, cudaMemcpyDeviceToHost, ctx->copy_out));
    }
    B200_CUDA_OK(cudaEventRecord(ev[2], ctx->copy_out));
    B200_CUDA_OK(cudaStreamWaitEvent(stream, ev[2], 0));
    return 0;
}

// Enqueue every step on `stream` (which may be capturing).
int enqueue_plan(Plan& plan, DeviceContext* ctx, const pyc_tensor* inputs, pyc_tensor* outputs, cudaStream_t stream, size_t* kernels) {
    *kernels = 0;
    if (plan.pipe_gemm >= 0) {
        if (enqueue_pipelined(plan, ctx, inputs, outputs, stream, kernels) != 0) return -1;
        B200_CUDA_OK(cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, stream));
        return 0;
    }
    for (Step& s : plan.steps) {
        switch (s.kind) {
            case S_H2D: {
                const void* src = s.via_stage ? static_cast<const void*>(static_cast<char*>(ctx->pinned) + s.stage_off) : inputs[s.ext].data;
                B200_CUDA_OK(cudaMemcpyAsync(value_ptr(plan, ctx, inputs, outputs, s.out), src, s.bytes, cudaMemcpyHostToDevice, stream));
                break;
            }
            case S_D2H: {
                void* dst = s.via_stage ? static_cast<void*>(static_cast<char*>(ctx->pinned) + s.stage_off) : outputs[s.ext].data;
                B200_CUDA_OK(cudaMemcpyAsync(dst, value_ptr(plan, ctx, inputs, outputs, s.in0), s.bytes, cudaMemcpyDeviceToHost, stream));
                break;
            }
            case S_COPY:
                B200_CUDA_OK(cudaMemcpyAsync(outputs[s.ext].data, value_ptr(plan, ctx, inputs, outputs, s.in0), s.bytes, cudaMemcpyDefault, stream));
                break;
            case S_GEMM: {
                GemmProblem p;
                p.dtype = plan.values[resolve(plan.values, s.out)].dtype;
                p.M = s.M; p.N = s.N; p.K = s.K;
                p.A = value_ptr(plan, ctx, inputs, outputs, s.in0);
                p.B = value_ptr(plan, ctx, inputs, outputs, s.in1);
                p.D = value_ptr(plan, ctx, inputs, outputs, s.out);
                p.add_mode = s.add_mode; p.add = s.in2 >= 0 ? value_ptr(plan, ctx, inputs, outputs, s.in2) : nullptr; p.act = s.act;
                const GemmConfig* cfg = choose_gemm_config(p);
                if (!cfg) { set_error("no GEMM configuration for %dx%dx%d", s.M, s.N, s.K); return -1; }
                if (plan.symbol.empty()) plan.symbol = gemm_symbol(p.dtype, *cfg);
                s.symbol = gemm_symbol(p.dtype, *cfg); s.chosen_by = last_selection_source();
                if (launch_gemm(*cfg, p, stream) != 0) return -1;
                ++*kernels;
                break;
            }
            case S_ADD:
                if (launch_add(plan.values[s.out].dtype, value_ptr(plan, ctx, inputs, outputs, s.in0), value_ptr(plan, ctx, inputs, outputs, s.in1),
                               value_ptr(plan, ctx, inputs, outputs, s.out), plan.values[s.out].elems, stream) != 0) return -1;
                ++*kernels;
                break;
            case S_BIAS_ACT:
                if (launch_bias_act(plan.values[s.out].dtype, value_ptr(plan, ctx, inputs, outputs, s.in0),
                                    s.in1 >= 0 ? value_ptr(plan, ctx, inputs, outputs, s.in1) : nullptr, s.add_mode, s.act,
                                    value_ptr(plan, ctx, inputs, outputs, s.out), s.rows, s.cols, stream) != 0) return -1;
                ++*kernels;
                break;
            case S_LAYERNORM:
                if (launch_layernorm(plan.values[s.out].dtype, value_ptr(plan, ctx, inputs, outputs, s.in0),
                                     s.in1 >= 0 ? value_ptr(plan, ctx, inputs, outputs, s.in1) : nullptr,
                                     s.in2 >= 0 ? value_ptr(plan, ctx, inputs, outputs, s.in2) : nullptr,
                                     value_ptr(plan, ctx, inputs, outputs, s.out), s.rows, s.cols, 1e-5f, stream) != 0) return -1;
                ++*kernels;
                break;
            case S_SOFTMAX:
                if (launch_softmax(plan.values[s.out].dtype, value_ptr(plan, ctx, inputs, outputs, s.in0), value_ptr(plan, ctx, inputs, outputs, s.out),
                                   s.rows, s.cols, stream) != 0) return -1;
                s.symbol = std::string("b200_softmax_") + (plan.values[s.out].dtype == PYC_DTYPE_F32 ? "f32" : plan.values[s.out].dtype == PYC_DTYPE_BF16 ? "bf16" : "f16");
                ++*kernels;
                break;
            case S_ATTENTION: {
                const pyc_dtype dt = plan.values[s.out].dtype;
                if (launch_attention(dt, s.xp[3], s.xp[1], s.xp[2], value_ptr(plan, ctx, inputs, outputs, s.in0), value_ptr(plan, ctx, inputs, outputs, s.in1),
                                     value_ptr(plan, ctx, inputs, outputs, s.in2), value_ptr(plan, ctx, inputs, outputs, s.out),
                                     1.0f / sqrtf(static_cast<float>(s.xp[2])), s.xp[0], stream, ctx->status_dev) != 0) return -1;
                s.symbol = std::string("b200_attention_") + (dt == PYC_DTYPE_F32 ? "f32" : dt == PYC_DTYPE_BF16 ? "bf16" : "f16") + (s.xp[0] ? "_causal" : "");
                ++*kernels;
                break;
            }
            case S_CONV2D: {
                const pyc_dtype dt = plan.values[s.out].dtype;
                if (launch_conv2d(dt, s.xp[5], s.xp[6], s.xp[7], s.xp[8], s.xp[9], s.xp[10], s.xp[11], s.xp[0], s.xp[1], s.xp[2], s.xp[3],
                                  value_ptr(plan, ctx, inputs, outputs, s.in0), value_ptr(plan, ctx, inputs, outputs, s.in1),
                                  s.in2 >= 0 ? value_ptr(plan, ctx, inputs, outputs, s.in2) : nullptr, s.xp[4], value_ptr(plan, ctx, inputs, outputs, s.out),
                                  stream, ctx->status_dev) != 0) return -1;
                s.symbol = std::string("b200_conv2d_fprop_") + (dt == PYC_DTYPE_F32 ? "f32" : dt == PYC_DTYPE_BF16 ? "bf16" : "f16");
                ++*kernels;
                break;
            }
            case S_FFN_FP8: {
                pyc_b200_ffn_args a;
                memset(&a, 0, sizeof(a));
                a.tokens = s.xp[0]; a.hidden = s.xp[1]; a.inner = s.xp[2];
                a.x = value_ptr(plan, ctx, inputs, outputs, s.in0);
                a.w1 = value_ptr(plan, ctx, inputs, outputs, s.in1); a.w1_scale = static_cast<const float*>(value_ptr(plan, ctx, inputs, outputs, s.in2));
                a.w2 = value_ptr(plan, ctx, inputs, outputs, s.in3); a.w2_scale = static_cast<const float*>(value_ptr(plan, ctx, inputs, outputs, s.in4));
                a.out = value_ptr(plan, ctx, inputs, outputs, s.out);
                if (pyc_b200_ffn_block(&a, value_ptr(plan, ctx, inputs, outputs, s.scratch), plan.values[s.scratch].bytes, stream) != 0) return -1;
                s.symbol = "b200_ffn_fp8_block";
                *kernels += 4;
                break;
            }
            case S_REDUCE_SUM:
                if (launch_reduce_sum(plan.values[s.out].dtype, value_ptr(plan, ctx, inputs, outputs, s.in0),
                                      value_ptr(plan, ctx, inputs, outputs, s.out), s.rows, s.cols, stream) != 0) return -1;
                ++*kernels;
                break;
        }
    }
    // Status word back to its pinned mirror at the end of every run.
    B200_CUDA_OK(cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, stream));
    return 0;
}

// ---- what ran: the sidecar plan ---------------------------------------------------------------------------------
// PyC's own fusion pass is lossy (pass_manager.c:241-267 renames ops to "matmul_fused" and drops the epilogue) and its
// kernel catalog for that key holds placeholders (compiler_api.c:2094-2122), so pyc_run_stats.selected_kernel_symbol
// cannot name the kernel that ran.  The backend therefore keeps, per module content, a text plan: one line per step with
// the kernel symbol, who chose it, and the IR ops the step absorbed.  pyc_b200_last_plan() returns it.
const char* kind_name(pyc_ir_op_kind k) {
    switch (k) {
        case PYC_IR_OP_INPUT: return "input"; case PYC_IR_OP_CONST: return "const"; case PYC_IR_OP_MATMUL: return "matmul";
        case PYC_IR_OP_ADD: return "add"; case PYC_IR_OP_RELU: return "relu"; case PYC_IR_OP_GELU: return "gelu";
        case PYC_IR_OP_REDUCE_SUM: return "reduce_sum"; case PYC_IR_OP_LAYERNORM: return "layernorm"; case PYC_IR_OP_OUTPUT: return "output";
        default: return "op";
    }
}
const char* dtype_name(pyc_dtype d) { return d == PYC_DTYPE_F32 ? "f32" : d == PYC_DTYPE_BF16 ? "bf16" : d == PYC_DTYPE_F16 ? "f16" : "raw"; }

uint64_t module_content_hash(const pyc_ir_module* module) {
    uint64_t h = 1469598103934665603ull;
    h = fnv1a(h, &module->op_count, sizeof(module->op_count));
    for (size_t i = 0; i < module->op_count; ++i) {
        const pyc_ir_op& op = module->ops[i];
        h = fnv1a(h, &op.kind, sizeof(op.kind));
        h = fnv1a(h, &op.dtype, sizeof(op.dtype));
        h = fnv1a(h, &op.shape.rank, sizeof(op.shape.rank));
        h = fnv1a(h, op.shape.dims, sizeof(int64_t) * op.shape.rank);
        h = fnv1a(h, &op.input_count, sizeof(op.input_count));
        h = fnv1a(h, op.input_ids, sizeof(int) * op.input_count);
    }
    return h;
}

std::string describe_plan(const Plan& plan, const pyc_ir_module* m) {
    std::string out;
    char buf[320];
    auto op_ref = [&](int id) { char b[96]; snprintf(b, sizeof(b), "%s#%d", kind_name(m->ops[id].kind), id); return std::string(b); };
    for (size_t si = 0; si < plan.steps.size(); ++si) {
        const Step& s = plan.steps[si];
        std::string kernel, ops = s.op_main >= 0 ? op_ref(s.op_main) : std::string("?");
        const pyc_dtype dt = s.out >= 0 ? plan.values[resolve(plan.values, s.out)].dtype : (s.in0 >= 0 ? plan.values[resolve(plan.values, s.in0)].dtype : PYC_DTYPE_UNKNOWN);
        switch (s.kind) {
            case S_H2D: kernel = "copy_h2d"; break;
            case S_D2H: kernel = "copy_d2h"; break;
            case S_COPY: kernel = "copy_d2d"; break;
            case S_GEMM: kernel = s.symbol.empty() ? std::string("b200_gemm_") + dtype_name(dt) : s.symbol; break;
            case S_ADD: kernel = std::string("b200_add_") + dtype_name(dt); break;
            case S_BIAS_ACT: kernel = std::string("b200_bias_act_") + dtype_name(dt); break;
            case S_LAYERNORM: kernel = std::string("b200_layernorm_") + dtype_name(dt); break;
            case S_REDUCE_SUM: kernel = std::string("b200_reduce_sum_") + dtype_name(dt); break;
            case S_SOFTMAX: case S_ATTENTION: case S_CONV2D: case S_FFN_FP8: kernel = s.symbol; break;
        }
        if (s.op_add >= 0) ops += " + " + op_ref(s.op_add);
        if (s.op_act >= 0) ops += " + " + op_ref(s.op_act);
        if (s.kind == S_GEMM && (int)si == plan.pipe_gemm && plan.pipe_chunks > 1) { snprintf(buf, sizeof(buf), " x%d row chunks", plan.pipe_chunks); ops += buf; }
        snprintf(buf, sizeof(buf), "step %zu: %s%s%s%s <- %s\n", si, kernel.c_str(), s.chosen_by.empty() ? "" : " [", s.chosen_by.c_str(),
                 s.chosen_by.empty() ? "" : "]", ops.c_str());
        out += buf;
    }
    return out;
}

std::mutex g_plan_table_mu;
std::map<uint64_t, std::string> g_plan_table;   // module content hash -> plan text of its most recent run
std::string g_last_plan_text;

void publish_plan(const Plan& plan) {
    std::lock_guard<std::mutex> lk(g_plan_table_mu);
    if (g_plan_table.size() >= 256 && !g_plan_table.count(plan.module_hash)) g_plan_table.clear();
    g_plan_table[plan.module_hash] = plan.description;
    g_last_plan_text = plan.description;
}

// 0 = ran, 1 = unsupported module (fall back), -1 = error.
int run_on_gpu(const pyc_ir_module* module, const pyc_tensor* inputs, size_t n_in, pyc_tensor* outputs, size_t n_out,
               pyc_cuda_dispatch_trace* trace, char* reason, size_t reason_size) {
    DeviceContext* ctx = current_context();
    if (!ctx) { snprintf(reason, reason_size, "b200_no_context"); return -1; }
    if (ctx->cc_major != 10) { snprintf(reason, reason_size, "b200_requires_sm100_found_sm%d%d", ctx->cc_major, ctx->cc_minor); return 1; }
    std::lock_guard<std::mutex> lk(ctx->mu);

    std::vector<MemKind> in_mem(n_in), out_mem(n_out);
    for (size_t i = 0; i < n_in; ++i) in_mem[i] = inputs[i].data ? classify_pointer(inputs[i].data) : MEM_PAGEABLE;
    for (size_t i = 0; i < n_out; ++i) out_mem[i] = outputs[i].data ? classify_pointer(outputs[i].data) : MEM_PAGEABLE;
    const bool skip_out = env_true("PYC_CUDA_SKIP_HOST_OUTPUT_COPY");
    const bool replay_enabled = env_default_true("PYC_CUDA_ENABLE_GRAPH_REPLAY");

    // Key: module content + tensor descriptors + switches.
    // Two independent 64-bit hashes of the same key material: `base` indexes the cache, `check` is stored with the entry and
    // compared on a hit, so a collision of the index cannot replay another call's graph.
    uint64_t base = 1469598103934665603ull, check = 0x84222325cbf29ce4ull;
    { base = fnv1a(base, &module->op_count, sizeof(module->op_count)); check = fnv1a(check * 31 + 7, &module->op_count, sizeof(module->op_count)); }
    for (size_t i = 0; i < module->op_count; ++i) {
        const pyc_ir_op& op = module->ops[i];
        { base = fnv1a(base, &op.kind, sizeof(op.kind)); check = fnv1a(check * 31 + 7, &op.kind, sizeof(op.kind)); }
        { base = fnv1a(base, &op.dtype, sizeof(op.dtype)); check = fnv1a(check * 31 + 7, &op.dtype, sizeof(op.dtype)); }
        { base = fnv1a(base, &op.shape.rank, sizeof(op.shape.rank)); check = fnv1a(check * 31 + 7, &op.shape.rank, sizeof(op.shape.rank)); }
        { base = fnv1a(base, op.shape.dims, sizeof(int64_t) * op.shape.rank); check = fnv1a(check * 31 + 7, op.shape.dims, sizeof(int64_t) * op.shape.rank); }
        { base = fnv1a(base, &op.input_count, sizeof(op.input_count)); check = fnv1a(check * 31 + 7, &op.input_count, sizeof(op.input_count)); }
        { base = fnv1a(base, op.input_ids, sizeof(int) * op.input_count); check = fnv1a(check * 31 + 7, op.input_ids, sizeof(int) * op.input_count); }
    }
    // Tensor descriptors: address, size, where the memory lives, and the dtype/shape the planner reads when the INPUT op
    // itself carries none (two calls that differ only there must not share a plan).
    auto hash_tensor = [&](const pyc_tensor& t, MemKind mk) {
        { base = fnv1a(base, &t.data, sizeof(void*)); check = fnv1a(check * 31 + 7, &t.data, sizeof(void*)); } { base = fnv1a(base, &t.size_bytes, sizeof(size_t)); check = fnv1a(check * 31 + 7, &t.size_bytes, sizeof(size_t)); } { base = fnv1a(base, &mk, sizeof(MemKind)); check = fnv1a(check * 31 + 7, &mk, sizeof(MemKind)); }
        { base = fnv1a(base, &t.dtype, sizeof(t.dtype)); check = fnv1a(check * 31 + 7, &t.dtype, sizeof(t.dtype)); } { base = fnv1a(base, &t.shape.rank, sizeof(t.shape.rank)); check = fnv1a(check * 31 + 7, &t.shape.rank, sizeof(t.shape.rank)); }
        { base = fnv1a(base, t.shape.dims, sizeof(int64_t) * (t.shape.rank <= PYC_IR_MAX_DIMS ? t.shape.rank : PYC_IR_MAX_DIMS)); check = fnv1a(check * 31 + 7, t.shape.dims, sizeof(int64_t) * (t.shape.rank <= PYC_IR_MAX_DIMS ? t.shape.rank : PYC_IR_MAX_DIMS)); }
    };
    for (size_t i = 0; i < n_in; ++i) hash_tensor(inputs[i], in_mem[i]);
    for (size_t i = 0; i < n_out; ++i) hash_tensor(outputs[i], out_mem[i]);
    { base = fnv1a(base, &skip_out, sizeof(skip_out)); check = fnv1a(check * 31 + 7, &skip_out, sizeof(skip_out)); }
    // Switches that change which kernel a captured graph holds.
    for (const char* name : {"PYC_B200_AUTOTUNE", "PYC_B200_GEMM_L2_HINTS", "PYC_B200_GEMM_GROUP_M", "PYC_CUDA_BF16_GEMM_SYMBOL",
                             "PYC_CUDA_ENABLE_PROMOTED_GEMM", "PYC_B200_REGISTRY_SELECT", "PYC_B200_PIPELINE_CHUNKS"}) {
        const char* v = getenv(name);
        { base = fnv1a(base, name, strlen(name)); check = fnv1a(check * 31 + 7, name, strlen(name)); }
        if (v) { base = fnv1a(base, v, strlen(v) + 1); check = fnv1a(check * 31 + 7, v, strlen(v) + 1); }
    }
    {
        const uint64_t epoch = selection_epoch();   // a new autotune winner invalidates graphs captured with the old choice
        { base = fnv1a(base, &epoch, sizeof(epoch)); check = fnv1a(check * 31 + 7, &epoch, sizeof(epoch)); }
        if (!env_is_false_value("PYC_CUDA_ENABLE_PROMOTED_GEMM")) {
            std::string promoted;                   // so does a promotion made through PyC's registry since the capture
            if (registry_promoted_symbol("matmul", &promoted)) { base = fnv1a(base, promoted.data(), promoted.size()); check = fnv1a(check * 31 + 7, promoted.data(), promoted.size()); }
        }
    }
    // PYC_B200_PIPELINE_HOST_COPIES=0 keeps uploads, kernel and downloads strictly one after another.
    const bool pipeline_enabled = env_default_true("PYC_B200_PIPELINE_HOST_COPIES");
    { base = fnv1a(base, &pipeline_enabled, sizeof(pipeline_enabled)); check = fnv1a(check * 31 + 7, &pipeline_enabled, sizeof(pipeline_enabled)); }

    // PYC_CUDA_ASSUME_STATIC_LHS/RHS (cuda_backend.c:2521-2522, 2625-2636): once a host operand has
    // been uploaded for this module and nothing else used the arena since, do not upload it again.
    unsigned want_static = 0;
    if (n_in > 0 && in_mem[0] != MEM_DEVICE && env_true("PYC_CUDA_ASSUME_STATIC_LHS")) want_static |= 1u;
    if (n_in > 1 && in_mem[1] != MEM_DEVICE && env_true("PYC_CUDA_ASSUME_STATIC_RHS")) want_static |= 2u;
    // `pin_mask` keeps static operands alive in the arena for the whole plan; `skip_mask` drops
    // their upload once they are resident (same module + descriptors ran last, with pinning).
    const unsigned pin_mask = want_static;
    const unsigned skip_mask = (want_static && ctx->resident_base == base && ctx->last_base == base) ? want_static : 0u;
    const uint64_t key = base ^ (0x9e3779b97f4a7c15ull * (1 + pin_mask + 4 * skip_mask));

    // A key that already has a captured graph also has its plan: replays skip planning altogether.
    std::shared_ptr<Plan> plan_holder;
    if (replay_enabled) {
        auto hit = ctx->graphs.find(key);
        if (hit != ctx->graphs.end() && hit->second.check != check) { cudaGraphExecDestroy(hit->second.exec); ctx->graphs.erase(hit); hit = ctx->graphs.end(); }
        if (hit != ctx->graphs.end() && hit->second.plan) plan_holder = std::static_pointer_cast<Plan>(hit->second.plan);
    }
    if (!plan_holder) {
        plan_holder = std::make_shared<Plan>();
        // The skip variant is planned with the same pinning so every offset matches the uploading variant.
        const int rc = build_plan(module, inputs, n_in, outputs, n_out, in_mem, out_mem, skip_out, pin_mask, plan_holder.get());
        if (rc != 0) { snprintf(reason, reason_size, rc > 0 ? "b200_unsupported_module" : "b200_bad_arguments"); return rc; }
        if (skip_mask) {
            std::vector<Step> kept;
            for (const Step& s : plan_holder->steps) if (!(s.kind == S_H2D && s.ext < 2 && (skip_mask & (1u << s.ext)))) kept.push_back(s);
            plan_holder->steps.swap(kept);
        }
        if (pipeline_enabled) plan_pipeline(plan_holder.get());
        if (ctx->ensure_arena(plan_holder->arena_peak) != 0 || ctx->ensure_pinned(plan_holder->stage_bytes) != 0) { snprintf(reason, reason_size, "b200_out_of_memory"); return -1; }
        // PYC_B200_AUTOTUNE=1: the first time a GEMM shape is planned, time its tile configurations (outside any capture)
        // and let the measured winner, not the shape heuristic, go into the graph.  Timings also reach PyC's registry.
        if (env_true("PYC_B200_AUTOTUNE")) {
            for (const Step& st : plan_holder->steps)
                if (st.kind == S_GEMM) {
                    const pyc_dtype dt = plan_holder->values[resolve(plan_holder->values, st.out)].dtype;
                    if (!has_gemm_winner(dt, st.M, st.N, st.K)) autotune_gemm_unlocked(ctx, dt, st.M, st.N, st.K, 5, nullptr, nullptr, st.add_mode, st.act);
                }
        }
    }
    Plan& plan = *plan_holder;
    ctx->last_plan_peak = plan.arena_peak;

    // Host -> pinned staging (outside the graph; PyC does the same at cuda_backend.c:551-650).
    double t0 = now_ms();
    for (const Step& s : plan.steps)
        if (s.kind == S_H2D && s.via_stage) memcpy(static_cast<char*>(ctx->pinned) + s.stage_off, inputs[s.ext].data, s.bytes);
    if (trace) trace->copy_in_ms = now_ms() - t0;

    cudaStream_t launch_stream = ctx->active_stream();
    const bool async = ctx->async && plan.all_device;
    size_t kernels = 0;
    bool replayed = false;
    t0 = now_ms();
    if (replay_enabled) {
        auto it = ctx->graphs.find(key);
        if (it == ctx->graphs.end()) {
            if (ctx->graphs.size() >= 64) ctx->drop_graphs();
            cudaGraph_t graph = nullptr;
            CachedGraph cg;
            if (cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
                snprintf(reason, reason_size, "b200_capture_begin_failed:%s", cudaGetErrorString(cudaGetLastError())); return -1;
            }
            const int rc = enqueue_plan(plan, ctx, inputs, outputs, ctx->stream, &kernels);
            const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
            if (rc != 0 || ce != cudaSuccess || !graph) {
                if (graph) cudaGraphDestroy(graph);
                cudaGetLastError();
                snprintf(reason, reason_size, "b200_capture_failed:%.90s", last_error()); return -1;
            }
            const cudaError_t ie = cudaGraphInstantiate(&cg.exec, graph, 0);
            cudaGraphDestroy(graph);
            if (ie != cudaSuccess) { snprintf(reason, reason_size, "b200_graph_instantiate_failed:%s", cudaGetErrorString(ie)); cudaGetLastError(); return -1; }
            cg.kernels = kernels;
            cg.plan = plan_holder;
            cg.check = check;
            it = ctx->graphs.emplace(key, cg).first;
        } else {
            replayed = true;
            kernels = it->second.kernels;
        }
        if (cudaGraphLaunch(it->second.exec, launch_stream) != cudaSuccess) {
            snprintf(reason, reason_size, "b200_graph_launch_failed:%s", cudaGetErrorString(cudaGetLastError())); return -1;
        }
        it->second.replays++;
        ctx->graph_replays++;
        count_launch(replayed ? kernels : 0);  // capture already counted the kernels once
    } else {
        if (enqueue_plan(plan, ctx, inputs, outputs, launch_stream, &kernels) != 0) { snprintf(reason, reason_size, "b200_launch_failed:%.100s", last_error()); return -1; }
    }
    if (plan.description.empty()) { plan.module_hash = module_content_hash(module); plan.description = describe_plan(plan, module); }
    publish_plan(plan);
    ctx->last_graph_kernels = kernels;
    ctx->last_plan_total = plan.arena_total;
    // Until this run is known to have succeeded nothing counts as resident: a failed upload must not be skipped next time.
    ctx->last_base = 0;
    ctx->resident_base = 0;
    if (trace) { trace->kernel_ms = now_ms() - t0; trace->graph_replayed = replayed ? 1 : 0; }

    if (!async) {
        t0 = now_ms();
        const cudaError_t se = cudaStreamSynchronize(launch_stream);
        if (trace) trace->sync_ms = now_ms() - t0;
        if (se != cudaSuccess) { snprintf(reason, reason_size, "b200_sync_failed:%s", cudaGetErrorString(se)); cudaGetLastError(); return -1; }
        if (*ctx->status_host != 0) {
            snprintf(reason, reason_size, "b200_kernel_wait_timeout:0x%x", *ctx->status_host);
            cudaMemsetAsync(ctx->status_dev, 0, sizeof(int), launch_stream);
            cudaStreamSynchronize(launch_stream);
            *ctx->status_host = 0;
            return -1;
        }
        t0 = now_ms();
        for (const Step& s : plan.steps)
            if (s.kind == S_D2H && s.via_stage) memcpy(outputs[s.ext].data, static_cast<char*>(ctx->pinned) + s.stage_off, s.bytes);
        if (trace) trace->copy_out_ms = now_ms() - t0;
    }
    // Success (in async mode: everything was enqueued without error): the static operands of this key are in the arena.
    ctx->last_base = base;
    ctx->resident_base = want_static ? base : 0;
    const char* mode = !replay_enabled ? "b200_stream" : replayed ? "b200_graph_replay" : "b200_graph_capture";
    if (plan.symbol.empty()) snprintf(reason, reason_size, "%s", mode);
    else snprintf(reason, reason_size, "%s:%s", mode, plan.symbol.c_str());
    return 0;
}

int detect_cuda(char* reason, size_t n) {
    if (env_true("PYC_CUDA_DISABLE")) { snprintf(reason, n, "disabled_by_env"); return 0; }
    if (env_true("PYC_CUDA_SIMULATE_AVAILABLE")) { snprintf(reason, n, "cuda_simulated_available"); return 1; }
    int count = 0;
    const cudaError_t e = cudaGetDeviceCount(&count);
    if (e == cudaSuccess && count > 0) { snprintf(reason, n, "cuda_runtime_detected"); return 1; }
    if (e != cudaSuccess) { cudaGetLastError(); snprintf(reason, n, "cuda_runtime_error_%d", static_cast<int>(e)); }
    else snprintf(reason, n, "cuda_runtime_no_device");
    return 0;
}

bool real_device_present() {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return false; }
    return count > 0;
}

}  // namespace

extern "C" {

void pyc_cuda_dispatch_trace_init(pyc_cuda_dispatch_trace* trace) {
    if (!trace) return;
    memset(trace, 0, sizeof(*trace));
}

pyc_kernel_hardware_family pyc_cuda_current_hardware_family(void) {
    const char* o = getenv("PYC_CUDA_FORCE_HARDWARE_FAMILY");
    if (o && o[0]) {
        if (!strcmp(o, "hopper")) return PYC_KERNEL_HARDWARE_HOPPER;
        if (!strcmp(o, "ada")) return PYC_KERNEL_HARDWARE_ADA;
        if (!strcmp(o, "generic")) return PYC_KERNEL_HARDWARE_GENERIC;
    }
    if (!real_device_present()) return PYC_KERNEL_HARDWARE_GENERIC;
    DeviceContext* c = current_context();
    if (!c) return PYC_KERNEL_HARDWARE_GENERIC;
    if (c->cc_major >= 9) return PYC_KERNEL_HARDWARE_HOPPER;
    if (c->cc_major == 8 && c->cc_minor >= 9) return PYC_KERNEL_HARDWARE_ADA;
    return PYC_KERNEL_HARDWARE_GENERIC;
}

pyc_cuda_dispatch_status pyc_cuda_dispatch(const pyc_ir_module* module, const pyc_tensor* inputs, size_t input_count,
                                           pyc_tensor* outputs, size_t output_count, pyc_cpu_executor_fn cpu_executor,
                                           void* executor_ctx, pyc_cuda_dispatch_trace* trace) {
    // NULL cpu_executor is an error in PyC as well (cuda_backend.c:2822-2824).
    if (!module || !inputs || !outputs || !cpu_executor) return PYC_CUDA_DISPATCH_ERROR;
    pyc_cuda_dispatch_trace_init(trace);
    if (trace) trace->cuda_requested = 1;
    if (env_true("PYC_CUDA_FORCE_ERROR")) { set_reason(trace, "forced_error"); return PYC_CUDA_DISPATCH_ERROR; }

    char why[PYC_CUDA_REASON_MAX] = "", native[PYC_CUDA_REASON_MAX] = "";
    const int available = detect_cuda(why, sizeof(why));
    if (trace) trace->cuda_available = available;
    int native_rc = 1;
    const bool forced_fallback = env_true("PYC_CUDA_FORCE_FALLBACK");
    if (available && !forced_fallback) {
        registry_init_once();
        if (real_device_present()) {
            native_rc = run_on_gpu(module, inputs, input_count, outputs, output_count, trace, native, sizeof(native));
            if (native_rc == 0) { set_reason(trace, native); return PYC_CUDA_DISPATCH_OK; }
            if (native_rc < 0) {
                // A CUDA failure on a present GPU is reported, never papered over by the CPU.
                set_reason(trace, native[0] ? native : "b200_native_failed");
                return PYC_CUDA_DISPATCH_ERROR;
            }
        } else if (env_true("PYC_CUDA_SIMULATE_AVAILABLE")) {
            // PyC's test double (cuda_backend.c:2871-2880): no GPU, the env switch asks the
            // dispatch contract to be exercised anyway.
            if (run_simulated_device(module, inputs, input_count, outputs, output_count) == 0) {
                set_reason(trace, "cuda_native_simulated");
                return PYC_CUDA_DISPATCH_OK;
            }
        }
    }
    if (cpu_executor(module, inputs, input_count, outputs, output_count, executor_ctx) != 0) {
        if (trace) {
            char buf[PYC_CUDA_REASON_MAX];
            if (native[0]) snprintf(buf, sizeof(buf), "%.100s;cpu_fallback_failed", native); else snprintf(buf, sizeof(buf), "cpu_fallback_failed");
            set_reason(trace, buf);
        }
        return PYC_CUDA_DISPATCH_ERROR;
    }
    if (trace) {
        trace->fallback_to_cpu = 1;
        if (forced_fallback) set_reason(trace, "cuda_forced_fallback");
        else if (available && native_rc > 0) set_reason(trace, "cuda_native_unsupported_fallback");
        else if (available) set_reason(trace, "cuda_native_failed_fallback");
        else set_reason(trace, why);
    }
    return PYC_CUDA_DISPATCH_FALLBACK;
}


int pyc_b200_plan_arena(const pyc_ir_module* module, const pyc_tensor* inputs, size_t input_count, pyc_tensor* outputs, size_t output_count,
                        int tensors_on_device, pyc_alloc_request* requests_out, size_t* offsets_out, size_t capacity, size_t* count_out,
                        size_t* peak_bytes_out) {
    if (!module || !inputs || !outputs || !count_out) { set_error("pyc_b200_plan_arena: NULL argument"); return -1; }
    const MemKind kind = tensors_on_device ? MEM_DEVICE : MEM_PAGEABLE;
    std::vector<MemKind> in_mem(input_count, kind), out_mem(output_count, kind);
    Plan plan;
    const int rc = build_plan(module, inputs, input_count, outputs, output_count, in_mem, out_mem, false, 0u, &plan);
    if (rc != 0) { set_error(rc > 0 ? "pyc_b200_plan_arena: module uses an op the GPU path does not know" : "pyc_b200_plan_arena: malformed module or tensors"); return -1; }
    size_t n = 0;
    for (size_t i = 0; i < plan.values.size(); ++i) {
        const Value& v = plan.values[i];
        if (v.kind != V_TEMP) continue;
        if (n < capacity && requests_out && offsets_out) {
            requests_out[n].tensor_id = static_cast<int>(i);
            requests_out[n].size_bytes = v.bytes;
            requests_out[n].alignment = 1024;
            requests_out[n].start_step = v.def_step;
            requests_out[n].end_step = v.last_step;
            offsets_out[n] = v.arena_off;
        }
        ++n;
    }
    *count_out = n;
    if (peak_bytes_out) *peak_bytes_out = plan.arena_peak;
    return 0;
}

int pyc_b200_last_plan(const pyc_ir_module* module, char* out, size_t out_size) {
    std::lock_guard<std::mutex> lk(g_plan_table_mu);
    const std::string* text = nullptr;
    if (module) {
        auto it = g_plan_table.find(module_content_hash(module));
        if (it != g_plan_table.end()) text = &it->second;
    } else if (!g_last_plan_text.empty()) {
        text = &g_last_plan_text;
    }
    if (!text) { set_error("pyc_b200_last_plan: this module has not run on the GPU in this process"); return -1; }
    if (out && out_size) { strncpy(out, text->c_str(), out_size - 1); out[out_size - 1] = '\0'; }
    return static_cast<int>(text->size());
}

}  // extern "C"
