// Host stand-in for the device, used ONLY when PYC_CUDA_SIMULATE_AVAILABLE=1 and
// no GPU is present.  PyC ships the same test double
// (src/compiler/runtime/cuda_backend.c:1392-1695, execute_native_cuda_graph_simulated)
// so that its dispatch-contract tests (tests/compiler_next/test_cuda_backend.c)
// run on machines without CUDA; its row-bias ADD semantics
// (cuda_backend.c:1556-1568) are what those tests pin.  It is never taken when a
// device exists and never stands in for a kernel: the dispatch reports it with
// the reason string "cuda_native_simulated".
#include <math.h>
#include <string.h>

#include <vector>

#include "internal.h"

namespace b200 {

int run_simulated_device(const pyc_ir_module* m, const pyc_tensor* inputs, size_t n_in, pyc_tensor* outputs, size_t n_out) {
    const size_t n = m->op_count;
    std::vector<std::vector<float>> val(n);
    std::vector<const void*> raw(n, nullptr);       // INPUT payloads, for byte-exact passthrough
    std::vector<size_t> raw_bytes(n, 0), cols(n, 0);
    size_t in_i = 0, out_i = 0;
    for (size_t i = 0; i < n; ++i) {
        const pyc_ir_op& op = m->ops[i];
        for (size_t j = 0; j < op.input_count; ++j)
            if (op.input_ids[j] < 0 || static_cast<size_t>(op.input_ids[j]) >= i) return -1;
        switch (op.kind) {
            case PYC_IR_OP_INPUT: {
                if (in_i >= n_in || !inputs[in_i].data) return -1;
                const pyc_tensor& t = inputs[in_i++];
                raw[i] = t.data; raw_bytes[i] = t.size_bytes;
                const pyc_shape& s = op.shape.rank ? op.shape : t.shape;
                cols[i] = s.rank ? static_cast<size_t>(s.dims[s.rank - 1]) : 0;
                if (t.dtype == PYC_DTYPE_F32) { val[i].resize(t.size_bytes / 4); memcpy(val[i].data(), t.data, val[i].size() * 4); }
                break;
            }
            case PYC_IR_OP_MATMUL: {
                if (op.input_count < 2) return -1;
                const pyc_ir_op &a = m->ops[op.input_ids[0]], &b = m->ops[op.input_ids[1]];
                if (a.shape.rank != 2 || b.shape.rank != 2 || a.shape.dims[1] != b.shape.dims[0]) return -1;
                const size_t M = a.shape.dims[0], K = a.shape.dims[1], N = b.shape.dims[1];
                const std::vector<float>&A = val[op.input_ids[0]], &B = val[op.input_ids[1]];
                if (A.size() < M * K || B.size() < K * N) return -1;
                val[i].assign(M * N, 0.0f); cols[i] = N;
                for (size_t r = 0; r < M; ++r) for (size_t c = 0; c < N; ++c) { float s = 0.0f; for (size_t t = 0; t < K; ++t) s += A[r * K + t] * B[t * N + c]; val[i][r * N + c] = s; }
                break;
            }
            case PYC_IR_OP_ADD: {
                if (op.input_count < 2) return -1;
                int ia = op.input_ids[0], ib = op.input_ids[1];
                if (val[ia].size() < val[ib].size()) { int t = ia; ia = ib; ib = t; }
                const std::vector<float>&A = val[ia], &B = val[ib];
                if (A.empty() || B.empty()) return -1;
                val[i] = A; cols[i] = cols[ia];
                if (B.size() == A.size()) for (size_t j = 0; j < A.size(); ++j) val[i][j] += B[j];
                else if (B.size() == 1) for (size_t j = 0; j < A.size(); ++j) val[i][j] += B[0];
                else if (cols[ia] && B.size() == cols[ia]) for (size_t j = 0; j < A.size(); ++j) val[i][j] += B[j % cols[ia]];
                else return -1;
                break;
            }
            case PYC_IR_OP_RELU: case PYC_IR_OP_GELU: {
                if (op.input_count < 1 || val[op.input_ids[0]].empty()) return -1;
                val[i] = val[op.input_ids[0]]; cols[i] = cols[op.input_ids[0]];
                for (float& v : val[i]) v = op.kind == PYC_IR_OP_RELU ? (v > 0.0f ? v : 0.0f) : 0.5f * v * (1.0f + erff(v * 0.70710678f));
                break;
            }
            case PYC_IR_OP_OUTPUT: {
                if (op.input_count < 1 || out_i >= n_out || !outputs[out_i].data) return -1;
                pyc_tensor& o = outputs[out_i++];
                const int src = op.input_ids[0];
                if (raw[src]) { if (o.size_bytes < raw_bytes[src]) return -1; memcpy(o.data, raw[src], raw_bytes[src]); break; }
                if (val[src].empty() || o.size_bytes < val[src].size() * 4) return -1;
                memcpy(o.data, val[src].data(), val[src].size() * 4);
                break;
            }
            default:
                return -1;
        }
    }
    return 0;
}

}  // namespace b200
