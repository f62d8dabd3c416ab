// Per-token fp8 (e4m3) quantisation of bf16 activations, optionally fused with the
// LayerNorm in front of it, and the FFN block that strings the fp8 GEMMs together.
//
// PyC has no fp8 path; these kernels belong to the transformer-FFN benchmark
// configuration (LayerNorm -> fp8 GEMM -> GELU -> fp8 GEMM).  Both quantisers are
// HBM-bound: one CTA per row, the row is read once (kept as packed 16-byte words in
// registers), scale = amax / 448 per row, values rounded to nearest-even e4m3.
//   layernorm_quant : x[rows,cols] bf16 -> LN (eps, optional gamma/beta) -> q[rows,cols] e4m3 + scale[rows]
//   quant_rows      : x[rows,cols] bf16 ->                                 q[rows,cols] e4m3 + scale[rows]
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "internal.h"

namespace b200 {

namespace {

constexpr int QT = 256;  // threads per row

__device__ __forceinline__ float q_block_reduce(float v, float* scratch, bool is_max) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const float w = __shfl_xor_sync(0xffffffffu, v, o); v = is_max ? fmaxf(v, w) : v + w; }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) scratch[w] = v;
    __syncthreads();
    v = l < QT / 32 ? scratch[l] : (is_max ? 0.0f : 0.0f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { const float x = __shfl_xor_sync(0xffffffffu, v, o); v = is_max ? fmaxf(v, x) : v + x; }
    return v;
}

// Sum, sum of squares, minimum and maximum over the block in ONE exchange (two barriers).
__device__ __forceinline__ void q_block_reduce_stats(float& s, float& ss, float& mn, float& mx, float (*scratch4)[4]) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o); ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) { scratch4[w][0] = s; scratch4[w][1] = ss; scratch4[w][2] = mn; scratch4[w][3] = mx; }
    __syncthreads();
    const bool in = l < QT / 32;
    s = in ? scratch4[l][0] : 0.0f; ss = in ? scratch4[l][1] : 0.0f; mn = in ? scratch4[l][2] : INFINITY; mx = in ? scratch4[l][3] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o); ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// VPT vectors of 8 bf16 per thread cached (cols <= QT*8*VPT); cols % 8 == 0.  The widest form keeps 32 registers of raw
// row data per thread, so it is built for two resident CTAs per SM (128 registers) instead of four (64, which spilled).
template <int VPT, bool LN>
__global__ void __launch_bounds__(QT, VPT >= 8 ? 2 : (VPT >= 4 && LN) ? 3 : 4)
rowquant_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                uint8_t* __restrict__ q, float* __restrict__ scale, size_t rows, size_t cols, float eps) {
    __shared__ float scratch[8];
    const size_t nvec = cols / 8;
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const __nv_bfloat16* xr = x + row * cols;
        uint4 raw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const size_t vi = threadIdx.x + static_cast<size_t>(i) * QT;
            if (vi < nvec) raw[i] = __ldg(reinterpret_cast<const uint4*>(xr) + vi);
        }
        float mean = 0.0f, rstd = 1.0f;
        if constexpr (LN) {
            if (!gamma && !beta) {
                // Plain normalisation: (x - mean) * rstd is monotonic in x, so the row's largest |y| follows from its minimum
                // and maximum, and mean, variance, min and max come out of one block exchange.  Sums are taken about the row's
                // first element so that a large common offset does not cancel in E[x^2] - E[x]^2.
                __shared__ float scratch4[QT / 32][4];
                const float pivot = __bfloat162float(xr[0]);
                float s = 0.0f, ss = 0.0f, mn = INFINITY, mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    if (threadIdx.x + static_cast<size_t>(i) * QT < nvec) {
                        float f[8]; unpack8(raw[i], f);
#pragma unroll
                        for (int j = 0; j < 8; ++j) { const float d = f[j] - pivot; s += d; ss = fmaf(d, d, ss); mn = fminf(mn, f[j]); mx = fmaxf(mx, f[j]); }
                    }
                q_block_reduce_stats(s, ss, mn, mx, scratch4);
                const float n_inv = 1.0f / static_cast<float>(cols);
                const float ds = s * n_inv;
                mean = pivot + ds;
                rstd = rsqrtf(fmaxf(ss * n_inv - ds * ds, 0.0f) + eps);
                const float amax_y = fmaxf(fabsf(mx - mean), fabsf(mn - mean)) * rstd;
                const float sc_y = amax_y > 0.0f ? amax_y * (1.0f / 448.0f) : 1.0f;
                if (threadIdx.x == 0) scale[row] = sc_y;
                const float a = rstd / sc_y, b = -mean * a;     // quantised value = x * a + b
                uint2* qr = reinterpret_cast<uint2*>(q + row * cols);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const size_t vi = threadIdx.x + static_cast<size_t>(i) * QT;
                    if (vi < nvec) {
                        float f[8]; unpack8(raw[i], f);
                        uint2 o;
                        o.x = pack_e4m3x4(fmaf(f[0], a, b), fmaf(f[1], a, b), fmaf(f[2], a, b), fmaf(f[3], a, b));
                        o.y = pack_e4m3x4(fmaf(f[4], a, b), fmaf(f[5], a, b), fmaf(f[6], a, b), fmaf(f[7], a, b));
                        qr[vi] = o;
                    }
                }
                continue;
            }
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
                if (threadIdx.x + static_cast<size_t>(i) * QT < nvec) { float f[8]; unpack8(raw[i], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) s += f[j]; }
            mean = q_block_reduce(s, scratch, false) / static_cast<float>(cols);
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < VPT; ++i)
                if (threadIdx.x + static_cast<size_t>(i) * QT < nvec) { float f[8]; unpack8(raw[i], f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) { const float d = f[j] - mean; ss = fmaf(d, d, ss); } }
            rstd = rsqrtf(q_block_reduce(ss, scratch, false) / static_cast<float>(cols) + eps);
        }
        // value after the optional LayerNorm
        auto value = [&](const float (&f)[8], size_t vi, float (&y)[8]) {
            if constexpr (LN) {
                float g[8], b[8];
                if (gamma) unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + vi), g);
                if (beta) unpack8(__ldg(reinterpret_cast<const uint4*>(beta) + vi), b);
#pragma unroll
                for (int j = 0; j < 8; ++j) { float v = (f[j] - mean) * rstd; if (gamma) v *= g[j]; if (beta) v += b[j]; y[j] = v; }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) y[j] = f[j];
            }
        };
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const size_t vi = threadIdx.x + static_cast<size_t>(i) * QT;
            if (vi < nvec) { float f[8], y[8]; unpack8(raw[i], f); value(f, vi, y);
#pragma unroll
                for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(y[j])); }
        }
        amax = q_block_reduce(amax, scratch, true);
        const float sc = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
        const float inv = 1.0f / sc;
        if (threadIdx.x == 0) scale[row] = sc;
        uint2* qrow = reinterpret_cast<uint2*>(q + row * cols);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const size_t vi = threadIdx.x + static_cast<size_t>(i) * QT;
            if (vi < nvec) {
                float f[8], y[8]; unpack8(raw[i], f); value(f, vi, y);
                uint2 o;
                o.x = pack_e4m3x4(y[0] * inv, y[1] * inv, y[2] * inv, y[3] * inv);
                o.y = pack_e4m3x4(y[4] * inv, y[5] * inv, y[6] * inv, y[7] * inv);
                qrow[vi] = o;
            }
        }
    }
}

// One WARP per row, for rows of exactly VW * 256 elements (1024 / 2048 / 4096) without gamma / beta.  With a whole CTA per
// row a thread owns 16 elements of a 4096-wide row and the two block exchanges (shuffles, shared memory, two barriers)
// cost as many instructions as the arithmetic: 23 instructions per element, 2.4 TB/s.  Here a lane owns VW * 8
// elements, the statistics are five shuffle steps, nothing is shared between warps, and a warp has VW 16-byte loads in
// flight.  Same formulas as above: LayerNorm sums about the row's first element, the row's largest |y| from its minimum
// and maximum, quantised value = x * a + b.
template <int VW, bool LN>
__global__ void __launch_bounds__(QT, VW >= 16 ? 1 : 2)
rowquant_warp_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, size_t rows, float eps) {
    constexpr size_t COLS = static_cast<size_t>(VW) * 256;
    const int lane = threadIdx.x & 31;
    const size_t step = static_cast<size_t>(gridDim.x) * (QT / 32);
    const size_t row0 = blockIdx.x * static_cast<size_t>(QT / 32) + (threadIdx.x >> 5);
    uint4 raw[VW], ahead[VW];      // the warp's next row is fetched while the current one is reduced and written
    if (row0 < rows) {
#pragma unroll
        for (int i = 0; i < VW; ++i) raw[i] = __ldg(reinterpret_cast<const uint4*>(x + row0 * COLS) + lane + 32 * i);
    }
    for (size_t row = row0; row < rows; row += step) {
        if (row + step < rows) {
#pragma unroll
            for (int i = 0; i < VW; ++i) ahead[i] = __ldg(reinterpret_cast<const uint4*>(x + (row + step) * COLS) + lane + 32 * i);
        }
        float a, b, sc;
        if constexpr (LN) {
            const float pivot = __uint_as_float(__shfl_sync(0xffffffffu, raw[0].x, 0) << 16);   // the row's first element
            float s = 0.0f, ss = 0.0f, mn = INFINITY, mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < VW; ++i) {
                float f[8]; unpack8(raw[i], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) { const float d = f[j] - pivot; s += d; ss = fmaf(d, d, ss); mn = fminf(mn, f[j]); mx = fmaxf(mx, f[j]); }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                s += __shfl_xor_sync(0xffffffffu, s, o); ss += __shfl_xor_sync(0xffffffffu, ss, o);
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            const float n_inv = 1.0f / static_cast<float>(COLS);
            const float ds = s * n_inv, mean = pivot + ds;
            const float rstd = rsqrtf(fmaxf(ss * n_inv - ds * ds, 0.0f) + eps);
            const float amax_y = fmaxf(fabsf(mx - mean), fabsf(mn - mean)) * rstd;
            sc = amax_y > 0.0f ? amax_y * (1.0f / 448.0f) : 1.0f;
            a = rstd / sc; b = -mean * a;
        } else {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < VW; ++i) {
                float f[8]; unpack8(raw[i], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            sc = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
            a = 1.0f / sc; b = 0.0f;
        }
        if (lane == 0) scale[row] = sc;
        uint2* qr = reinterpret_cast<uint2*>(q + row * COLS);
#pragma unroll
        for (int i = 0; i < VW; ++i) {
            float f[8]; unpack8(raw[i], f);
            uint2 o;
            if constexpr (LN) {
                o.x = pack_e4m3x4(fmaf(f[0], a, b), fmaf(f[1], a, b), fmaf(f[2], a, b), fmaf(f[3], a, b));
                o.y = pack_e4m3x4(fmaf(f[4], a, b), fmaf(f[5], a, b), fmaf(f[6], a, b), fmaf(f[7], a, b));
            } else {   // the plain quantiser multiplies by the reciprocal scale, as the CTA-per-row kernel does
                o.x = pack_e4m3x4(f[0] * a, f[1] * a, f[2] * a, f[3] * a);
                o.y = pack_e4m3x4(f[4] * a, f[5] * a, f[6] * a, f[7] * a);
            }
            qr[lane + 32 * i] = o;
        }
#pragma unroll
        for (int i = 0; i < VW; ++i) raw[i] = ahead[i];
    }
}

template <bool LN>
int launch_rowquant(const void* x, const void* gamma, const void* beta, void* q, float* scale, size_t rows, size_t cols, float eps, cudaStream_t s) {
    if (rows == 0 || cols == 0 || cols % 8 != 0 || !x || !q || !scale) { set_error("row quantise: needs cols %% 8 == 0 and non-NULL pointers"); return -1; }
    auto al = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (!al(x) || !al(gamma) || !al(beta) || reinterpret_cast<uintptr_t>(q) % 8) { set_error("row quantise: pointers must be 16-byte aligned"); return -1; }
    const size_t nvec = cols / 8;
    size_t grid = rows;
    const size_t cap = static_cast<size_t>(sm_count()) * 64;
    if (grid > cap) grid = cap;
    const auto* xb = static_cast<const __nv_bfloat16*>(x); const auto* g = static_cast<const __nv_bfloat16*>(gamma); const auto* b = static_cast<const __nv_bfloat16*>(beta);
    auto* qq = static_cast<uint8_t*>(q);
    if (!gamma && !beta && rows >= 64 && (cols == 1024 || cols == 2048 || cols == 4096)) {   // one warp per row
        size_t wgrid = (rows + QT / 32 - 1) / (QT / 32);
        const size_t wcap = static_cast<size_t>(sm_count()) * (cols == 4096 ? 1 : 2);   // resident CTAs: the 4096-wide form holds 64 registers of row data per lane
        if (wgrid > wcap) wgrid = wcap;
        if (cols == 4096) rowquant_warp_kernel<16, LN><<<static_cast<unsigned>(wgrid), QT, 0, s>>>(xb, qq, scale, rows, eps);
        else if (cols == 2048) rowquant_warp_kernel<8, LN><<<static_cast<unsigned>(wgrid), QT, 0, s>>>(xb, qq, scale, rows, eps);
        else rowquant_warp_kernel<4, LN><<<static_cast<unsigned>(wgrid), QT, 0, s>>>(xb, qq, scale, rows, eps);
        B200_CUDA_OK(cudaGetLastError());
        count_launch();
        return 0;
    }
    if (nvec <= QT * 2) rowquant_kernel<2, LN><<<static_cast<unsigned>(grid), QT, 0, s>>>(xb, g, b, qq, scale, rows, cols, eps);
    else if (nvec <= QT * 4) rowquant_kernel<4, LN><<<static_cast<unsigned>(grid), QT, 0, s>>>(xb, g, b, qq, scale, rows, cols, eps);
    else if (nvec <= QT * 8) rowquant_kernel<8, LN><<<static_cast<unsigned>(grid), QT, 0, s>>>(xb, g, b, qq, scale, rows, cols, eps);
    else { set_error("row quantise: rows wider than %d elements are not supported", QT * 8 * 8); return -1; }
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int pyc_b200_quantize_rows(const void* x_bf16, void* q_e4m3, float* row_scale, size_t rows, size_t cols, void* stream) {
    return launch_rowquant<false>(x_bf16, nullptr, nullptr, q_e4m3, row_scale, rows, cols, 0.0f, static_cast<cudaStream_t>(stream));
}

int pyc_b200_layernorm_quantize(const void* x_bf16, const void* gamma, const void* beta, void* q_e4m3, float* row_scale,
                                size_t rows, size_t cols, float eps, void* stream) {
    return launch_rowquant<true>(x_bf16, gamma, beta, q_e4m3, row_scale, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

int pyc_b200_gemm_fp8(int M, int N, int K, const void* A_e4m3, const void* B_e4m3, int b_col_major, const float* row_scale,
                      const float* col_scale, const void* bias_bf16, pyc_b200_activation act, void* D_bf16, void* stream) {
    return launch_gemm_fp8(M, N, K, A_e4m3, B_e4m3, b_col_major, row_scale, col_scale, bias_bf16, act, D_bf16,
                           static_cast<cudaStream_t>(stream), device_status_word());
}

size_t pyc_b200_ffn_workspace_bytes(int tokens, int hidden, int inner) {
    if (tokens <= 0 || hidden <= 0 || inner <= 0) return 0;
    const size_t T = tokens, H = hidden, I = inner;
    return align256(T * H) + align256(T * 4) + align256(T * I * 2) + align256(T * I) + align256(T * 4);
}

// Optional per-phase timing: five events the caller owns, recorded on the block's stream at the start and after each of
// the four kernels.  Thread-local, so it only affects calls of the thread that set it.
static thread_local void* const* g_ffn_phase_events = nullptr;
int pyc_b200_ffn_phase_events(void* const* events5) { g_ffn_phase_events = events5; return 0; }
static inline void ffn_mark(int i, cudaStream_t s) {
    if (g_ffn_phase_events && g_ffn_phase_events[i]) cudaEventRecord(static_cast<cudaEvent_t>(g_ffn_phase_events[i]), s);
}

static int ffn_block_impl(const pyc_b200_ffn_args* a, void* workspace, size_t workspace_bytes, void* stream, const b200::Fp8Scatter* scatter,
                          const b200::Fp8SwitchReduce* switch_reduce = nullptr) {
    if (!a || !a->x || !a->w1 || !a->w2 || !a->w1_scale || !a->w2_scale || (!a->out && !scatter) || !workspace) { set_error("ffn: NULL argument"); return -1; }
    const size_t need = pyc_b200_ffn_workspace_bytes(a->tokens, a->hidden, a->inner);
    if (need == 0 || workspace_bytes < need) { set_error("ffn: workspace of %zu bytes needed, %zu given", need, workspace_bytes); return -1; }
    if (reinterpret_cast<uintptr_t>(workspace) % 256) { set_error("ffn: workspace must be 256-byte aligned"); return -1; }
    const size_t T = a->tokens, H = a->hidden, I = a->inner;
    char* p = static_cast<char*>(workspace);
    void* xq = p; p += align256(T * H);
    float* xs = reinterpret_cast<float*>(p); p += align256(T * 4);
    void* h = p; p += align256(T * I * 2);
    void* hq = p; p += align256(T * I);
    float* hs = reinterpret_cast<float*>(p);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* st = device_status_word();
    if (!st) return -1;
    // 1. LayerNorm + per-token quantisation   2. fp8 GEMM1 (+bias) + GELU -> bf16
    // 3. per-token quantisation               4. fp8 GEMM2 (+bias) -> bf16 (a partial sum when the inner dimension is sharded;
    //                                            with `scatter`, every row goes straight to the receive slot of the rank that owns it)
    ffn_mark(0, s);
    if (launch_rowquant<true>(a->x, a->ln_gamma, a->ln_beta, xq, xs, T, H, a->eps > 0.0f ? a->eps : 1e-5f, s) != 0) return -1;
    ffn_mark(1, s);
    if (launch_gemm_fp8(a->tokens, a->inner, a->hidden, xq, a->w1, 0, xs, a->w1_scale, a->b1, PYC_B200_ACT_GELU, h, s, st) != 0) return -1;
    ffn_mark(2, s);
    if (launch_rowquant<false>(h, nullptr, nullptr, hq, hs, T, I, 0.0f, s) != 0) return -1;
    ffn_mark(3, s);
    if (launch_gemm_fp8(a->tokens, a->hidden, a->inner, hq, a->w2, 0, hs, a->w2_scale, a->b2, PYC_B200_ACT_NONE, a->out, s, st, scatter, switch_reduce) != 0) return -1;
    ffn_mark(4, s);
    return 0;
}

int pyc_b200_ffn_block(const pyc_b200_ffn_args* a, void* workspace, size_t workspace_bytes, void* stream) {
    return ffn_block_impl(a, workspace, workspace_bytes, stream, nullptr);
}

// Tensor-parallel block through PyC's collective interface (include/pyc/collective_comm.h:30-42): this rank's shard of
// the block, then ONE all-reduce (sum) of the [tokens, hidden] bf16 partial sums, issued through the caller's vtable on
// the same stream.  The communicator handle is whatever the launcher created for that backend (PyC passes it around as
// "comm_handle", distributed_runtime.c:16-42).
int pyc_b200_ffn_block_tp(const pyc_b200_ffn_args* a, const pyc_collective_comm* comm, pyc_comm_handle_t comm_handle, int world, int rank,
                          void* workspace, size_t workspace_bytes, void* stream) {
    if (!a) { set_error("ffn tp: NULL arguments"); return -1; }
    if (world < 1 || rank < 0 || rank >= world) { set_error("ffn tp: bad world/rank %d/%d", rank, world); return -1; }
    if (world > 1 && (!comm || !comm->all_reduce || !comm_handle)) { set_error("ffn tp: world %d needs a collective vtable with all_reduce and a communicator handle", world); return -1; }
    if (!a->out) { set_error("ffn tp: NULL output"); return -1; }
    if (ffn_block_impl(a, workspace, workspace_bytes, stream, nullptr) != 0) return -1;
    if (world == 1) return 0;
    const size_t count = static_cast<size_t>(a->tokens) * static_cast<size_t>(a->hidden);
    const pyc_comm_status st = comm->all_reduce(comm->backend_ctx, comm_handle, a->out, a->out, count, PYC_DTYPE_BF16, PYC_REDUCE_SUM, stream);
    if (st != PYC_COMM_OK) {
        set_error("ffn tp: all_reduce through the collective vtable failed with pyc_comm_status %d (%s)", static_cast<int>(st),
                  st == PYC_COMM_ERR_TIMEOUT ? "timeout" : st == PYC_COMM_ERR_HARDWARE ? "hardware/transport" : "invalid argument or unsupported dtype");
        return -1;
    }
    return 0;
}

int pyc_b200_ffn_block_switch_reduce(const pyc_b200_ffn_args* a, void* workspace, size_t workspace_bytes, void* multicast_out,
                                     void* const* flag_ptrs, void* const* fin_ptrs, void* epoch_counters, int world, int rank, void* stream) {
    if (!a || !multicast_out || !flag_ptrs || !fin_ptrs || !epoch_counters || world < 2 || world > PYC_B200_TP_MAX_RANKS || rank < 0 || rank >= world) {
        set_error("ffn switch reduce: bad world/rank or NULL argument"); return -1;
    }
    b200::Fp8SwitchReduce sw;
    sw.multicast_d = multicast_out; sw.epochs = epoch_counters; sw.world = world; sw.rank = rank;
    for (int i = 0; i < PYC_B200_TP_MAX_RANKS; ++i) { sw.flags[i] = i < world ? flag_ptrs[i] : nullptr; sw.fin[i] = i < world ? fin_ptrs[i] : nullptr; }
    return ffn_block_impl(a, workspace, workspace_bytes, stream, nullptr, &sw);
}

int pyc_b200_ffn_block_scatter(const pyc_b200_ffn_args* a, void* workspace, size_t workspace_bytes, void* const* recv_slots, int world, int rank,
                               void* stream) {
    if (!recv_slots || world < 1 || world > PYC_B200_TP_MAX_RANKS || rank < 0 || rank >= world) { set_error("ffn scatter: bad world/rank or NULL slot table"); return -1; }
    if (a && a->tokens % world != 0) { set_error("ffn scatter: %d tokens do not split over %d ranks", a->tokens, world); return -1; }
    b200::Fp8Scatter sc;
    sc.world = world; sc.rank = rank;
    for (int i = 0; i < PYC_B200_TP_MAX_RANKS; ++i) sc.dst[i] = i < world ? recv_slots[i] : nullptr;
    return ffn_block_impl(a, workspace, workspace_bytes, stream, &sc);
}

}  // extern "C"
