// HBM-bound elementwise and row-reduction kernels: add, bias+activation,
// layernorm, softmax, reduce_sum.  128-bit coalesced loads/stores, warp-shuffle
// reductions, each row read from HBM exactly once (kept in registers between the
// statistics pass and the normalisation pass).
//
// These are the ops PyC's IR names (include/pyc/ir.h:29-39) but its executors do
// not implement on the GPU: ADD/RELU run as host loops after the GEMM
// (src/compiler/runtime/cuda_backend.c:1697-1742), GELU / LAYERNORM / REDUCE_SUM
// are rejected (cuda_backend.c:1153-1159).  Semantics: GELU = exact erf form;
// LAYERNORM = last axis, biased variance, eps inside the square root, optional
// gamma/beta; REDUCE_SUM / softmax = over the trailing axis.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "math.cuh"

namespace b200 {
namespace {

template <typename T> struct VecInfo;
template <> struct VecInfo<float> { static constexpr int N = 4; };
template <> struct VecInfo<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct VecInfo<__half> { static constexpr int N = 8; };

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
__device__ __forceinline__ void from_f(float& d, float v) { d = v; }
__device__ __forceinline__ void from_f(__nv_bfloat16& d, float v) { d = __float2bfloat16_rn(v); }
__device__ __forceinline__ void from_f(__half& d, float v) { d = __float2half_rn(v); }

// VEC elements of T as one 16-byte (or, for VEC == 1, scalar) access.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[VEC]) {
    if constexpr (VEC == 1) {
        f[0] = to_f(*p);
    } else {
        union { uint4 u; T t[VEC]; } x;
        x.u = __ldg(reinterpret_cast<const uint4*>(p));
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = to_f(x.t[i]);
    }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[VEC]) {
    if constexpr (VEC == 1) {
        from_f(*p, f[0]);
    } else {
        union { uint4 u; T t[VEC]; } x;
#pragma unroll
        for (int i = 0; i < VEC; ++i) from_f(x.t[i], f[i]);
        *reinterpret_cast<uint4*>(p) = x.u;
    }
}

template <int ACT>
__device__ __forceinline__ float act_fn(float v) {
    if constexpr (ACT == PYC_B200_ACT_RELU) return v > 0.0f ? v : 0.0f;
    if constexpr (ACT == PYC_B200_ACT_GELU) return gelu_erf(v);
    return v;
}

// Activation over a register vector; GELU takes the elements two at a time (packed fp32 pairs).
template <int ACT, int VEC>
__device__ __forceinline__ void act_vec(float (&v)[VEC]) {
    if constexpr (ACT == PYC_B200_ACT_GELU && VEC == 8) {          // eight per 16 bytes: a 16-bit storage type
#pragma unroll
        for (int j = 0; j < VEC; j += 2) gelu_erf_x2_16bit(v[j], v[j + 1]);
    } else if constexpr (ACT == PYC_B200_ACT_GELU && VEC % 2 == 0) {
#pragma unroll
        for (int j = 0; j < VEC; j += 2) gelu_erf_x2(v[j], v[j + 1]);
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = act_fn<ACT>(v[j]);
    }
}

// ------------------------------------------------------------------ add ------
template <typename T, int VEC>
__global__ void __launch_bounds__(256) add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t nvec) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < nvec; i += 2 * stride) {
        const size_t i2 = i + stride;
        const bool two = i2 < nvec;
        float x[VEC], y[VEC], x2[VEC], y2[VEC];
        load_vec<T, VEC>(a + i * VEC, x);
        load_vec<T, VEC>(b + i * VEC, y);
        if (two) { load_vec<T, VEC>(a + i2 * VEC, x2); load_vec<T, VEC>(b + i2 * VEC, y2); }
#pragma unroll
        for (int j = 0; j < VEC; ++j) x[j] += y[j];
        store_vec<T, VEC>(out + i * VEC, x);
        if (two) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) x2[j] += y2[j];
            store_vec<T, VEC>(out + i2 * VEC, x2);
        }
    }
}

// --------------------------------------------------------- bias + activation --
template <typename T, int VEC, int ACT>
__global__ void __launch_bounds__(256) bias_act_kernel(const T* __restrict__ x, const T* __restrict__ add, int add_mode,
                                                      T* __restrict__ out, size_t nvec, size_t cols) {
    const float sadd = add_mode == PYC_B200_ADD_SCALAR ? to_f(add[0]) : 0.0f;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    constexpr int UNROLL = 4;  // independent 16-byte loads in flight per thread
    for (size_t i0 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += UNROLL * stride) {
        float v[UNROLL][VEC];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const size_t i = i0 + u * stride;
            if (i < nvec) load_vec<T, VEC>(x + i * VEC, v[u]);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const size_t i = i0 + u * stride;
            if (i >= nvec) continue;
            if (add_mode == PYC_B200_ADD_MATRIX || add_mode == PYC_B200_ADD_ROW_BIAS) {
                float y[VEC];
                const size_t off = add_mode == PYC_B200_ADD_MATRIX ? i * VEC : (i * VEC) % cols;
                load_vec<T, VEC>(add + off, y);
#pragma unroll
                for (int j = 0; j < VEC; ++j) v[u][j] += y[j];
            }
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[u][j] += sadd;
            act_vec<ACT, VEC>(v[u]);
            store_vec<T, VEC>(out + i * VEC, v[u]);
        }
    }
}

// Row bias (+ activation): every thread owns one 16-byte column slot, keeps its slice of the bias in registers and
// walks down the rows, so there is no index arithmetic beyond one add per row.  The next group of rows is fetched as raw
// 16-byte words before the current group is converted and computed: with GELU on a 2-byte type the arithmetic of a group
// is as long as its memory time, and without the prefetch a warp has no load in flight while it computes.
template <typename T, int VEC>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float (&f)[VEC]) {
    union { uint4 u; T t[VEC]; } x;
    x.u = raw;
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = to_f(x.t[i]);
}

template <typename T, int VEC, int ACT>
__global__ void __launch_bounds__(256) row_bias_act_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ out,
                                                          size_t rows, size_t cols) {
    static_assert(VEC * sizeof(T) == 16, "one 16-byte slot per thread");
    const size_t vec_per_row = cols / VEC;
    const size_t col_vec = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    if (col_vec >= vec_per_row) return;
    float b[VEC];
    load_vec<T, VEC>(bias + col_vec * VEC, b);
    constexpr int UNROLL = 4;
    const size_t step = static_cast<size_t>(gridDim.y);
    const T* xp = x + col_vec * VEC;
    T* op = out + col_vec * VEC;
    uint4 cur[UNROLL], nxt[UNROLL];
    auto fetch = [&](size_t r0, uint4 (&dst)[UNROLL]) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const size_t r = r0 + static_cast<size_t>(u) * step;
            if (r < rows) dst[u] = __ldg(reinterpret_cast<const uint4*>(xp + r * cols));
        }
    };
    size_t r0 = blockIdx.y;
    if (r0 < rows) fetch(r0, cur);
    for (; r0 < rows; r0 += step * UNROLL) {
        const size_t rn = r0 + step * UNROLL;
        if (rn < rows) fetch(rn, nxt);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const size_t r = r0 + static_cast<size_t>(u) * step;
            if (r >= rows) continue;
            float v[VEC];
            unpack_vec<T, VEC>(cur[u], v);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] += b[j];
            act_vec<ACT, VEC>(v);
            store_vec<T, VEC>(op + r * cols, v);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) cur[u] = nxt[u];
    }
}

// ------------------------------------------------------------ row reductions --
enum RowOp { ROW_LAYERNORM = 0, ROW_SOFTMAX = 1, ROW_SUM = 2 };

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if constexpr (THREADS > 32) {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
        __syncthreads();
        if (l == 0) scratch[w] = v;
        __syncthreads();
        v = l < THREADS / 32 ? scratch[l] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}
// Two sums in one round.
template <int THREADS>
__device__ __forceinline__ void block_sum2(float& a, float& b, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
    if constexpr (THREADS > 32) {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
        __syncthreads();
        if (l == 0) { scratch[w] = a; scratch[8 + w] = b; }
        __syncthreads();
        a = l < THREADS / 32 ? scratch[l] : 0.0f;
        b = l < THREADS / 32 ? scratch[8 + l] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
    }
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if constexpr (THREADS > 32) {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
        __syncthreads();
        if (l == 0) scratch[w] = v;
        __syncthreads();
        v = l < THREADS / 32 ? scratch[l] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    return v;
}

// Raw storage of one vector access: the row stays in registers between passes as packed
// 16-byte words (4 registers per 8 bf16), not as widened floats, which keeps occupancy up.
template <typename T, int VEC> struct RawVec { uint4 u; };
template <typename T> struct RawVec<T, 1> { T u; };
template <typename T, int VEC>
__device__ __forceinline__ RawVec<T, VEC> load_raw(const T* p) {
    RawVec<T, VEC> r;
    if constexpr (VEC == 1) r.u = *p; else r.u = __ldg(reinterpret_cast<const uint4*>(p));
    return r;
}
template <typename T, int VEC>
__device__ __forceinline__ void widen(const RawVec<T, VEC>& r, float (&f)[VEC]) {
    if constexpr (VEC == 1) {
        f[0] = to_f(r.u);
    } else {
        union { uint4 u; T t[VEC]; } x;
        x.u = r.u;
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = to_f(x.t[i]);
    }
}

// Running maximum over packed 16-bit pairs (exact: a maximum needs no widening); four instructions per 8 elements.
__device__ __forceinline__ void raw_max_acc(const uint4& u, __nv_bfloat162& m) {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
    m = __hmax2(m, __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3])));
}
__device__ __forceinline__ void raw_max_acc(const uint4& u, __half2& m) {
    const __half2* p = reinterpret_cast<const __half2*>(&u);
    m = __hmax2(m, __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3])));
}
__device__ __forceinline__ float pair_max(const __nv_bfloat162& m) { return fmaxf(__low2float(m), __high2float(m)); }
__device__ __forceinline__ float pair_max(const __half2& m) { return fmaxf(__low2float(m), __high2float(m)); }
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> { using type = __nv_bfloat162; __device__ static type lowest() { return __floats2bfloat162_rn(-INFINITY, -INFINITY); } };
template <> struct Pair16<__half> { using type = __half2; __device__ static type lowest() { return __floats2half2_rn(-INFINITY, -INFINITY); } };

// One row per group of THREADS threads (THREADS = 32: four rows per CTA).  Each thread
// owns up to VPT vectors of its row in registers; CACHED == false is the any-width form
// that re-reads the row from global memory instead.
template <typename T, int VEC, int THREADS, int VPT, bool CACHED, int OP>
__global__ void __launch_bounds__(THREADS >= 128 ? THREADS : 128, THREADS >= 256 ? 4 : 8)
row_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ out,
           size_t rows, size_t cols, float eps) {
    constexpr int ROWS_PER_CTA = THREADS >= 128 ? 1 : 128 / THREADS;
    constexpr int NV = CACHED ? VPT : 1;
    __shared__ float scratch[16];
    const int tid = THREADS >= 128 ? threadIdx.x : (threadIdx.x % THREADS);
    const size_t nvec = cols / VEC;
    for (size_t row = blockIdx.x * static_cast<size_t>(ROWS_PER_CTA) + (THREADS >= 128 ? 0 : threadIdx.x / THREADS);
         row < rows; row += static_cast<size_t>(gridDim.x) * ROWS_PER_CTA) {
        const T* xr = x + row * cols;
        T* orow = out + (OP == ROW_SUM ? 0 : row * cols);
        RawVec<T, VEC> raw[NV];
        // Visit every vector this thread owns: from registers when cached, else from global memory.
        auto for_each = [&](auto&& fn) {
            if constexpr (CACHED) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const size_t vi = tid + static_cast<size_t>(i) * THREADS;
                    if (vi < nvec) { float f[VEC]; widen<T, VEC>(raw[i], f); fn(f, vi); }
                }
            } else {
                for (size_t vi = tid; vi < nvec; vi += THREADS) { float f[VEC]; widen<T, VEC>(load_raw<T, VEC>(xr + vi * VEC), f); fn(f, vi); }
            }
        };
        if constexpr (CACHED) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const size_t vi = tid + static_cast<size_t>(i) * THREADS;
                if (vi < nvec) raw[i] = load_raw<T, VEC>(xr + vi * VEC);
            }
        }
        if constexpr (OP == ROW_SUM) {
            float s = 0.0f;
            for_each([&](float (&f)[VEC], size_t) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) s += f[j];
            });
            s = block_sum<THREADS>(s, scratch);
            if (tid == 0) from_f(out[row], s);
        } else if constexpr (OP == ROW_LAYERNORM) {
            // One pass: sums of (x - p) and (x - p)^2 with the pivot p = first element of the row, which keeps the
            // variance free of cancellation whatever the row's mean is.
            const float pivot = to_f(xr[0]);
            float s = 0.0f, ss = 0.0f;
            for_each([&](float (&f)[VEC], size_t) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) { const float d = f[j] - pivot; s += d; ss = fmaf(d, d, ss); }
            });
            block_sum2<THREADS>(s, ss, scratch);
            const float inv_n = 1.0f / static_cast<float>(cols);
            const float dmean = s * inv_n;
            const float mean = pivot + dmean;
            const float rstd = rsqrtf(fmaxf(ss * inv_n - dmean * dmean, 0.0f) + eps);
            const float shift = -mean * rstd;   // y = x * rstd + shift: one FMA per element
            if (gamma || beta) {                // block-uniform: the affine form pays for its loads only when asked
                for_each([&](float (&f)[VEC], size_t vi) {
                    float g[VEC], b[VEC];
                    if (gamma) load_vec<T, VEC>(gamma + vi * VEC, g);
                    if (beta) load_vec<T, VEC>(beta + vi * VEC, b);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        float y = fmaf(f[j], rstd, shift);
                        if (gamma) y *= g[j];
                        if (beta) y += b[j];
                        f[j] = y;
                    }
                    store_vec<T, VEC>(orow + vi * VEC, f);
                });
            } else {
                for_each([&](float (&f)[VEC], size_t vi) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) f[j] = fmaf(f[j], rstd, shift);
                    store_vec<T, VEC>(orow + vi * VEC, f);
                });
            }
        } else {  // softmax
            float mx = -INFINITY;
            if constexpr (CACHED && VEC == 8) {       // 16-bit storage: the maximum straight from the packed pairs
                typename Pair16<T>::type m2 = Pair16<T>::lowest();
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    if (tid + static_cast<size_t>(i) * THREADS < nvec) raw_max_acc(raw[i].u, m2);
                mx = pair_max(m2);
            } else {
                for_each([&](float (&f)[VEC], size_t) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) mx = fmaxf(mx, f[j]);
                });
            }
            mx = block_max<THREADS>(mx, scratch);
            // exp(x - max) = 2^(x*log2e - max*log2e): one FMA + one special-function op per element (arguments <= 0: the
            // flush-to-zero form needs none of exp2f's range handling; 2 ulp)
            const float l2e = 1.4426950408889634f, mshift = -mx * l2e;
            float den = 0.0f;
            if constexpr (CACHED && VPT * VEC * (sizeof(T) == 4 ? 2 : 1) <= 32) {
                float e[NV][VEC];   // the exponentials are computed once and kept for the normalising pass (when they fit in registers)
                unsigned long long den2 = 0ull;   // bit pattern of (0.0f, 0.0f)
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const size_t vi = tid + static_cast<size_t>(i) * THREADS;
                    if (vi < nvec) {
                        float f[VEC];
                        widen<T, VEC>(raw[i], f);
                        if constexpr (VEC % 2 == 0) {   // exponent arguments and the running sum two elements per instruction
                            const unsigned long long l2e2 = f32x2_splat(l2e), ms2 = f32x2_splat(mshift);
#pragma unroll
                            for (int j = 0; j < VEC; j += 2) {
                                float t0, t1;
                                f32x2_unpack(f32x2_fma(f32x2_pack(f[j], f[j + 1]), l2e2, ms2), t0, t1);
                                e[i][j] = ex2_approx(t0); e[i][j + 1] = ex2_approx(t1);
                                den2 = f32x2_add(den2, f32x2_pack(e[i][j], e[i][j + 1]));
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < VEC; ++j) { e[i][j] = ex2_approx(fmaf(f[j], l2e, mshift)); den += e[i][j]; }
                        }
                    }
                }
                if constexpr (VEC % 2 == 0) { float lo, hi; f32x2_unpack(den2, lo, hi); den = lo + hi; }
                const float inv = 1.0f / block_sum<THREADS>(den, scratch);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const size_t vi = tid + static_cast<size_t>(i) * THREADS;
                    if (vi < nvec) {
                        if constexpr (VEC % 2 == 0) {
                            const unsigned long long inv2 = f32x2_splat(inv);
#pragma unroll
                            for (int j = 0; j < VEC; j += 2) f32x2_unpack(f32x2_mul(f32x2_pack(e[i][j], e[i][j + 1]), inv2), e[i][j], e[i][j + 1]);
                        } else {
#pragma unroll
                            for (int j = 0; j < VEC; ++j) e[i][j] *= inv;
                        }
                        store_vec<T, VEC>(orow + vi * VEC, e[i]);
                    }
                }
            } else {
                for_each([&](float (&f)[VEC], size_t) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) den += ex2_approx(fmaf(f[j], l2e, mshift));
                });
                const float inv = 1.0f / block_sum<THREADS>(den, scratch);
                for_each([&](float (&f)[VEC], size_t vi) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) f[j] = ex2_approx(fmaf(f[j], l2e, mshift)) * inv;
                    store_vec<T, VEC>(orow + vi * VEC, f);
                });
            }
        }
    }
}

inline int flat_grid(size_t work_items, int threads) {
    const size_t blocks = (work_items + threads - 1) / threads;
    const size_t cap = static_cast<size_t>(sm_count()) * 8;  // 8 CTAs of 256 threads fill an SM's 2048 thread slots
    return static_cast<int>(blocks < cap ? (blocks ? blocks : 1) : cap);
}

inline bool aligned16(const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; }

template <typename T, int VEC, int OP>
int launch_row_vec(const T* x, const T* g, const T* b, T* out, size_t rows, size_t cols, float eps, cudaStream_t s) {
    const size_t nvec = cols / VEC;
    const size_t max_grid = static_cast<size_t>(sm_count()) * 32;
#define B200_ROW(THREADS, VPT, CACHED)                                                                        \
    do {                                                                                                       \
        constexpr int RPC = (THREADS) >= 128 ? 1 : 128 / (THREADS);                                            \
        size_t grid = (rows + RPC - 1) / RPC;                                                                  \
        if (grid > max_grid) grid = max_grid;                                                                  \
        row_kernel<T, VEC, THREADS, VPT, CACHED, OP><<<static_cast<unsigned>(grid), (THREADS) >= 128 ? (THREADS) : 128, 0, s>>>( \
            x, g, b, out, rows, cols, eps);                                                                    \
    } while (0)
    if (nvec <= 32 * 4) B200_ROW(32, 4, true);
    else if (nvec <= 128 * 4) B200_ROW(128, 4, true);
    else if (nvec <= 256 * 4) B200_ROW(256, 4, true);
    else if (nvec <= 256 * 8) B200_ROW(256, 8, true);
    else B200_ROW(256, 1, false);
#undef B200_ROW
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

template <typename T, int OP>
int launch_row_typed(const void* x, const void* g, const void* b, void* out, size_t rows, size_t cols, float eps, cudaStream_t s) {
    constexpr int V = VecInfo<T>::N;
    const bool vec = cols % V == 0 && aligned16(x) && aligned16(g) && aligned16(b) && (OP == ROW_SUM || aligned16(out));
    if (vec) return launch_row_vec<T, V, OP>(static_cast<const T*>(x), static_cast<const T*>(g), static_cast<const T*>(b), static_cast<T*>(out), rows, cols, eps, s);
    return launch_row_vec<T, 1, OP>(static_cast<const T*>(x), static_cast<const T*>(g), static_cast<const T*>(b), static_cast<T*>(out), rows, cols, eps, s);
}

template <int OP>
int launch_row(pyc_dtype dt, const void* x, const void* g, const void* b, void* out, size_t rows, size_t cols, float eps, cudaStream_t s) {
    if (rows == 0 || cols == 0) { set_error("row op: empty shape"); return -1; }
    switch (dt) {
        case PYC_DTYPE_F32: return launch_row_typed<float, OP>(x, g, b, out, rows, cols, eps, s);
        case PYC_DTYPE_BF16: return launch_row_typed<__nv_bfloat16, OP>(x, g, b, out, rows, cols, eps, s);
        case PYC_DTYPE_F16: return launch_row_typed<__half, OP>(x, g, b, out, rows, cols, eps, s);
        default: set_error("row op: unsupported dtype %d", static_cast<int>(dt)); return -1;
    }
}

template <typename T>
int launch_add_typed(const void* a, const void* b, void* out, size_t n, cudaStream_t s) {
    constexpr int V = VecInfo<T>::N;
    if (n % V == 0 && aligned16(a) && aligned16(b) && aligned16(out)) {
        add_kernel<T, V><<<flat_grid(n / V, 256), 256, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n / V);
    } else {
        add_kernel<T, 1><<<flat_grid(n, 256), 256, 0, s>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n);
    }
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

template <typename T, int ACT>
int launch_bias_act_typed(const void* x, const void* add, int add_mode, void* out, size_t rows, size_t cols, cudaStream_t s) {
    constexpr int V = VecInfo<T>::N;
    const size_t n = rows * cols;
    if (!add) add_mode = PYC_B200_ADD_NONE;
    if (add_mode == PYC_B200_ADD_ROW_BIAS && cols % V == 0 && aligned16(x) && aligned16(out) && aligned16(add)) {
        const size_t vec_per_row = cols / V;
        const unsigned threads = vec_per_row >= 256 ? 256 : static_cast<unsigned>((vec_per_row + 31) / 32 * 32);
        const unsigned gx = static_cast<unsigned>((vec_per_row + threads - 1) / threads);
        size_t gy = (static_cast<size_t>(sm_count()) * 8 * 256 / threads + gx - 1) / gx;  // fill every SM's thread slots
        if (gy > rows) gy = rows;
        if (gy > 65535) gy = 65535;
        row_bias_act_kernel<T, V, ACT><<<dim3(gx, static_cast<unsigned>(gy)), threads, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(add),
                                                                                      static_cast<T*>(out), rows, cols);
    } else if (cols % V == 0 && aligned16(x) && aligned16(out) && (add_mode == PYC_B200_ADD_SCALAR || aligned16(add))) {
        bias_act_kernel<T, V, ACT><<<flat_grid(n / V, 256), 256, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(add), add_mode, static_cast<T*>(out), n / V, cols);
    } else {
        bias_act_kernel<T, 1, ACT><<<flat_grid(n, 256), 256, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(add), add_mode, static_cast<T*>(out), n, cols);
    }
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

}  // namespace

int launch_add(pyc_dtype dt, const void* a, const void* b, void* out, size_t n, cudaStream_t s) {
    if (n == 0) { set_error("add: empty"); return -1; }
    switch (dt) {
        case PYC_DTYPE_F32: return launch_add_typed<float>(a, b, out, n, s);
        case PYC_DTYPE_BF16: return launch_add_typed<__nv_bfloat16>(a, b, out, n, s);
        case PYC_DTYPE_F16: return launch_add_typed<__half>(a, b, out, n, s);
        default: set_error("add: unsupported dtype %d", static_cast<int>(dt)); return -1;
    }
}

int launch_bias_act(pyc_dtype dt, const void* x, const void* add, int add_mode, int act, void* out, size_t rows, size_t cols, cudaStream_t s) {
    if (rows == 0 || cols == 0) { set_error("bias_act: empty"); return -1; }
    if (act != PYC_B200_ACT_NONE && act != PYC_B200_ACT_RELU && act != PYC_B200_ACT_GELU) { set_error("bias_act: unknown activation %d", act); return -1; }
#define B200_BIAS_ACT(T)                                                                                          \
    (act == PYC_B200_ACT_GELU   ? launch_bias_act_typed<T, PYC_B200_ACT_GELU>(x, add, add_mode, out, rows, cols, s) \
     : act == PYC_B200_ACT_RELU ? launch_bias_act_typed<T, PYC_B200_ACT_RELU>(x, add, add_mode, out, rows, cols, s) \
                                : launch_bias_act_typed<T, PYC_B200_ACT_NONE>(x, add, add_mode, out, rows, cols, s))
    switch (dt) {
        case PYC_DTYPE_F32: return B200_BIAS_ACT(float);
        case PYC_DTYPE_BF16: return B200_BIAS_ACT(__nv_bfloat16);
        case PYC_DTYPE_F16: return B200_BIAS_ACT(__half);
        default: set_error("bias_act: unsupported dtype %d", static_cast<int>(dt)); return -1;
    }
#undef B200_BIAS_ACT
}

int launch_layernorm(pyc_dtype dt, const void* x, const void* gamma, const void* beta, void* out, size_t rows, size_t cols, float eps, cudaStream_t s) {
    return launch_row<ROW_LAYERNORM>(dt, x, gamma, beta, out, rows, cols, eps, s);
}
int launch_softmax(pyc_dtype dt, const void* x, void* out, size_t rows, size_t cols, cudaStream_t s) {
    return launch_row<ROW_SOFTMAX>(dt, x, nullptr, nullptr, out, rows, cols, 0.0f, s);
}
int launch_reduce_sum(pyc_dtype dt, const void* x, void* out, size_t rows, size_t cols, cudaStream_t s) {
    return launch_row<ROW_SUM>(dt, x, nullptr, nullptr, out, rows, cols, 0.0f, s);
}

}  // namespace b200
