// fp32-accurate GEMM on the CUDA cores with the same fused epilogue as the
// tensor-core kernel: D = act(alpha * A*B + add_scale * add).
//
// Replaces the fp32 lane of PyC's CUDA backend (cublasGemmEx / cublasLt with
// TF32 at src/compiler/runtime/cuda_backend.c:770-1081, the CUTLASS SIMT kernel
// at cutlass_kernels/gemm/kernel.cu:89-99 and the hand-written cp.async kernel
// at cutlass_kernels/gemm/ada_async_kernel.cu:150-250).  Products are formed
// from unrounded fp32 inputs and accumulated with FMA in ascending k, so results
// stay within 1e-5 (norm-wise) of PyC's CPU executor; TF32 would not.
// It is also the any-shape path for bf16/f16 matrices whose leading dimensions
// do not satisfy TMA's 16-byte stride rule.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <type_traits>

#include "internal.h"
#include "math.cuh"

namespace b200 {
namespace {

constexpr int BK = 16;

__device__ __forceinline__ float ldf(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float ldf(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void stf(__half* p, float v) { *p = __float2half_rn(v); }

__device__ __forceinline__ float act_fn(float v, int act) {
    if (act == PYC_B200_ACT_RELU) return v > 0.0f ? v : 0.0f;
    if (act == PYC_B200_ACT_GELU) return gelu_erf(v);
    return v;
}

struct SimtParams {
    const void* A; const void* B; void* D; const void* add;
    int M, N, K;
    int b_col_major, add_mode, act;
    float alpha, add_scale;
};

template <typename T, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(SimtParams p) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int A_PER = BM * BK / THREADS;
    constexpr int B_PER = BK * BN / THREADS;
    static_assert(BM * BK % THREADS == 0 && BK * BN % THREADS == 0, "tile/threads mismatch");
    __shared__ float As[2][BK][BM + 4];
    __shared__ float Bs[2][BK][BN + 4];

    const T* A = reinterpret_cast<const T*>(p.A);
    const T* B = reinterpret_cast<const T*>(p.B);
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int M = p.M, N = p.N, K = p.K;

    float ra[A_PER], rb[B_PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A_PER; ++i) {  // A tile: consecutive threads walk k (contiguous in memory)
            const int e = tid + i * THREADS, r = e / BK, c = e % BK;
            const int gr = m0 + r, gc = k0 + c;
            ra[i] = (gr < M && gc < K) ? ldf(A + static_cast<size_t>(gr) * K + gc) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < B_PER; ++i) {
            const int e = tid + i * THREADS;
            if (p.b_col_major) {  // B stored [N,K]: walk k fastest
                const int c = e / BK, r = e % BK, gr = k0 + r, gc = n0 + c;
                rb[i] = (gr < K && gc < N) ? ldf(B + static_cast<size_t>(gc) * K + gr) : 0.0f;
            } else {
                const int r = e / BN, c = e % BN, gr = k0 + r, gc = n0 + c;
                rb[i] = (gr < K && gc < N) ? ldf(B + static_cast<size_t>(gr) * N + gc) : 0.0f;
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER; ++i) { const int e = tid + i * THREADS; As[buf][e % BK][e / BK] = ra[i]; }
#pragma unroll
        for (int i = 0; i < B_PER; ++i) {
            const int e = tid + i * THREADS;
            if (p.b_col_major) Bs[buf][e % BK][e / BK] = rb[i]; else Bs[buf][e / BN][e % BN] = rb[i];
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = 0; k0 < K; k0 += BK) {
        const bool more = k0 + BK < K;
        if (more) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[buf][kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[buf][kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) { stash(buf ^ 1); __syncthreads(); buf ^= 1; }
    }

    T* D = reinterpret_cast<T*>(p.D);
    const T* add = reinterpret_cast<const T*>(p.add);
    const float sadd = p.add_mode == PYC_B200_ADD_SCALAR ? p.add_scale * ldf(add) : 0.0f;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = m0 + ty * TM + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int c = n0 + tx * TN + j;
            if (c >= N) continue;
            float v = p.alpha * acc[i][j] + sadd;
            if (p.add_mode == PYC_B200_ADD_ROW_BIAS) v += p.add_scale * ldf(add + c);
            else if (p.add_mode == PYC_B200_ADD_MATRIX) v += p.add_scale * ldf(add + static_cast<size_t>(r) * N + c);
            stf(D + static_cast<size_t>(r) * N + c, act_fn(v, p.act));
        }
    }
}

// Latency variant for small fp32 problems (the 512^3 graph): 32 x 64 tile, 4 x 4 outputs per thread, operands brought
// in with 16-byte cp.async into a 3-stage ring of 32-deep k-slices, 16-byte shared-memory reads (8 loads per 64 FMAs).
// One wave of small CTAs covers most of the SMs, which leaves one CTA per SM: with 128 threads that is ONE warp per
// scheduler, and a lone warp issues its dependent FMA chain at well under half rate.  So the CTA has 512 threads:
// four groups of 128 each take a quarter of every k-slice (two of its eight 4-deep steps) into their own accumulators,
// and the four partial tiles are summed through shared memory once, after the last slice.  Within a group k ascends;
// the four partial sums are added in group order.  Needs K % 4 == 0, N % 4 == 0, 16-byte aligned A, B and D,
// row-major B.
constexpr int LBM = 32, LBN = 64, LBK = 32, LSTAGES = 3, LPAD = 4, LGROUPS = 4, LTHREADS = 128 * LGROUPS;
constexpr int L_A_FLOATS = LBM * (LBK + LPAD), L_B_FLOATS = LBK * LBN;
static_assert(LSTAGES * (L_A_FLOATS + L_B_FLOATS) >= LGROUPS * LBM * LBN, "the partial tiles reuse the operand ring");
static_assert((LBK / 4) % LGROUPS == 0, "every group takes the same number of 4-deep steps of a slice");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(LTHREADS)
gemm_simt_latency_kernel(SimtParams p) {
    __shared__ __align__(16) float ring[LSTAGES * (L_A_FLOATS + L_B_FLOATS)];
    auto As = [&](int buf, int r, int k) -> float* { return ring + buf * L_A_FLOATS + r * (LBK + LPAD) + k; };
    auto Bs = [&](int buf, int k, int c) -> float* { return ring + LSTAGES * L_A_FLOATS + buf * L_B_FLOATS + k * LBN + c; };
    const float* A = reinterpret_cast<const float*>(p.A);
    const float* B = reinterpret_cast<const float*>(p.B);
    const int tid = threadIdx.x, group = tid >> 7, lt = tid & 127, tx = lt & 15, ty = lt >> 4;
    const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
    const int M = p.M, N = p.N, K = p.K;
    const int steps = (K + LBK - 1) / LBK;

    auto issue = [&](int step, int buf) {
        const int k0 = step * LBK;
        if (tid < 256) {                // A: 32 rows x 8 chunks of 4 floats
            const int r = tid >> 3, kc = (tid & 7) * 4;
            const bool ok = (m0 + r) < M && (k0 + kc) < K;
            cp_async16(As(buf, r, kc), ok ? A + static_cast<size_t>(m0 + r) * K + k0 + kc : A, ok);
        }
        {                               // B: 32 k-rows x 16 chunks of 4 floats
            const int r = tid >> 4, nc = (tid & 15) * 4;
            const bool ok = (k0 + r) < K && (n0 + nc) < N;
            cp_async16(Bs(buf, r, nc), ok ? B + static_cast<size_t>(k0 + r) * N + n0 + nc : B, ok);
        }
    };

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

#pragma unroll
    for (int s = 0; s < LSTAGES - 1; ++s) { if (s < steps) issue(s, s); cp_async_commit(); }
    for (int step = 0; step < steps; ++step) {
        cp_async_wait<LSTAGES - 2>();
        __syncthreads();                       // slice `step` has landed for everyone; the slot refilled below was read last step
        const int nxt = step + LSTAGES - 1;
        if (nxt < steps) issue(nxt, nxt % LSTAGES);
        cp_async_commit();
        const int buf = step % LSTAGES;
#pragma unroll
        for (int q = 0; q < LBK / 4 / LGROUPS; ++q) {
            const int k4 = group * (LBK / 4 / LGROUPS) + q;
            float4 a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(As(buf, ty * 4 + i, k4 * 4));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) b[kk] = *reinterpret_cast<const float4*>(Bs(buf, k4 * 4 + kk, tx * 4));
#pragma unroll
            for (int i = 0; i < 4; ++i) {   // ascending k inside the group's share of the slice
                const float av[4] = {a[i].x, a[i].y, a[i].z, a[i].w};
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    acc[i][0] = fmaf(av[kk], b[kk].x, acc[i][0]); acc[i][1] = fmaf(av[kk], b[kk].y, acc[i][1]);
                    acc[i][2] = fmaf(av[kk], b[kk].z, acc[i][2]); acc[i][3] = fmaf(av[kk], b[kk].w, acc[i][3]);
                }
            }
        }
    }

    // Partial tiles through the (now idle) ring, then every thread finishes one float4 of the 32 x 64 tile.
    cp_async_wait<0>();
    __syncthreads();
    float* part = ring;                        // [group][LBM][LBN]
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(part + (group * LBM + ty * 4 + i) * LBN + tx * 4) =
            make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    __syncthreads();
    const int orow = tid >> 4, ocol = (tid & 15) * 4;
    float4 s = *reinterpret_cast<const float4*>(part + orow * LBN + ocol);
#pragma unroll
    for (int g = 1; g < LGROUPS; ++g) {
        const float4 t = *reinterpret_cast<const float4*>(part + (g * LBM + orow) * LBN + ocol);
        s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }

    float* D = reinterpret_cast<float*>(p.D);
    const float* add = reinterpret_cast<const float*>(p.add);
    const float sadd = p.add_mode == PYC_B200_ADD_SCALAR ? p.add_scale * __ldg(add) : 0.0f;
    const int r = m0 + orow, c0 = n0 + ocol;
    if (r >= M || c0 >= N) return;             // N % 4 == 0: a thread's four columns are in or out together
    float v[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[j] = p.alpha * v[j] + sadd;
        if (p.add_mode == PYC_B200_ADD_ROW_BIAS) v[j] += p.add_scale * __ldg(add + c0 + j);
        else if (p.add_mode == PYC_B200_ADD_MATRIX) v[j] += p.add_scale * __ldg(add + static_cast<size_t>(r) * N + c0 + j);
        v[j] = act_fn(v[j], p.act);
    }
    *reinterpret_cast<float4*>(D + static_cast<size_t>(r) * N + c0) = make_float4(v[0], v[1], v[2], v[3]);
}

// Throughput variant for large fp32 problems: 128 x 128 x 32 tile, 256 threads, 8 x 8 outputs per thread, two CTAs per SM,
// and the FMAs issued as packed pairs (fma.rn.f32x2: two independent IEEE fp32 FMAs per instruction, so half the issue
// slots; each lane is bit-identical to fmaf).  What bounds an fp32 GEMM on this SM next to the FMA pipe is the
// shared-memory return path (128 bytes per clock): a thread with a TM x TN register tile reads (TM + TN) * 4 bytes per
// TM * TN FMAs, so a 4 x 4 tile can feed only half of the 128 FMA lanes and an 8 x 8 tile just feeds all of them.
// Neither operand is stored twice to make the pairs: a pair of accumulators holds a DIAGONAL of a 2 x 2 block,
//   P = {C[i][j], C[i+1][j+1]} += {a_i, a_i+1} * {b_j, b_j+1},    Q = {C[i][j+1], C[i+1][j]} += {a_i, a_i+1} * {b_j+1, b_j},
// so A pairs come straight out of a 16-byte read of the transposed A tile and B needs one swapped copy in registers.
// Operands arrive by cp.async into a two-slot ring of 32-deep k-slices (one barrier per 32 k-steps; 8-deep slices cost
// 7 % in barriers): A element by element, which is what transposes it ([k][m], row stride 132 floats: the 8 k x 4 rows a
// warp copies per instruction are 4 full 32-byte sectors in global memory and 32 different banks in shared memory),
// B in 16-byte pieces.  Needs row-major B, N % 4 == 0 and 16-byte aligned B and D.  k ascends, one accumulator per output.
constexpr int XBM = 128, XBN = 128, XBK = 32, XSTAGES = 2, XTHREADS = 256, XA_STRIDE = XBM + 4;
constexpr int X_SMEM_BYTES = XSTAGES * XBK * (XA_STRIDE + XBN) * 4;

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem, bool valid) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = valid ? 4 : 0;   // 0 source bytes: the destination is zero-filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ffma2(unsigned long long& d, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__global__ void __launch_bounds__(XTHREADS, 2)
gemm_simt_x2_kernel(SimtParams p) {
    extern __shared__ __align__(16) float x_smem[];
    float (*As)[XBK][XA_STRIDE] = reinterpret_cast<float (*)[XBK][XA_STRIDE]>(x_smem);               // [slot][k][m]
    float (*Bs)[XBK][XBN] = reinterpret_cast<float (*)[XBK][XBN]>(x_smem + XSTAGES * XBK * XA_STRIDE);   // [slot][k][n]
    const float* __restrict__ A = reinterpret_cast<const float*>(p.A);
    const float* __restrict__ B = reinterpret_cast<const float*>(p.B);
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * XBM, n0 = blockIdx.x * XBN;
    const int M = p.M, N = p.N, K = p.K;
    const int steps = (K + XBK - 1) / XBK;
    const int a_k = tid & 7, a_row = tid >> 3;           // A: k = a_k + 8q, rows a_row + 32i
    const int b_row = tid >> 5, b_nc = (tid & 31) * 4;   // B: k-rows b_row + 8i, four columns from b_nc

    auto issue = [&](int step, int slot) {
        const int k0 = step * XBK;
#pragma unroll
        for (int i = 0; i < XBK / 2; ++i) {
            const int r = a_row + 32 * (i / (XBK / 8)), kq = a_k + 8 * (i % (XBK / 8));
            const bool ok = (m0 + r) < M && (k0 + kq) < K;
            cp_async4(&As[slot][kq][r], ok ? A + static_cast<size_t>(m0 + r) * K + k0 + kq : A, ok);
        }
#pragma unroll
        for (int i = 0; i < XBK / 8; ++i) {
            const int br = b_row + 8 * i;
            const bool ok = (k0 + br) < K && (n0 + b_nc) < N;
            cp_async16(&Bs[slot][br][b_nc], ok ? B + static_cast<size_t>(k0 + br) * N + n0 + b_nc : B, ok);
        }
    };

    unsigned long long P[4][4], Q[4][4];   // row pair ip: rows (ip/2)*64 + ty*4 + (ip%2)*2 + {0,1}; column pair jp: (jp/2)*64 + tx*4 + (jp%2)*2 + {0,1}
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { P[i][j] = 0ull; Q[i][j] = 0ull; }

#pragma unroll
    for (int s = 0; s < XSTAGES - 1; ++s) { if (s < steps) issue(s, s); cp_async_commit(); }
    for (int step = 0; step < steps; ++step) {
        cp_async_wait<XSTAGES - 2>();
        __syncthreads();                       // slice `step` has landed for everyone; the slot refilled below was read last step
        const int nxt = step + XSTAGES - 1;
        if (nxt < steps) issue(nxt, nxt % XSTAGES);
        cp_async_commit();
        const int slot = step % XSTAGES;
#pragma unroll
        for (int kk = 0; kk < XBK; ++kk) {
            unsigned long long ap[4], bp[4], bs[4];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(&As[slot][kk][h * 64 + ty * 4]);
                ap[h * 2] = v.x; ap[h * 2 + 1] = v.y;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float4 v = *reinterpret_cast<const float4*>(&Bs[slot][kk][h * 64 + tx * 4]);
                bp[h * 2] = pack2(v.x, v.y); bp[h * 2 + 1] = pack2(v.z, v.w);
                bs[h * 2] = pack2(v.y, v.x); bs[h * 2 + 1] = pack2(v.w, v.z);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) { ffma2(P[i][j], ap[i], bp[j]); ffma2(Q[i][j], ap[i], bs[j]); }
        }
    }

    float* D = reinterpret_cast<float*>(p.D);
    const float* add = reinterpret_cast<const float*>(p.add);
    const float sadd = p.add_mode == PYC_B200_ADD_SCALAR ? p.add_scale * __ldg(add) : 0.0f;
#pragma unroll
    for (int ip = 0; ip < 4; ++ip) {
        const int r0 = m0 + (ip >> 1) * 64 + ty * 4 + (ip & 1) * 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int c0 = n0 + h * 64 + tx * 4;
            if (c0 >= N) continue;              // N % 4 == 0: a thread's four columns are in or out together
            float v[2][4];
            unpack2(P[ip][h * 2], v[0][0], v[1][1]);     unpack2(Q[ip][h * 2], v[0][1], v[1][0]);
            unpack2(P[ip][h * 2 + 1], v[0][2], v[1][3]); unpack2(Q[ip][h * 2 + 1], v[0][3], v[1][2]);
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int r = r0 + rr;
                if (r >= M) continue;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float o = p.alpha * v[rr][j] + sadd;
                    if (p.add_mode == PYC_B200_ADD_ROW_BIAS) o += p.add_scale * __ldg(add + c0 + j);
                    else if (p.add_mode == PYC_B200_ADD_MATRIX) o += p.add_scale * __ldg(add + static_cast<size_t>(r) * N + c0 + j);
                    v[rr][j] = act_fn(o, p.act);
                }
                *reinterpret_cast<float4*>(D + static_cast<size_t>(r) * N + c0) = make_float4(v[rr][0], v[rr][1], v[rr][2], v[rr][3]);
            }
        }
    }
}

template <typename T, int BM, int BN, int TM, int TN>
int launch_one(const SimtParams& sp, cudaStream_t stream) {
    dim3 grid((sp.N + BN - 1) / BN, (sp.M + BM - 1) / BM);
    gemm_simt_kernel<T, BM, BN, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, stream>>>(sp);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

bool latency_kernel_ok(const SimtParams& sp) {
    return !sp.b_col_major && sp.K % 4 == 0 && sp.N % 4 == 0 && reinterpret_cast<uintptr_t>(sp.A) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(sp.B) % 16 == 0 && reinterpret_cast<uintptr_t>(sp.D) % 16 == 0;
}

template <typename T>
int launch_typed(const GemmConfig& cfg, const SimtParams& sp, cudaStream_t stream) {
    if constexpr (std::is_same<T, float>::value) {
        if (cfg.bm == XBM && cfg.bn == XBN && cfg.bk == XBK) {
            if (!latency_kernel_ok(sp)) { set_error("simt_x2_128x128x32 needs row-major B, K %% 4 == 0, N %% 4 == 0 and 16-byte aligned pointers"); return -1; }
            static std::atomic<bool> opted_in[64];   // the opt-in for more than 48 KB of dynamic shared memory is per device
            int dev = 0;
            B200_CUDA_OK(cudaGetDevice(&dev));
            if (dev < 0 || dev >= 64 || !opted_in[dev].load(std::memory_order_acquire)) {
                B200_CUDA_OK(cudaFuncSetAttribute(gemm_simt_x2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, X_SMEM_BYTES));
                if (dev >= 0 && dev < 64) opted_in[dev].store(true, std::memory_order_release);
            }
            dim3 grid((sp.N + XBN - 1) / XBN, (sp.M + XBM - 1) / XBM);
            gemm_simt_x2_kernel<<<grid, XTHREADS, X_SMEM_BYTES, stream>>>(sp);
            B200_CUDA_OK(cudaGetLastError());
            count_launch();
            return 0;
        }
        if (cfg.bm == 32 && cfg.bn == 64 && cfg.bk == 32) {
            if (!latency_kernel_ok(sp)) { set_error("simt_async_32x64x32 needs row-major B, K %% 4 == 0, N %% 4 == 0 and 16-byte aligned pointers"); return -1; }
            dim3 grid((sp.N + LBN - 1) / LBN, (sp.M + LBM - 1) / LBM);
            gemm_simt_latency_kernel<<<grid, LTHREADS, 0, stream>>>(sp);
            B200_CUDA_OK(cudaGetLastError());
            count_launch();
            return 0;
        }
    }
    if (cfg.bm == 128 && cfg.bn == 128) return launch_one<T, 128, 128, 8, 8>(sp, stream);
    if (cfg.bm == 64 && cfg.bn == 64) return launch_one<T, 64, 64, 4, 4>(sp, stream);
    if (cfg.bm == 32 && cfg.bn == 64) return launch_one<T, 32, 64, 2, 4>(sp, stream);
    set_error("no SIMT GEMM instance for tile %dx%d", cfg.bm, cfg.bn);
    return -1;
}

}  // namespace

int launch_gemm_simt(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream) {
    SimtParams sp;
    sp.A = p.A; sp.B = p.B; sp.D = p.D; sp.add = p.add;
    sp.M = p.M; sp.N = p.N; sp.K = p.K;
    sp.b_col_major = p.b_col_major ? 1 : 0;
    sp.add_mode = p.add ? p.add_mode : PYC_B200_ADD_NONE;
    sp.act = p.act; sp.alpha = p.alpha; sp.add_scale = p.add_scale;
    switch (p.dtype) {
        case PYC_DTYPE_F32: return launch_typed<float>(cfg, sp, stream);
        case PYC_DTYPE_BF16: return launch_typed<__nv_bfloat16>(cfg, sp, stream);
        case PYC_DTYPE_F16: return launch_typed<__half>(cfg, sp, stream);
        default: set_error("SIMT GEMM: unsupported dtype %d", static_cast<int>(p.dtype)); return -1;
    }
}

}  // namespace b200
