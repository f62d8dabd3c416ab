// NHWC forward convolution as an implicit GEMM on the tcgen05 tensor cores, with
// a fused bias + ReLU epilogue.
//
// Replaces PyC's CUTLASS sm80 implicit-GEMM kernel
// (src/compiler/cutlass_kernels/conv2d/kernel.cu:24-44, dispatch :80-111; fp16
// only there, no epilogue).  Problem definition as PyC hands it to CUTLASS at
// conv2d/kernel.cu:92-98: input [N,H,W,C], filter [K,R,S,C], cross-correlation,
// symmetric padding, dilation 1, groups 1, output [N,P,Q,K].
//
// GEMM view: M = N*P*Q output pixels, N = K filters, K = R*S*C.  No im2col
// buffer exists anywhere.  An M-tile is a TN x TP x TQ brick of 128 output pixels
// (brick shape picked per problem so that it tiles P, Q, N with the least
// waste); for filter tap (r,s) and a 64-channel slice its A operand is ONE 4-D
// TMA box of the input at (c0, q0-pad+s, p0-pad+r, n0): rows that fall into the
// padding are out of bounds for the tensor map and arrive as zeros.  The B
// operand is a [BN x 64] K-major box of the filter.  Everything after the loads
// (tcgen05.mma into TMEM, double-buffered accumulators, epilogue warps) has the
// structure of the GEMM kernel in gemm_tc.cu.  Stride-1 convolutions with
// C % 8 == 0 take this path; anything else runs the direct kernel below.
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "internal.h"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;

struct ConvParams {
    int N, H, W, C, K, R, S, pad_h, pad_w, P, Q;
    int tq, tp, tn;            // brick extents (powers of two, tq*tp*tn == 128)
    int tiles_q, tiles_p, tiles_n_img, tiles_k;
    const void* bias;
    void* out;
    int relu;
};

template <int FMT> struct CElem;
template <> struct CElem<1> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float to_f(T v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T from_f(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { __nv_bfloat162 p = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&p); }
};
template <> struct CElem<0> {
    using T = __half;
    static __device__ __forceinline__ float to_f(T v) { return __half2float(v); }
    static __device__ __forceinline__ T from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { __half2 p = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&p); }
};

template <int BN, int STAGES, int FMT, int CTAS_PER_SM>
__global__ void __launch_bounds__(192, CTAS_PER_SM)
conv2d_tc_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW, ConvParams cp, int* status) {
    constexpr int B_STAGE_BYTES = BN * BK * 2;
    constexpr uint32_t STAGE_TX = A_STAGE_BYTES + B_STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr uint32_t IDESC = make_idesc(FMT, FMT, 0, 0, BM, BN);
    using E = CElem<FMT>;
    using T = typename E::T;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = cp.tiles_q * cp.tiles_p * cp.tiles_n_img;
    const int num_tiles = tiles_m * cp.tiles_k;
    const int c_chunks = (cp.C + BK - 1) / BK;
    const int num_kb = cp.R * cp.S * c_chunks;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmIn);
        prefetch_tmap(&tmW);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    // tile -> (filter block kt, brick origin n0,p0,q0); filter blocks of the same brick are adjacent
    auto tile_origin = [&](int tile, int& kt, int& n0, int& p0, int& q0) {
        kt = tile % cp.tiles_k;
        int mt = tile / cp.tiles_k;
        q0 = (mt % cp.tiles_q) * cp.tq; mt /= cp.tiles_q;
        p0 = (mt % cp.tiles_p) * cp.tp; mt /= cp.tiles_p;
        n0 = mt * cp.tn;
    };

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t a_dst0 = smem_u32(sA), b_dst0 = smem_u32(sB);
            uint32_t stage = 0, phase = 0, adst = a_dst0, bdst = b_dst0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int kt, n0, p0, q0;
                tile_origin(tile, kt, n0, p0, q0);
                // k-block kb = (r * S + s) * c_chunks + cc, walked with counters instead of divisions
                int cc = 0, s = 0, r = 0, rs = 0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, status, 0x11)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * stage;
                    mbar_arrive_expect_tx(fb, STAGE_TX);
                    tma_load_4d(adst, &tmIn, fb, cc * BK, q0 - cp.pad_w + s, p0 - cp.pad_h + r, n0);
                    tma_load_3d(bdst, &tmW, fb, cc * BK, rs, kt * BN);
                    if (++cc == c_chunks) { cc = 0; ++rs; if (++s == cp.S) { s = 0; ++r; } }
                    adst += A_STAGE_BYTES; bdst += B_STAGE_BYTES;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; adst = a_dst0; bdst = b_dst0; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // constant descriptor high word, stepped low words (this thread shares its scheduler with an epilogue warp)
            constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 16), b_lo0 = smem_desc_lo(smem_u32(sB), 16);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, status, 0x12)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, status, 0x13)) { ok = false; break; }
                    tc_fence_after();
                    umma_f16(d_tmem, smem_desc_join(a_lo, DESC_HI), smem_desc_join(b_lo, DESC_HI), IDESC, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k4 = 1; k4 < BK / 16; ++k4)
                        umma_f16(d_tmem, smem_desc_join(a_lo + k4 * 2, DESC_HI), smem_desc_join(b_lo + k4 * 2, DESC_HI), IDESC, 1u);
                    umma_commit(empty0 + 8 * stage);
                    a_lo += A_STAGE_BYTES >> 4; b_lo += B_STAGE_BYTES >> 4;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                }
                if (ok) umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int wq = warp & 3;
        int it = 0;
        const T* bias = reinterpret_cast<const T*>(cp.bias);
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            int kt, n0, p0, q0;
            tile_origin(tile, kt, n0, p0, q0);
            // row m of the brick: q fastest, then p, then image (the order the TMA box lands in shared memory)
            const int m = wq * 32 + lane;
            const int q = q0 + (m % cp.tq), p = p0 + (m / cp.tq) % cp.tp, n = n0 + m / (cp.tq * cp.tp);
            const bool row_ok = q < cp.Q && p < cp.P && n < cp.N;
            T* orow = reinterpret_cast<T*>(cp.out) + ((static_cast<size_t>(n) * cp.P + p) * cp.Q + q) * cp.K;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase, status, 0x14)) break;
            tc_fence_after();
            const bool vec_ok = (cp.K % 8 == 0) && (reinterpret_cast<uintptr_t>(cp.out) % 16 == 0);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t rr[32];
                tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + acc * BN + c * 32, rr);
                tmem_ld_wait();
                const int col0 = kt * BN + c * 32;  // warp-uniform
                if (col0 < cp.K && row_ok) {         // lanes outside the image only skip the stores; every lane stays in the loop
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rr[j]);
                    if (bias) {
                        if (vec_ok && col0 + 32 <= cp.K && reinterpret_cast<uintptr_t>(bias) % 16 == 0) {
#pragma unroll
                            for (int qd = 0; qd < 4; ++qd) {  // 16-byte loads, the same address in every lane
                                union { uint4 u; T t[8]; } b;
                                b.u = __ldg(reinterpret_cast<const uint4*>(bias + col0) + qd);
#pragma unroll
                                for (int t = 0; t < 8; ++t) v[qd * 8 + t] += E::to_f(b.t[t]);
                            }
                        } else {
                            for (int j = 0; j < 32; ++j) if (col0 + j < cp.K) v[j] += E::to_f(bias[col0 + j]);
                        }
                    }
                    if (cp.relu) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
                    }
                    if (vec_ok && col0 + 32 <= cp.K) {
                        uint4* dst = reinterpret_cast<uint4*>(orow + col0);
#pragma unroll
                        for (int qd = 0; qd < 4; ++qd) {
                            uint4 u;
                            u.x = E::pack(v[qd * 8 + 0], v[qd * 8 + 1]); u.y = E::pack(v[qd * 8 + 2], v[qd * 8 + 3]);
                            u.z = E::pack(v[qd * 8 + 4], v[qd * 8 + 5]); u.w = E::pack(v[qd * 8 + 6], v[qd * 8 + 7]);
                            dst[qd] = u;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j) if (col0 + j < cp.K) orow[col0 + j] = E::from_f(v[j]);
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(status) != ST_OK) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Direct convolution for everything the tensor-core path does not take (stride != 1,
// C % 8 != 0, fp32): one thread per output element, fp32 accumulate in (r,s,c) order.
__device__ __forceinline__ float cld(const float* p) { return __ldg(p); }
__device__ __forceinline__ float cld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float cld(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void cst(float* p, float v) { *p = v; }
__device__ __forceinline__ void cst(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void cst(__half* p, float v) { *p = __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
conv2d_direct_kernel(const T* __restrict__ in, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ out,
                     int N, int H, int W, int C, int K, int R, int S, int pad_h, int pad_w, int sh, int sw, int P, int Q, int relu) {
    const size_t total = static_cast<size_t>(N) * P * Q * K;
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int k = static_cast<int>(idx % K);
        size_t pix = idx / K;
        const int q = static_cast<int>(pix % Q); pix /= Q;
        const int p = static_cast<int>(pix % P);
        const int n = static_cast<int>(pix / P);
        float acc = 0.0f;
        for (int r = 0; r < R; ++r) {
            const int h = p * sh - pad_h + r;
            if (h < 0 || h >= H) continue;
            for (int s = 0; s < S; ++s) {
                const int x = q * sw - pad_w + s;
                if (x < 0 || x >= W) continue;
                const T* ip = in + ((static_cast<size_t>(n) * H + h) * W + x) * C;
                const T* wp = w + ((static_cast<size_t>(k) * R + r) * S + s) * C;
                for (int c = 0; c < C; ++c) acc = fmaf(cld(ip + c), cld(wp + c), acc);
            }
        }
        if (bias) acc += cld(bias + k);
        if (relu) acc = fmaxf(acc, 0.0f);
        cst(out + idx, acc);
    }
}

template <int BN, int STAGES>
constexpr size_t conv_smem_bytes() { return 1024 + static_cast<size_t>(STAGES) * (A_STAGE_BYTES + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16; }

template <int BN, int STAGES, int FMT, int CTAS_PER_SM = 1>
int launch_conv_tc(const CUtensorMap& tmIn, const CUtensorMap& tmW, const ConvParams& cp, cudaStream_t stream, int* status) {
    auto kernel = conv2d_tc_kernel<BN, STAGES, FMT, CTAS_PER_SM>;
    constexpr size_t smem = conv_smem_bytes<BN, STAGES>();
    static std::atomic<bool> attr_set[16];   // zero-initialised; set-once per device, a repeated set is harmless
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 16 && !attr_set[dev]) {
        B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_set[dev] = true;
    }
    const int tiles = cp.tiles_q * cp.tiles_p * cp.tiles_n_img * cp.tiles_k;
    const int slots = sm_count() * CTAS_PER_SM;
    kernel<<<tiles < slots ? tiles : slots, 192, smem, stream>>>(tmIn, tmW, cp, status);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

template <typename T>
int launch_direct(const void* in, const void* w, const void* bias, void* out, int N, int H, int W, int C, int K, int R, int S,
                  int pad_h, int pad_w, int sh, int sw, int P, int Q, int relu, cudaStream_t stream) {
    const size_t total = static_cast<size_t>(N) * P * Q * K;
    size_t blocks = (total + 255) / 256;
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    conv2d_direct_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const T*>(in), static_cast<const T*>(w), static_cast<const T*>(bias),
                                                                              static_cast<T*>(out), N, H, W, C, K, R, S, pad_h, pad_w, sh, sw, P, Q, relu);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

}  // namespace

int launch_conv2d(pyc_dtype dt, int N, int H, int W, int C, int K, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w,
                  const void* in, const void* filt, const void* bias, int relu, void* out, cudaStream_t stream, int* status) {
    if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0 || pad_h < 0 || pad_w < 0 || !in || !filt || !out) {
        set_error("conv2d: bad shape or NULL pointer"); return -1;
    }
    const int P = (H - R + 2 * pad_h) / stride_h + 1, Q = (W - S + 2 * pad_w) / stride_w + 1;
    if (P <= 0 || Q <= 0) { set_error("conv2d: empty output"); return -1; }
    const bool tc = (dt == PYC_DTYPE_BF16 || dt == PYC_DTYPE_F16) && stride_h == 1 && stride_w == 1 && C % 8 == 0 && status &&
                    reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(filt) % 16 == 0;
    if (!tc) {
        switch (dt) {
            case PYC_DTYPE_F32: return launch_direct<float>(in, filt, bias, out, N, H, W, C, K, R, S, pad_h, pad_w, stride_h, stride_w, P, Q, relu, stream);
            case PYC_DTYPE_BF16: return launch_direct<__nv_bfloat16>(in, filt, bias, out, N, H, W, C, K, R, S, pad_h, pad_w, stride_h, stride_w, P, Q, relu, stream);
            case PYC_DTYPE_F16: return launch_direct<__half>(in, filt, bias, out, N, H, W, C, K, R, S, pad_h, pad_w, stride_h, stride_w, P, Q, relu, stream);
            default: set_error("conv2d: unsupported dtype %d", static_cast<int>(dt)); return -1;
        }
    }
    ConvParams cp;
    // Brick of 128 output pixels: powers of two tq*tp*tn == 128 with the least padding waste; ties go to the widest row run.
    double best = -1.0;
    for (int tq = 128; tq >= 1; tq >>= 1)
        for (int tp = 128 / tq; tp >= 1; tp >>= 1) {
            const int tn = 128 / (tq * tp);
            const double util = static_cast<double>(Q) / (((Q + tq - 1) / tq) * tq) * P / (((P + tp - 1) / tp) * tp) * N / (((N + tn - 1) / tn) * tn);
            if (util > best + 1e-9) { best = util; cp.tq = tq; cp.tp = tp; cp.tn = tn; }
        }
    cp.N = N; cp.H = H; cp.W = W; cp.C = C; cp.K = K; cp.R = R; cp.S = S; cp.pad_h = pad_h; cp.pad_w = pad_w; cp.P = P; cp.Q = Q;
    cp.tiles_q = (Q + cp.tq - 1) / cp.tq; cp.tiles_p = (P + cp.tp - 1) / cp.tp; cp.tiles_n_img = (N + cp.tn - 1) / cp.tn;
    cp.bias = bias; cp.out = out; cp.relu = relu;
    const int bn = K <= 64 ? 64 : K <= 128 ? 128 : 256;
    cp.tiles_k = (K + bn - 1) / bn;

    CUtensorMap tmIn, tmW;
    const uint64_t in_dims[4] = {static_cast<uint64_t>(C), static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(N)};
    const uint64_t in_str[3] = {static_cast<uint64_t>(C) * 2, static_cast<uint64_t>(W) * C * 2, static_cast<uint64_t>(H) * W * C * 2};
    const uint32_t in_box[4] = {BK, static_cast<uint32_t>(cp.tq), static_cast<uint32_t>(cp.tp), static_cast<uint32_t>(cp.tn)};
    if (encode_tmap(&tmIn, in, 2, 4, in_dims, in_str, in_box, true) != 0) return -1;
    const uint64_t w_dims[3] = {static_cast<uint64_t>(C), static_cast<uint64_t>(R) * S, static_cast<uint64_t>(K)};
    const uint64_t w_str[2] = {static_cast<uint64_t>(C) * 2, static_cast<uint64_t>(R) * S * C * 2};
    const uint32_t w_box[3] = {BK, 1, static_cast<uint32_t>(bn)};
    if (encode_tmap(&tmW, filt, 2, 3, w_dims, w_str, w_box, true) != 0) return -1;

    const bool bf16 = dt == PYC_DTYPE_BF16;
    // 64 filters: two CTAs per SM (4-stage rings, 128 TMEM columns each).  With N = 64 an MMA reads 6 KB of operands from
    // shared memory for 32 cycles of math, and a cycle-stamp timeline shows ~83 cycles per 128x64x16 MMA: the kernel is bound
    // by the operand reads, not by its loads (a variant that fetched each input brick once with its halo, a third of the
    // L2 traffic, ran at the same 30 us on 64 x 56 x 56 x 64) -- the second CTA fills the gaps between tiles: 36 -> 31 us.
    if (bn == 64) return bf16 ? launch_conv_tc<64, 4, 1, 2>(tmIn, tmW, cp, stream, status) : launch_conv_tc<64, 4, 0, 2>(tmIn, tmW, cp, stream, status);
    if (bn == 128) return bf16 ? launch_conv_tc<128, 6, 1>(tmIn, tmW, cp, stream, status) : launch_conv_tc<128, 6, 0>(tmIn, tmW, cp, stream, status);
    return bf16 ? launch_conv_tc<256, 4, 1>(tmIn, tmW, cp, stream, status) : launch_conv_tc<256, 4, 0>(tmIn, tmW, cp, stream, status);
}

}  // namespace b200

extern "C" {

int pyc_b200_conv2d(pyc_dtype dtype, int N, int H, int W, int C_in, int K, int R, int S, int pad_h, int pad_w, int stride_h, int stride_w,
                    const void* input, const void* filter, const void* bias, int relu, void* output, void* stream) {
    return b200::launch_conv2d(dtype, N, H, W, C_in, K, R, S, pad_h, pad_w, stride_h, stride_w, input, filter, bias, relu, output,
                               static_cast<cudaStream_t>(stream), b200::device_status_word());
}

int pyc_cutlass_conv2d_dispatch(const char* symbol, int N, int H, int W, int C_in, int K, int R, int S, int pad_h, int pad_w,
                                int stride_h, int stride_w, const void* input, const void* filter, void* output, void* stream) {
    if (!symbol) return -1;
    pyc_dtype dt;
    if (!strcmp(symbol, "b200_conv2d_fprop_bf16") || !strcmp(symbol, "cutlass_conv2d_fprop_bf16")) dt = PYC_DTYPE_BF16;
    else if (!strcmp(symbol, "b200_conv2d_fprop_f16") || !strcmp(symbol, "cutlass_conv2d_fprop_f16")) dt = PYC_DTYPE_F16;
    else if (!strcmp(symbol, "b200_conv2d_fprop_f32")) dt = PYC_DTYPE_F32;
    else { b200::set_error("unknown conv2d symbol %s", symbol); return -1; }
    return pyc_b200_conv2d(dt, N, H, W, C_in, K, R, S, pad_h, pad_w, stride_h, stride_w, input, filter, nullptr, 0, output, stream);
}

}  // extern "C"
