// Fused attention forward: Out = softmax(scale * Q K^T [+ causal mask]) V, online
// softmax with fp32 statistics, both contractions on the tcgen05 tensor cores.
//
// Replaces PyC's attention "kernel", whose body copies Q to the output
// (src/compiler/cutlass_kernels/attention/kernel.cu:30-59); the definition
// implemented here is the one in that file's header comment (:6-8), with an
// optional causal mask (key index <= query index).
//
// One CTA per (batch*head, block of 128 queries), 192 threads:
//   warp 0     TMA producer: Q once, then K and V blocks of 128 keys (2-deep rings)
//   warp 1     TMEM owner + single-thread MMA issuer:
//                S[j&1] = Q K_j^T        (128x128xD,  S in TMEM, double buffered)
//                O     += P_j V_j        (128xDx128,  O in TMEM, V as MN-major operand)
//   warps 2-5  softmax, one query row per thread: S row from TMEM (two passes of
//              32-column chunks: max, then exp2/sum), P_j -> bf16 -> shared memory
//              in the 128-byte-swizzled K-major operand layout, O rescaled in TMEM
//              only when some row's running max moved.
// QK^T of block j+1 is issued before the issuer waits for P_j, so the tensor pipe
// works under the softmax of block j.  Causal blocks above the diagonal are never
// loaded or multiplied.  Every wait is bounded (status word, see ptx_sm100.cuh).
//
// Layout: Q, K, V, Out are [batch_heads, seq, d] contiguous; tensor maps are 3-D
// (d, seq, batch_heads) so rows past `seq` read as zeros instead of the next head.
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>
#include <string.h>

#include "internal.h"
#include "math.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int BQ = 128;   // queries per CTA
constexpr int BKV = 128;  // keys per block

template <int FMT> struct AElem;
template <> struct AElem<1> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ uint32_t pack(float a, float b) { __nv_bfloat162 p = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&p); }
};
template <> struct AElem<0> {
    using T = __half;
    static __device__ __forceinline__ uint32_t pack(float a, float b) { __half2 p = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&p); }
};

// 2^x on the MUFU in one instruction (flush-to-zero; exp2f() adds range handling the softmax does not need:
// arguments are <= 0 up to the lazy-rescale margin and -inf gives 0).
// max of three in one instruction (sm_100 max.f32 with three sources)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x on the FMA pipe for x <= 0 (Cody-Waite split + cubic on the fraction, relative error 7.5e-5, well inside what the
// 16-bit P keeps).  The softmax is co-limited by the MUFU (16 exp2 per clock per SM), so a fixed share of the elements
// takes this route instead.
__device__ __forceinline__ float poly_exp2(float x) {
    x = fmaxf(x, -126.0f);
    const float magic = 12582912.0f;                 // 1.5 * 2^23: adding it rounds x to the nearest integer in the low mantissa bits
    const float t = x + magic;
    const float f = x - (t - magic);                 // fraction in [-0.5, 0.5]
    float p = fmaf(0.05517165f, f, 0.24261113f);     // cubic fitted for minimum relative error of 2^f on [-0.5, 0.5]: 7.5e-5
    p = fmaf(p, f, 0.69326097f);
    p = fmaf(p, f, 0.99992806f);
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));   // scale by 2^round(x): add to the exponent field
}

struct AttnParams {
    int seq, batch_heads, causal;
    float scale_log2;  // scale * log2(e)
    void* out;
};

// Shared-memory map (HD = 128): Q 32 KB | K 2 x 32 KB | V 2 x 32 KB | P 32 KB | barriers
template <int HD>
struct AttnSmem {
    static constexpr int TILE = BQ * HD * 2;       // one [128 x HD] 16-bit tile
    static constexpr int P_BYTES = BQ * BKV * 2;
    static constexpr int Q_OFF = 0, K_OFF = TILE, V_OFF = 3 * TILE, P_OFF = 5 * TILE, BAR_OFF = 5 * TILE + P_BYTES;
    static constexpr int NUM_BARS = 16;
    static constexpr size_t BYTES = 1024 + BAR_OFF + NUM_BARS * 8 + 16;
};

template <int HD, int FMT>
__global__ void __launch_bounds__(192, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, AttnParams ap, int* status) {
    using SM = AttnSmem<HD>;
    using E = AElem<FMT>;
    using T = typename E::T;
    constexpr int HALVES = HD / 64;                 // 64-column (128-byte) operand slabs per tile
    constexpr int HALF_BYTES = BQ * 128;            // [128 rows x 128 B]
    constexpr uint32_t IDESC_QK = make_idesc(FMT, FMT, 0, 0, BQ, BKV);
    constexpr uint32_t IDESC_PV = make_idesc(FMT, FMT, 0, 1, BQ, HD);
    constexpr uint32_t TMEM_COLS = 512;             // S0 @0, S1 @128, O @256
    constexpr uint32_t O_COL = 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SM::NUM_BARS);
    const uint32_t bar0 = smem_u32(bars);
    // barrier indices
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 24, v_full = bar0 + 40, v_empty = bar0 + 56,
                   s_full = bar0 + 72, s_empty = bar0 + 88, p_full = bar0 + 104, pv_done = bar0 + 112;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_qb = (ap.seq + BQ - 1) / BQ;
    const int qb = num_qb - 1 - static_cast<int>(blockIdx.x);  // longest (causal) blocks first
    const int bh = blockIdx.y;
    const int q0 = qb * BQ;
    const int kv_blocks_all = (ap.seq + BKV - 1) / BKV;
    const int nblk = ap.causal ? min(kv_blocks_all, qb + 1) : kv_blocks_all;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + 8 * i, 1); mbar_init(k_empty + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1); mbar_init(v_empty + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1); mbar_init(s_empty + 8 * i, 4);
        }
        mbar_init(p_full, 4);
        mbar_init(pv_done, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const uint32_t sQ = smem_u32(smem + SM::Q_OFF), sK = smem_u32(smem + SM::K_OFF), sV = smem_u32(smem + SM::V_OFF), sP = smem_u32(smem + SM::P_OFF);

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, SM::TILE);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) tma_load_3d(sQ + h * HALF_BYTES, &tmQ, q_full, h * 64, q0, bh);
            for (int j = 0; j < nblk; ++j) {
                const int st = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;
                if (!mbar_wait(k_empty + 8 * st, par, status, 0x21)) break;
                mbar_arrive_expect_tx(k_full + 8 * st, SM::TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sK + st * SM::TILE + h * HALF_BYTES, &tmK, k_full + 8 * st, h * 64, j * BKV, bh);
                if (!mbar_wait(v_empty + 8 * st, par, status, 0x22)) break;
                mbar_arrive_expect_tx(v_full + 8 * st, SM::TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sV + st * SM::TILE + h * HALF_BYTES, &tmV, v_full + 8 * st, h * 64, j * BKV, bh);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            auto issue_qk = [&](int j) {  // S[j&1] = Q K_j^T
                const int st = j & 1;
                const uint32_t d = tmem_base + (j & 1) * BKV;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t off = (ks / 4) * HALF_BYTES + (ks % 4) * 32;
                    umma_f16(d, make_smem_desc_sw128(sQ + off, 16, 1024), make_smem_desc_sw128(sK + st * SM::TILE + off, 16, 1024), IDESC_QK, ks != 0);
                }
                umma_commit(s_full + 8 * (j & 1));
                umma_commit(k_empty + 8 * st);
            };
            bool ok = mbar_wait(q_full, 0, status, 0x23) && mbar_wait(k_full, 0, status, 0x24);
            if (ok) { tc_fence_after(); issue_qk(0); }
            for (int j = 0; j < nblk && ok; ++j) {
                if (j + 1 < nblk) {
                    const int jn = j + 1;
                    if (!mbar_wait(k_full + 8 * (jn & 1), (jn >> 1) & 1, status, 0x25)) { ok = false; break; }
                    if (!mbar_wait(s_empty + 8 * (jn & 1), ((jn >> 1) & 1) ^ 1, status, 0x26)) { ok = false; break; }
                    tc_fence_after();
                    issue_qk(jn);
                }
                const int st = j & 1;
                if (!mbar_wait(v_full + 8 * st, (j >> 1) & 1, status, 0x27)) { ok = false; break; }
                if (!mbar_wait(p_full, j & 1, status, 0x28)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < BKV / 16; ++ks) {  // O += P_j V_j
                    const uint64_t adesc = make_smem_desc_sw128(sP + (ks / 4) * HALF_BYTES + (ks % 4) * 32, 16, 1024);
                    const uint64_t bdesc = make_smem_desc_sw128(sV + st * SM::TILE + ks * 2048, HALF_BYTES, 1024);
                    umma_f16(tmem_base + O_COL, adesc, bdesc, IDESC_PV, (j | ks) != 0 ? 1u : 0u);
                }
                umma_commit(v_empty + 8 * st);
                umma_commit(pv_done);
            }
        }
    } else {
        const int wq = warp & 3;
        const int row = wq * 32 + lane;            // query row inside the block == TMEM lane
        const int qi = q0 + row;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (int j = 0; j < nblk && ok; ++j) {
            const uint32_t s_addr = lane_addr + (j & 1) * BKV;
            if (!mbar_wait(s_full + 8 * (j & 1), (j >> 1) & 1, status, 0x29)) { ok = false; break; }
            tc_fence_after();
            const int k0 = j * BKV;
            // keys this row may see in this block: [k0, k_lim)
            int k_lim = ap.seq;
            if (ap.causal) k_lim = min(k_lim, qi + 1);
            // pass 1: row max
            float m_blk = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(s_addr + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 32; ++t) if (k0 + c * 32 + t < k_lim) m_blk = fmaxf(m_blk, __uint_as_float(r[t]));
            }
            m_blk *= ap.scale_log2;  // scale > 0: max commutes with the scaling
            const float m_new = fmaxf(m_run, m_blk);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;  // fully masked so far: keep exp2 arguments finite
            const float alpha = exp2f(m_run - m_use);                // m_run = -inf -> 0
            // P and O are shared with the previous block's P*V: wait until it has finished.
            if (j > 0 && !mbar_wait(pv_done, (j - 1) & 1, status, 0x2a)) { ok = false; break; }
            tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {  // rescale this warp's 32 rows of O in TMEM
#pragma unroll 1
                for (int c = 0; c < HD / 16; ++c) {
                    uint32_t o[16];
                    tmem_ld_32x16(lane_addr + O_COL + c * 16, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int t = 0; t < 16; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * alpha);
                    tmem_st_32x16(lane_addr + O_COL + c * 16, o);
                }
                tmem_st_wait();
            }
            // pass 2: exponentiate, sum, write P (16-bit) into the swizzled K-major operand tile
            float l_blk = 0.0f;
#pragma unroll 1
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(s_addr + c * 32, r);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int t = 0; t < 32; t += 2) {
                    const int kk = k0 + c * 32 + t;
                    const float p0 = kk < k_lim ? exp2f(__uint_as_float(r[t]) * ap.scale_log2 - m_use) : 0.0f;
                    const float p1 = kk + 1 < k_lim ? exp2f(__uint_as_float(r[t + 1]) * ap.scale_log2 - m_use) : 0.0f;
                    l_blk += p0 + p1;
                    packed[t / 2] = E::pack(p0, p1);
                }
                // columns c*32 .. c*32+31 of row `row`: slab = c/2, 16-byte chunks (c%2)*4 .. +3, XOR-swizzled by row%8
                const uint32_t base = sP + (c / 2) * HALF_BYTES + row * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint32_t chunk = static_cast<uint32_t>(((c & 1) * 4 + q4) ^ (row & 7));
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + chunk * 16), "r"(packed[q4 * 4 + 0]), "r"(packed[q4 * 4 + 1]),
                                 "r"(packed[q4 * 4 + 2]), "r"(packed[q4 * 4 + 3]) : "memory");
                }
            }
            l_run = l_run * alpha + l_blk;
            m_run = m_new;
            fence_proxy_async();   // P (generic-proxy stores) must be visible to the tensor core's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(s_empty + 8 * (j & 1)); mbar_arrive(p_full); }
        }
        // epilogue: O / l -> 16-bit -> global
        if (ok && mbar_wait(pv_done, (nblk - 1) & 1, status, 0x2b)) {
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            T* orow = reinterpret_cast<T*>(ap.out) + (static_cast<size_t>(bh) * ap.seq + qi) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + O_COL + c * 32, r);
                tmem_ld_wait();
                if (qi < ap.seq) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 u;
                        u.x = E::pack(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
                        u.y = E::pack(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
                        u.z = E::pack(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
                        u.w = E::pack(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
                        dst[q4] = u;
                    }
                }
                __syncwarp();
            }
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

// ---------------------------------------------------------------------------------------
// Second kernel: the same computation arranged so that TWO CTAs fit on one SM and cover
// each other's softmax time with their tensor-core work.  Differences from the kernel
// above: key blocks of 64 (K/V stages of 16 KB, 96 KB of shared memory per CTA), 256
// TMEM columns per CTA (S0 | S1 | O), each softmax thread reads its 64 scores ONCE, and
// P never goes through shared memory: it is written back into the TMEM columns its scores
// came from (packed 2 x 16 bit per column) and the P*V product takes its A operand from
// TMEM.  S[j&1] cannot be overwritten by Q*K^T of block j+2 before P*V of block j has read
// it because both are issued, in that order, by the same thread to the in-order MMA pipe.
// ---------------------------------------------------------------------------------------
constexpr int BKV2 = 64;

template <int HD>
struct AttnSmem2 {
    static constexpr int Q_BYTES = BQ * HD * 2;
    static constexpr int KV_TILE = BKV2 * HD * 2;      // one [64 x HD] tile
    static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = Q_BYTES + 2 * KV_TILE, BAR_OFF = Q_BYTES + 4 * KV_TILE;
    static constexpr int NUM_BARS = 14;
    static constexpr size_t BYTES = 1024 + BAR_OFF + NUM_BARS * 8 + 16;
};

template <int HD, int FMT, bool POLY>
__global__ void __launch_bounds__(192, 2)
attention_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, AttnParams ap, int* status) {
    using SM = AttnSmem2<HD>;
    using E = AElem<FMT>;
    using T = typename E::T;
    constexpr int HALVES = HD / 64;
    constexpr int Q_SLAB = BQ * 128;                 // [128 rows x 128 B]
    constexpr int KV_SLAB = BKV2 * 128;              // [64 rows x 128 B]
    constexpr uint32_t IDESC_QK = make_idesc(FMT, FMT, 0, 0, BQ, BKV2);
    constexpr uint32_t IDESC_PV = make_idesc(FMT, FMT, 0, 1, BQ, HD);
    constexpr uint32_t TMEM_COLS = 256;              // S0 @0, S1 @64, O @128
    constexpr uint32_t O_COL = 128;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SM::NUM_BARS);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 24, v_full = bar0 + 40, v_empty = bar0 + 56,
                   s_full = bar0 + 72, p_full = bar0 + 88, pv_done = bar0 + 104;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_qb = (ap.seq + BQ - 1) / BQ;
    const int qb = num_qb - 1 - static_cast<int>(blockIdx.x);
    const int bh = blockIdx.y;
    const int q0 = qb * BQ;
    const int kv_blocks_all = (ap.seq + BKV2 - 1) / BKV2;
    const int nblk = ap.causal ? min(kv_blocks_all, (q0 + BQ + BKV2 - 1) / BKV2) : kv_blocks_all;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + 8 * i, 1); mbar_init(k_empty + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1); mbar_init(v_empty + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1); mbar_init(p_full + 8 * i, 4);
        }
        mbar_init(pv_done, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const uint32_t sQ = smem_u32(smem + SM::Q_OFF), sK = smem_u32(smem + SM::K_OFF), sV = smem_u32(smem + SM::V_OFF);

    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
            for (int h = 0; h < HALVES; ++h) tma_load_3d(sQ + h * Q_SLAB, &tmQ, q_full, h * 64, q0, bh);
            for (int j = 0; j < nblk; ++j) {
                const int st = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;
                if (!mbar_wait(k_empty + 8 * st, par, status, 0x51)) break;
                mbar_arrive_expect_tx(k_full + 8 * st, SM::KV_TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sK + st * SM::KV_TILE + h * KV_SLAB, &tmK, k_full + 8 * st, h * 64, j * BKV2, bh);
                if (!mbar_wait(v_empty + 8 * st, par, status, 0x52)) break;
                mbar_arrive_expect_tx(v_full + 8 * st, SM::KV_TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sV + st * SM::KV_TILE + h * KV_SLAB, &tmV, v_full + 8 * st, h * 64, j * BKV2, bh);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // Descriptor high words are constants and the low words differ from a per-stage base by compile-time steps, so
            // an MMA costs this thread one add besides its own issue: the thread shares its scheduler with softmax warps.
            constexpr uint32_t HI_K = smem_desc_hi_sw128(1024);
            const uint32_t q_lo = smem_desc_lo(sQ, 16), k_lo0 = smem_desc_lo(sK, 16), v_lo0 = smem_desc_lo(sV, KV_SLAB);
            auto issue_qk = [&](int j) {  // S[j&1] = Q K_j^T, 128 x 64 x HD
                const int st = j & 1;
                const uint32_t d = tmem_base + (j & 1) * BKV2;
                const uint32_t k_lo = k_lo0 + st * (SM::KV_TILE >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma_f16(d, smem_desc_join(q_lo + (((ks / 4) * Q_SLAB + (ks % 4) * 32) >> 4), HI_K),
                             smem_desc_join(k_lo + (((ks / 4) * KV_SLAB + (ks % 4) * 32) >> 4), HI_K), IDESC_QK, ks != 0);
                umma_commit(s_full + 8 * (j & 1));
                umma_commit(k_empty + 8 * st);
            };
            bool ok = mbar_wait(q_full, 0, status, 0x53);
            for (int j = 0; j < 2 && j < nblk && ok; ++j) {   // two score blocks in flight before the first P arrives
                if (!mbar_wait(k_full + 8 * (j & 1), 0, status, 0x54)) { ok = false; break; }
                tc_fence_after();
                issue_qk(j);
            }
            for (int j = 0; j < nblk && ok; ++j) {
                const int st = j & 1;
                if (!mbar_wait(v_full + 8 * st, (j >> 1) & 1, status, 0x55)) { ok = false; break; }
                if (!mbar_wait(p_full + 8 * (j & 1), (j >> 1) & 1, status, 0x56)) { ok = false; break; }
                tc_fence_after();
                const uint32_t p_tmem = tmem_base + (j & 1) * BKV2;   // P_j sits where S_j was: 32 columns of packed pairs
                const uint32_t v_lo = v_lo0 + st * (SM::KV_TILE >> 4);
#pragma unroll
                for (int ks = 0; ks < BKV2 / 16; ++ks)  // O += P_j V_j : 128 x HD x 64, A from TMEM (8 columns per 16 keys)
                    umma_f16_ts(tmem_base + O_COL, p_tmem + ks * 8, smem_desc_join(v_lo + ks * (2048 >> 4), HI_K),
                                IDESC_PV, (j | ks) != 0 ? 1u : 0u);
                umma_commit(v_empty + 8 * st);
                umma_commit(pv_done);
                if (j + 2 < nblk) {   // S[j&1] is free again once P*V of block j is in the pipe ahead of this
                    const int jn = j + 2;
                    if (!mbar_wait(k_full + 8 * (jn & 1), (jn >> 1) & 1, status, 0x57)) { ok = false; break; }
                    tc_fence_after();
                    issue_qk(jn);
                }
            }
        }
    } else {
        const int wq = warp & 3;
        const int row = wq * 32 + lane;
        const int qi = q0 + row;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        int k_lim = ap.seq;
        if (ap.causal) k_lim = min(k_lim, qi + 1);
        for (int j = 0; j < nblk && ok; ++j) {
            const uint32_t s_addr = lane_addr + (j & 1) * BKV2;
            if (!mbar_wait(s_full + 8 * (j & 1), (j >> 1) & 1, status, 0x58)) { ok = false; break; }
            tc_fence_after();
            const int k0 = j * BKV2;
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(s_addr, r0);
            tmem_ld_32x32(s_addr + 32, r1);
            tmem_ld_wait();
            // only blocks that touch the diagonal or the end of the sequence need per-element masking (warp-uniform test)
            const bool masked = (k0 + BKV2 > ap.seq) || (ap.causal && k0 + BKV2 > q0 + wq * 32 + 1);
            float m_blk = -INFINITY;
            if (masked) {
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    if (k0 + t >= k_lim) r0[t] = 0xff800000u;       // -inf
                    if (k0 + 32 + t >= k_lim) r1[t] = 0xff800000u;
                }
            }
            {   // four independent chains instead of one 64-deep dependency; three-input max halves the instruction count
                float mx[4] = {m_blk, m_blk, m_blk, m_blk};
#pragma unroll
                for (int t = 0; t < 32; t += 4) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) mx[u] = fmax3(mx[u], __uint_as_float(r0[t + u]), __uint_as_float(r1[t + u]));
                }
                m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            }
            m_blk *= ap.scale_log2;
            // Lazy rescale: the reference maximum only moves when the new block exceeds it by more than 2^8; until then P is
            // allowed to reach 256 (exact in bf16/f16 range, sums are fp32) and O needs no correction.
            const float m_new = fmaxf(m_run, m_blk);
            const bool move = m_new > m_run + 8.0f || m_run == -INFINITY;
            const float m_ref = move ? m_new : m_run;
            const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
            const float alpha = move ? fast_exp2(m_run - m_use) : 1.0f;   // m_run = -inf -> 0
            // exponent arguments and row sums two lanes per instruction (fma/add .f32x2); the exponentials themselves are
            // one special-function op each
            const unsigned long long sc2 = f32x2_splat(ap.scale_log2), mu2 = f32x2_splat(-m_use);
            unsigned long long l2[4] = {0ull, 0ull, 0ull, 0ull};   // bit pattern of (0.0f, 0.0f)
            uint32_t packed[32];
#pragma unroll
            for (int t = 0; t < 32; t += 2) {
                float xa0, xa1, xb0, xb1;
                f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(r0[t]), __uint_as_float(r0[t + 1])), sc2, mu2), xa0, xa1);
                f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(r1[t]), __uint_as_float(r1[t + 1])), sc2, mu2), xb0, xb1);
                const float a0 = fast_exp2(xa0), a1 = fast_exp2(xa1), b0 = fast_exp2(xb0);
                const float b1 = POLY ? poly_exp2(xb1) : fast_exp2(xb1);   // optionally one element in four on the FMA pipe
                l2[(t >> 1) & 3] = f32x2_add(l2[(t >> 1) & 3], f32x2_add(f32x2_pack(a0, a1), f32x2_pack(b0, b1)));
                packed[t / 2] = E::pack(a0, a1);          // keys k0 + t, t+1      -> column t/2
                packed[16 + t / 2] = E::pack(b0, b1);     // keys k0 + 32 + t, ..  -> column 16 + t/2
            }
            float l_part[4];
            {
                float lo, hi;
                f32x2_unpack(f32x2_add(f32x2_add(l2[0], l2[1]), f32x2_add(l2[2], l2[3])), lo, hi);
                l_part[0] = lo; l_part[1] = hi; l_part[2] = 0.0f; l_part[3] = 0.0f;
            }
            l_run = l_run * alpha + ((l_part[0] + l_part[1]) + (l_part[2] + l_part[3]));
            m_run = m_ref;
            // O is touched only when some row of this warp moved its reference maximum; only then must the previous P*V
            // (which accumulates into O) have finished.  P_j itself goes into S_j's columns, which nothing else uses now.
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                if (!mbar_wait(pv_done, (j - 1) & 1, status, 0x59)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld_32x32(lane_addr + O_COL + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int t = 0; t < 32; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * alpha);
                    tmem_st_32x32(lane_addr + O_COL + c * 32, o);
                }
            }
            tmem_st_32x32(s_addr, packed);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * (j & 1));
        }
        // The last P*V.  A parity wait is only meaningful when at most one completion is outstanding, and a warp may be a
        // whole key block ahead of the slowest one (whose P gates the previous P*V): wait for the previous P*V first.
        // Its own validity: Q*K^T of the last block was issued behind P*V of block nblk-3, so nblk-2 completions are certain.
        if (ok && nblk >= 2) ok = mbar_wait(pv_done, (nblk - 2) & 1, status, 0x5b);
        if (ok && mbar_wait(pv_done, (nblk - 1) & 1, status, 0x5a)) {
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            T* orow = reinterpret_cast<T*>(ap.out) + (static_cast<size_t>(bh) * ap.seq + qi) * HD;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + O_COL + c * 32, r);
                tmem_ld_wait();
                if (qi < ap.seq) {
                    uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 u;
                        u.x = E::pack(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
                        u.y = E::pack(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
                        u.z = E::pack(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
                        u.w = E::pack(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
                        dst[q4] = u;
                    }
                }
                __syncwarp();
            }
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

// ---------------------------------------------------------------------------------------
// Third kernel: the second kernel made persistent.  A CTA that handles one query block pays
// for its launch, barrier and TMEM set-up, the Q load before the first score block and the
// teardown; at 2048 keys that fixed part is a sizeable share of a causal CTA's life.  Here the
// grid is two CTAs per SM and every CTA keeps drawing work units from a global counter:
// barriers, TMEM and the K/V ring live across query blocks, the next Q is loaded as soon as
// the last Q*K^T of the current block has been issued, and the next block's first two score
// blocks are issued right behind the last P*V.  All pipeline counters (K/V stage, S buffer,
// P*V phase) run on ONE global key-block counter per role, so nothing is re-initialised
// between query blocks.  The producer thread draws the unit (atomicAdd) and hands it to the
// MMA thread and the softmax warps through a two-slot ring in shared memory.
// Work units: non-causal, one query block; causal, the pair (last - i, i) of one head, so
// that units are of equal length and the last units drawn are not the longest.  Units of one
// head are neighbours in the counter's order, so its K/V stay in L2.
// ---------------------------------------------------------------------------------------
template <int HD>
struct AttnSmem3 {
    static constexpr int Q_BYTES = BQ * HD * 2;
    static constexpr int KV_TILE = BKV2 * HD * 2;
    static constexpr int Q_OFF = 0, K_OFF = Q_BYTES, V_OFF = Q_BYTES + 2 * KV_TILE, BAR_OFF = Q_BYTES + 4 * KV_TILE;
    static constexpr int NUM_BARS = 20;
    static constexpr size_t BYTES = 1024 + BAR_OFF + NUM_BARS * 8 + 32;   // + TMEM slot + two schedule slots
};

struct AttnWork {   // unit number -> query blocks
    int num_qb, units_per_head, total_units;
    __device__ __forceinline__ int blocks_in_unit(int unit, bool causal) const {
        if (!causal) return 1;
        const int i = unit % units_per_head;
        return (num_qb - 1 - i) != i ? 2 : 1;
    }
    // q-block `part` (0 or 1) of `unit`: the long one first
    __device__ __forceinline__ void item(int unit, int part, bool causal, int& qb, int& bh) const {
        bh = unit / units_per_head;
        const int i = unit % units_per_head;
        if (!causal) { qb = num_qb - 1 - i; return; }
        qb = part == 0 ? num_qb - 1 - i : i;
    }
};

template <int HD, int FMT, bool POLY>
__global__ void __launch_bounds__(192, 2)
attention_tc3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, AttnParams ap, int* status, int* next_unit) {
    using SM = AttnSmem3<HD>;
    using E = AElem<FMT>;
    using T = typename E::T;
    constexpr int HALVES = HD / 64;
    constexpr int Q_SLAB = BQ * 128;
    constexpr int KV_SLAB = BKV2 * 128;
    constexpr uint32_t IDESC_QK = make_idesc(FMT, FMT, 0, 0, BQ, BKV2);
    constexpr uint32_t IDESC_PV = make_idesc(FMT, FMT, 0, 1, BQ, HD);
    constexpr uint32_t TMEM_COLS = 256;              // S0 @0, S1 @64, O @128
    constexpr uint32_t O_COL = 128;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SM::NUM_BARS);
    volatile int* sched = reinterpret_cast<volatile int*>(tmem_slot + 1);   // two slots: the unit each role works on next
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 24, v_full = bar0 + 40, v_empty = bar0 + 56,
                   s_full = bar0 + 72, p_full = bar0 + 88, pv_done = bar0 + 104, q_empty = bar0 + 112, o_free = bar0 + 120,
                   sched_full = bar0 + 128, sched_empty = bar0 + 144;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool causal = ap.causal != 0;
    AttnWork wk;
    wk.num_qb = (ap.seq + BQ - 1) / BQ;
    wk.units_per_head = causal ? (wk.num_qb + 1) / 2 : wk.num_qb;
    wk.total_units = wk.units_per_head * ap.batch_heads;
    const int kv_blocks_all = (ap.seq + BKV2 - 1) / BKV2;
    auto blocks_of = [&](int qb) { return causal ? min(kv_blocks_all, (qb * BQ + BQ + BKV2 - 1) / BKV2) : kv_blocks_all; };

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
        mbar_init(q_full, 1); mbar_init(q_empty, 1); mbar_init(o_free, 4);
        for (int i = 0; i < 2; ++i) { mbar_init(sched_full + 8 * i, 1); mbar_init(sched_empty + 8 * i, 5); }   // readers: MMA thread + 4 warps
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + 8 * i, 1); mbar_init(k_empty + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1); mbar_init(v_empty + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1); mbar_init(p_full + 8 * i, 4);
        }
        mbar_init(pv_done, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const uint32_t sQ = smem_u32(smem + SM::Q_OFF), sK = smem_u32(smem + SM::K_OFF), sV = smem_u32(smem + SM::V_OFF);

    if (warp == 0) {
        if (lane == 0) {
            uint32_t g = 0;      // key blocks loaded so far (all query blocks of this CTA)
            int item = 0;        // query blocks started so far
            bool ok = true;
            // Units are handed out by a global counter (SMs do not all run at the same speed, so a static split leaves the
            // slow ones behind); this thread draws the next unit and publishes it to the other roles through a two-slot ring.
            // The draw for the unit after this one is issued before this unit's loads and only looked at after them, so the
            // counter's round trip to L2 is not on the path of the next Q load.
            int unit = atomicAdd(next_unit, 1);
            for (uint32_t n = 0; ok; ++n) {
                const uint32_t slot = n & 1;
                if (!mbar_wait(sched_empty + 8 * slot, ((n >> 1) & 1) ^ 1, status, 0x60)) { ok = false; break; }
                if (unit >= wk.total_units) unit = -1;
                sched[slot] = unit;
                mbar_arrive(sched_full + 8 * slot);
                if (unit < 0) break;
                const int this_unit = unit;
                unit = atomicAdd(next_unit, 1);
                const int parts = wk.blocks_in_unit(this_unit, causal);
                for (int part = 0; part < parts && ok; ++part, ++item) {
                    int qb, bh;
                    wk.item(this_unit, part, causal, qb, bh);
                    const int nblk = blocks_of(qb);
                    if (item > 0 && !mbar_wait(q_empty, (item - 1) & 1, status, 0x61)) { ok = false; break; }
                    mbar_arrive_expect_tx(q_full, SM::Q_BYTES);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) tma_load_3d(sQ + h * Q_SLAB, &tmQ, q_full, h * 64, qb * BQ, bh);
                    for (int j = 0; j < nblk; ++j, ++g) {
                        const uint32_t st = g & 1, par = ((g >> 1) & 1) ^ 1;
                        if (!mbar_wait(k_empty + 8 * st, par, status, 0x62)) { ok = false; break; }
                        mbar_arrive_expect_tx(k_full + 8 * st, SM::KV_TILE);
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) tma_load_3d(sK + st * SM::KV_TILE + h * KV_SLAB, &tmK, k_full + 8 * st, h * 64, j * BKV2, bh);
                        if (!mbar_wait(v_empty + 8 * st, par, status, 0x63)) { ok = false; break; }
                        mbar_arrive_expect_tx(v_full + 8 * st, SM::KV_TILE);
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) tma_load_3d(sV + st * SM::KV_TILE + h * KV_SLAB, &tmV, v_full + 8 * st, h * 64, j * BKV2, bh);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t HI_K = smem_desc_hi_sw128(1024);
            const uint32_t q_lo = smem_desc_lo(sQ, 16), k_lo0 = smem_desc_lo(sK, 16), v_lo0 = smem_desc_lo(sV, KV_SLAB);
            auto issue_qk = [&](uint32_t gq) {  // S[gq&1] = Q K^T for global key block gq
                const uint32_t st = gq & 1;
                const uint32_t d = tmem_base + st * BKV2;
                const uint32_t k_lo = k_lo0 + st * (SM::KV_TILE >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma_f16(d, smem_desc_join(q_lo + (((ks / 4) * Q_SLAB + (ks % 4) * 32) >> 4), HI_K),
                             smem_desc_join(k_lo + (((ks / 4) * KV_SLAB + (ks % 4) * 32) >> 4), HI_K), IDESC_QK, ks != 0);
                umma_commit(s_full + 8 * st);
                umma_commit(k_empty + 8 * st);
            };
            uint32_t g = 0;      // key blocks whose P*V has been issued
            int item = 0;
            bool ok = true;
            for (uint32_t n = 0; ok; ++n) {
                const uint32_t slot = n & 1;
                if (!mbar_wait(sched_full + 8 * slot, (n >> 1) & 1, status, 0x6e)) { ok = false; break; }
                const int unit = sched[slot];
                mbar_arrive(sched_empty + 8 * slot);
                if (unit < 0) break;
                const int parts = wk.blocks_in_unit(unit, causal);
                for (int part = 0; part < parts && ok; ++part, ++item) {
                    int qb, bh;
                    wk.item(unit, part, causal, qb, bh);
                    const int nblk = blocks_of(qb);
                    if (!mbar_wait(q_full, item & 1, status, 0x64)) { ok = false; break; }
                    for (int j = 0; j < 2 && j < nblk && ok; ++j) {   // two score blocks in flight before the first P arrives
                        if (!mbar_wait(k_full + 8 * ((g + j) & 1), ((g + j) >> 1) & 1, status, 0x65)) { ok = false; break; }
                        tc_fence_after();
                        issue_qk(g + j);
                        if (j == nblk - 1) umma_commit(q_empty);   // Q may be replaced once these MMAs have read it
                    }
                    for (int j = 0; j < nblk && ok; ++j, ++g) {
                        const uint32_t st = g & 1, ph = (g >> 1) & 1;
                        if (!mbar_wait(v_full + 8 * st, ph, status, 0x66)) { ok = false; break; }
                        if (!mbar_wait(p_full + 8 * st, ph, status, 0x67)) { ok = false; break; }
                        // the first P*V of a query block overwrites O: the previous block's rows must have been read out
                        if (j == 0 && item > 0 && !mbar_wait(o_free, (item - 1) & 1, status, 0x68)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t p_tmem = tmem_base + st * BKV2;
                        const uint32_t v_lo = v_lo0 + st * (SM::KV_TILE >> 4);
#pragma unroll
                        for (int ks = 0; ks < BKV2 / 16; ++ks)
                            umma_f16_ts(tmem_base + O_COL, p_tmem + ks * 8, smem_desc_join(v_lo + ks * (2048 >> 4), HI_K),
                                        IDESC_PV, (j | ks) != 0 ? 1u : 0u);
                        umma_commit(v_empty + 8 * st);
                        umma_commit(pv_done);
                        if (j + 2 < nblk) {
                            if (!mbar_wait(k_full + 8 * st, ((g + 2) >> 1) & 1, status, 0x69)) { ok = false; break; }
                            tc_fence_after();
                            issue_qk(g + 2);
                            if (j + 2 == nblk - 1) umma_commit(q_empty);
                        }
                    }
                }
            }
        }
    } else {
        const int wq = warp & 3;
        const int row = wq * 32 + lane;
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        uint32_t g = 0;          // key blocks whose softmax this warp has done
        bool ok = true;
        for (uint32_t n = 0; ok; ++n) {
            const uint32_t slot = n & 1;
            if (!mbar_wait(sched_full + 8 * slot, (n >> 1) & 1, status, 0x6f)) { ok = false; break; }
            const int unit = sched[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(sched_empty + 8 * slot);
            if (unit < 0) break;
            const int parts = wk.blocks_in_unit(unit, causal);
            for (int part = 0; part < parts && ok; ++part) {
                int qb, bh;
                wk.item(unit, part, causal, qb, bh);
                const int nblk = blocks_of(qb);
                const int q0 = qb * BQ;
                const int qi = q0 + row;
                float m_run = -INFINITY, l_run = 0.0f;
                int k_lim = ap.seq;
                if (causal) k_lim = min(k_lim, qi + 1);
                for (int j = 0; j < nblk && ok; ++j, ++g) {
                    const uint32_t st = g & 1, ph = (g >> 1) & 1;
                    const uint32_t s_addr = lane_addr + st * BKV2;
                    if (!mbar_wait(s_full + 8 * st, ph, status, 0x6a)) { ok = false; break; }
                    tc_fence_after();
                    const int k0 = j * BKV2;
                    uint32_t r0[32], r1[32];
                    tmem_ld_32x32(s_addr, r0);
                    tmem_ld_32x32(s_addr + 32, r1);
                    tmem_ld_wait();
                    const bool masked = (k0 + BKV2 > ap.seq) || (causal && k0 + BKV2 > q0 + wq * 32 + 1);
                    float m_blk = -INFINITY;
                    if (masked) {
#pragma unroll
                        for (int t = 0; t < 32; ++t) {
                            if (k0 + t >= k_lim) r0[t] = 0xff800000u;       // -inf
                            if (k0 + 32 + t >= k_lim) r1[t] = 0xff800000u;
                        }
                    }
                    {
                        float mx[4] = {m_blk, m_blk, m_blk, m_blk};
#pragma unroll
                        for (int t = 0; t < 32; t += 4) {
#pragma unroll
                            for (int u = 0; u < 4; ++u) mx[u] = fmax3(mx[u], __uint_as_float(r0[t + u]), __uint_as_float(r1[t + u]));
                        }
                        m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                    }
                    m_blk *= ap.scale_log2;
                    // lazy rescale, as in the second kernel: the reference maximum moves only on a jump of more than 2^8
                    const float m_new = fmaxf(m_run, m_blk);
                    const bool move = m_new > m_run + 8.0f || m_run == -INFINITY;
                    const float m_ref = move ? m_new : m_run;
                    const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
                    const float alpha = move ? fast_exp2(m_run - m_use) : 1.0f;
                    const unsigned long long sc2 = f32x2_splat(ap.scale_log2), mu2 = f32x2_splat(-m_use);
                    unsigned long long l2[4] = {0ull, 0ull, 0ull, 0ull};
                    uint32_t packed[32];
#pragma unroll
                    for (int t = 0; t < 32; t += 2) {
                        float xa0, xa1, xb0, xb1;
                        f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(r0[t]), __uint_as_float(r0[t + 1])), sc2, mu2), xa0, xa1);
                        f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(r1[t]), __uint_as_float(r1[t + 1])), sc2, mu2), xb0, xb1);
                        const float a0 = fast_exp2(xa0), a1 = fast_exp2(xa1), b0 = fast_exp2(xb0);
                        const float b1 = POLY ? poly_exp2(xb1) : fast_exp2(xb1);
                        l2[(t >> 1) & 3] = f32x2_add(l2[(t >> 1) & 3], f32x2_add(f32x2_pack(a0, a1), f32x2_pack(b0, b1)));
                        packed[t / 2] = E::pack(a0, a1);
                        packed[16 + t / 2] = E::pack(b0, b1);
                    }
                    float l_lo, l_hi;
                    f32x2_unpack(f32x2_add(f32x2_add(l2[0], l2[1]), f32x2_add(l2[2], l2[3])), l_lo, l_hi);
                    l_run = l_run * alpha + (l_lo + l_hi);
                    m_run = m_ref;
                    if (j > 0 && __any_sync(0xffffffffu, move)) {
                        // P*V of key block g-1 done: it is the (g-1)-th completion of pv_done.  Q*K^T of block g was issued
                        // behind P*V of g-2, so at least g-1 completions have happened and the parity test cannot alias.
                        if (!mbar_wait(pv_done, (g - 1) & 1, status, 0x6b)) { ok = false; break; }
                        tc_fence_after();
#pragma unroll 1
                        for (int c = 0; c < HD / 32; ++c) {
                            uint32_t o[32];
                            tmem_ld_32x32(lane_addr + O_COL + c * 32, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int t = 0; t < 32; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * alpha);
                            tmem_st_32x32(lane_addr + O_COL + c * 32, o);
                        }
                    }
                    tmem_st_32x32(s_addr, packed);
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(p_full + 8 * st);
                }
                if (!ok) break;
                // Rows of this query block out; then O may be overwritten by the next block's first P*V.  A parity wait is only
                // meaningful when at most one completion is outstanding, and a warp may be a whole key block ahead of the slowest
                // one (whose P gates the previous P*V): wait for the previous P*V first (g-2 completions are certain here, since
                // Q*K^T of the last block was issued behind the P*V two blocks earlier), then for the last one.
                if (g >= 2 && !mbar_wait(pv_done, (g - 2) & 1, status, 0x6d)) { ok = false; break; }
                if (!mbar_wait(pv_done, (g - 1) & 1, status, 0x6c)) { ok = false; break; }
                tc_fence_after();
                const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                T* orow = reinterpret_cast<T*>(ap.out) + (static_cast<size_t>(bh) * ap.seq + qi) * HD;
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(lane_addr + O_COL + c * 32, r);
                    tmem_ld_wait();
                    if (qi < ap.seq) {
                        uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 u;
                            u.x = E::pack(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
                            u.y = E::pack(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
                            u.z = E::pack(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
                            u.w = E::pack(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
                            dst[q4] = u;
                        }
                    }
                    __syncwarp();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_free);
            }
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

// ---------------------------------------------------------------------------------------
// Fourth kernel: two 128-query tiles per CTA, key blocks of 128, sixteen softmax warps.
// One CTA per SM owns all 512 TMEM columns (S0 | S1 | O0 | O1); the single MMA thread alternates
// between the tiles:
//     P0_j V_j -> Q0 K_{j+1}^T  |  P1_j V_j -> Q1 K_{j+1}^T  |  ...
// so that while tile 0 is in its softmax the tensor pipe works for tile 1 and vice versa, and every
// K/V block fetched from L2 serves 256 queries.  P_j overwrites S_j in TMEM (packed 2 x 16 bit per
// column) and is the A operand of P*V.  With a single S buffer per tile no parity can alias: Q*K^T
// of block j+1 is issued behind P*V of block j, so when a softmax warp sees S_{j+1} the previous
// P*V has completed.
// Each tile has EIGHT softmax warps: a 32-lane TMEM window is shared by two warps, 16 query rows each, read with the
// 16x256b shape (four threads per row, 32 scores per thread and row), so row maxima are two shuffles and nothing is
// exchanged between warps.
// Measured on B200 (256 heads x 2048 x 128): 0.509 ms non-causal / 0.330 ms causal, against 0.501 / 0.305 for the
// 64-key kernels above, which therefore stay the default; this one is selected with PYC_B200_ATTENTION_KERNEL=4.
// A cycle-stamp timeline of its main loop shows a period of ~3300 cycles per key block for 2048 cycles of tensor work:
// each tile's chain Q*K^T (560) -> scores seen (110) -> TMEM load (70) -> softmax (1750) -> store, hand-over (350) ->
// P*V (480) is serial because a tile has one S buffer, and the softmax itself runs at ~60 % of the rate the same
// instruction mix reaches alone (a micro-benchmark of ex2 + fma.f32x2 + add.f32x2 + cvt.bf16x2 + max runs at the
// special-function unit's 8 cycles per warp instruction).  One warp per window (32x32b shape), handing P over in two
// halves, and one issuing thread per tile were measured too: equal, equal and 30 % slower.
// ---------------------------------------------------------------------------------------
template <int HD>
struct AttnSmem4 {
    static constexpr int TILE = 128 * HD * 2;          // one [128 x HD] 16-bit tile (a Q tile, a K block or a V block)
    static constexpr int Q_OFF = 0, K_OFF = 2 * TILE, V_OFF = 4 * TILE, BAR_OFF = 6 * TILE;
    static constexpr int NUM_BARS = 16;
    static constexpr size_t BYTES = 1024 + BAR_OFF + NUM_BARS * 8 + 16;
};

constexpr int ATTN4_THREADS = 18 * 32;   // 16 softmax warps, MMA warp, TMA warp

template <int HD, int FMT, int POLY>
__global__ void __launch_bounds__(ATTN4_THREADS, 1)
attention_tc4_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, AttnParams ap, int* status) {
    using SM = AttnSmem4<HD>;
    using E = AElem<FMT>;
    using T = typename E::T;
    constexpr int BK = 128;                          // keys per block
    constexpr int HALVES = HD / 64;
    constexpr int SLAB = 128 * 128;                  // [128 rows x 128 B]
    constexpr uint32_t IDESC_QK = make_idesc(FMT, FMT, 0, 0, BQ, BK);
    constexpr uint32_t IDESC_PV = make_idesc(FMT, FMT, 0, 1, BQ, HD);
    constexpr uint32_t TMEM_COLS = 512;              // S0 @0, S1 @128, O0 @256, O1 @256 + HD
    constexpr uint32_t O_COL = 256;
    constexpr int MMA_WARP = 16, TMA_WARP = 17;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SM::BAR_OFF);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SM::NUM_BARS);
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_empty = bar0 + 24, v_full = bar0 + 40, v_empty = bar0 + 56,
                   s_full = bar0 + 72, p_full = bar0 + 88, pv_done = bar0 + 104;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_pairs = (ap.seq + 2 * BQ - 1) / (2 * BQ);
    const int pair = num_pairs - 1 - static_cast<int>(blockIdx.x);   // longest (causal) work first
    const int bh = blockIdx.y;
    const int q_base = pair * 2 * BQ;
    const int kv_all = (ap.seq + BK - 1) / BK;
    int nblk[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int q0t = q_base + t * BQ;
        nblk[t] = q0t >= ap.seq ? 0 : (ap.causal ? min(kv_all, q0t / BK + 1) : kv_all);
    }
    const int n_loop = max(nblk[0], nblk[1]);

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + 8 * i, 1); mbar_init(k_empty + 8 * i, 1);
            mbar_init(v_full + 8 * i, 1); mbar_init(v_empty + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1); mbar_init(p_full + 8 * i, 8); mbar_init(pv_done + 8 * i, 1);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == MMA_WARP) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const uint32_t sQ = smem_u32(smem + SM::Q_OFF), sK = smem_u32(smem + SM::K_OFF), sV = smem_u32(smem + SM::V_OFF);

    if (warp == TMA_WARP) {
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, 2 * SM::TILE);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sQ + t * SM::TILE + h * SLAB, &tmQ, q_full, h * 64, q_base + t * BQ, bh);
            for (int j = 0; j < n_loop; ++j) {
                const int st = j & 1;
                const uint32_t par = ((j >> 1) & 1) ^ 1;
                if (!mbar_wait(k_empty + 8 * st, par, status, 0x71)) break;
                mbar_arrive_expect_tx(k_full + 8 * st, SM::TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sK + st * SM::TILE + h * SLAB, &tmK, k_full + 8 * st, h * 64, j * BK, bh);
                if (!mbar_wait(v_empty + 8 * st, par, status, 0x72)) break;
                mbar_arrive_expect_tx(v_full + 8 * st, SM::TILE);
#pragma unroll
                for (int h = 0; h < HALVES; ++h) tma_load_3d(sV + st * SM::TILE + h * SLAB, &tmV, v_full + 8 * st, h * 64, j * BK, bh);
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t HI = smem_desc_hi_sw128(1024);
            const uint32_t q_lo0 = smem_desc_lo(sQ, 16), k_lo0 = smem_desc_lo(sK, 16), v_lo0 = smem_desc_lo(sV, SLAB);
            auto issue_qk = [&](int t, int j) {   // S_t = Q_t K_j^T, 128 x 128 x HD
                const uint32_t d = tmem_base + t * BK;
                const uint32_t q_lo = q_lo0 + t * (SM::TILE >> 4), k_lo = k_lo0 + (j & 1) * (SM::TILE >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t off = ((ks / 4) * SLAB + (ks % 4) * 32) >> 4;
                    umma_f16(d, smem_desc_join(q_lo + off, HI), smem_desc_join(k_lo + off, HI), IDESC_QK, ks != 0);
                }
                umma_commit(s_full + 8 * t);
            };
            auto issue_pv = [&](int t, int j) {   // O_t += P_t V_j, 128 x HD x 128, A from TMEM (8 columns per 16 keys)
                const uint32_t p_tmem = tmem_base + t * BK, o = tmem_base + O_COL + t * HD;
                const uint32_t v_lo = v_lo0 + (j & 1) * (SM::TILE >> 4);
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks)
                    umma_f16_ts(o, p_tmem + ks * 8, smem_desc_join(v_lo + ks * (2048 >> 4), HI), IDESC_PV, (j | ks) != 0 ? 1u : 0u);
                umma_commit(pv_done + 8 * t);
            };
            bool ok = mbar_wait(q_full, 0, status, 0x73) && mbar_wait(k_full, 0, status, 0x74);
            if (ok) {
                tc_fence_after();
                if (nblk[0] > 0) issue_qk(0, 0);
                if (nblk[1] > 0) issue_qk(1, 0);
                umma_commit(k_empty);
            }
            for (int j = 0; j < n_loop && ok; ++j) {
                const int st = j & 1;
                if (!mbar_wait(v_full + 8 * st, (j >> 1) & 1, status, 0x75)) { ok = false; break; }
                bool k_next = false;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j >= nblk[t]) continue;
                    if (!mbar_wait(p_full + 8 * t, j & 1, status, 0x76)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(t, j);
                    if (j + 1 < nblk[t]) {
                        if (!k_next) {
                            if (!mbar_wait(k_full + 8 * ((j + 1) & 1), ((j + 1) >> 1) & 1, status, 0x77)) { ok = false; break; }
                            tc_fence_after();
                            k_next = true;
                        }
                        issue_qk(t, j + 1);
                    }
                }
                if (!ok) break;
                umma_commit(v_empty + 8 * st);
                if (j + 1 < n_loop) umma_commit(k_empty + 8 * ((j + 1) & 1));
            }
        }
    } else {
        // Softmax warps.  Warp w: tile t = w / 8, TMEM lane window 32 * (w % 4), rows 16 * ((w / 4) % 2) .. + 15 of it.
        // Thread 4*i + c of the warp: rows i ("A") and i + 8 ("B") of those sixteen, score columns 8k + 2c, 8k + 2c + 1.
        const int t = warp >> 3;
        const int row16 = (warp & 3) * 32 + ((warp >> 2) & 1) * 16;      // first of this warp's 16 query rows inside the tile
        const int c2 = (lane & 3) * 2;
        const int q0 = q_base + t * BQ;
        const int qa = q0 + row16 + (lane >> 2), qb = qa + 8;            // the thread's two query rows (global index)
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(row16) << 16);
        const uint32_t s_addr = lane_addr + t * BK, o_addr = lane_addr + O_COL + t * HD;
        const int my_blocks = nblk[t];
        float m_a = -INFINITY, m_b = -INFINITY;
        unsigned long long l_ab = 0ull;          // this thread's share of the two row sums
        bool ok = true;
        int lim_a = ap.seq, lim_b = ap.seq;
        if (ap.causal) { lim_a = min(lim_a, qa + 1); lim_b = min(lim_b, qb + 1); }
        const unsigned long long sc2 = f32x2_splat(ap.scale_log2);
        for (int j = 0; j < my_blocks && ok; ++j) {
            if (!mbar_wait(s_full + 8 * t, j & 1, status, 0x78)) { ok = false; break; }
            tc_fence_after();
            const int k0 = j * BK;
            uint32_t r[64];
            tmem_ld_16x256b_x16(s_addr, r);
            tmem_ld_wait();
            // only blocks that touch the diagonal or the end of the sequence need per-element masking (warp-uniform test)
            const bool masked = (k0 + BK > ap.seq) || (ap.causal && k0 + BK > q0 + row16 + 1);
            if (masked) {
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const int key = k0 + 8 * k + c2;
                    if (key >= lim_a) r[4 * k] = 0xff800000u;        // -inf
                    if (key + 1 >= lim_a) r[4 * k + 1] = 0xff800000u;
                    if (key >= lim_b) r[4 * k + 2] = 0xff800000u;
                    if (key + 1 >= lim_b) r[4 * k + 3] = 0xff800000u;
                }
            }
            float mx_a = -INFINITY, mx_b = -INFINITY;
            {
                float ma[2] = {-INFINITY, -INFINITY}, mb[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    ma[k & 1] = fmax3(ma[k & 1], __uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]));
                    mb[k & 1] = fmax3(mb[k & 1], __uint_as_float(r[4 * k + 2]), __uint_as_float(r[4 * k + 3]));
                }
                mx_a = fmaxf(ma[0], ma[1]); mx_b = fmaxf(mb[0], mb[1]);
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            }
            mx_a *= ap.scale_log2; mx_b *= ap.scale_log2;
            // Lazy rescale: a row's reference maximum only moves when the new block exceeds it by more than 2^8.
            const float na = fmaxf(m_a, mx_a), nb = fmaxf(m_b, mx_b);
            const bool move_a = na > m_a + 8.0f || m_a == -INFINITY, move_b = nb > m_b + 8.0f || m_b == -INFINITY;
            const float ra = move_a ? na : m_a, rb = move_b ? nb : m_b;
            const float ua = ra == -INFINITY ? 0.0f : ra, ub = rb == -INFINITY ? 0.0f : rb;
            const float alpha_a = move_a ? fast_exp2(m_a - ua) : 1.0f, alpha_b = move_b ? fast_exp2(m_b - ub) : 1.0f;   // m = -inf -> 0
            m_a = ra; m_b = rb;
            const unsigned long long mu_a = f32x2_splat(-ua), mu_b = f32x2_splat(-ub);
            l_ab = f32x2_mul(l_ab, f32x2_pack(alpha_a, alpha_b));
            if (j > 0 && __any_sync(0xffffffffu, move_a || move_b)) {
                // O_t is only touched when some row of this warp moved its reference maximum.  P*V of block j-1 has completed
                // (Q*K^T of this block was issued behind it); the wait is immediate and orders the TMEM accesses.
                if (!mbar_wait(pv_done + 8 * t, (j - 1) & 1, status, 0x79)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int cc = 0; cc < HD / 32; ++cc) {      // 32 columns at a time: the scores stay in registers meanwhile
                    uint32_t o[16];
                    tmem_ld_16x256b_x4(o_addr + cc * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        o[4 * k] = __float_as_uint(__uint_as_float(o[4 * k]) * alpha_a); o[4 * k + 1] = __float_as_uint(__uint_as_float(o[4 * k + 1]) * alpha_a);
                        o[4 * k + 2] = __float_as_uint(__uint_as_float(o[4 * k + 2]) * alpha_b); o[4 * k + 3] = __float_as_uint(__uint_as_float(o[4 * k + 3]) * alpha_b);
                    }
                    tmem_st_16x256b_x4(o_addr + cc * 32, o);
                }
            }
            // exponent arguments two lanes per instruction, one special-function op per exponential
            unsigned long long la = 0ull, lb = 0ull;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                float xa0, xa1, xb0, xb1;
                f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1])), sc2, mu_a), xa0, xa1);
                f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(r[4 * k + 2]), __uint_as_float(r[4 * k + 3])), sc2, mu_b), xb0, xb1);
                const float a0 = fast_exp2(xa0), b0 = fast_exp2(xb0);
                const float a1 = (POLY >= 1 && (k & 1)) || POLY >= 2 ? poly_exp2(xa1) : fast_exp2(xa1);
                const float b1 = (POLY >= 1 && (k & 1)) || POLY >= 2 ? poly_exp2(xb1) : fast_exp2(xb1);
                la = f32x2_add(la, f32x2_pack(a0, a1));
                lb = f32x2_add(lb, f32x2_pack(b0, b1));
                r[4 * k] = E::pack(a0, a1);          // packed in place: even elements are the 16x128b store's registers
                r[4 * k + 2] = E::pack(b0, b1);
            }
            tmem_st_16x128b_x16_even(s_addr, r);
            {
                float a_lo, a_hi, b_lo, b_hi;
                f32x2_unpack(la, a_lo, a_hi); f32x2_unpack(lb, b_lo, b_hi);
                l_ab = f32x2_add(l_ab, f32x2_pack(a_lo + a_hi, b_lo + b_hi));
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * t);
        }
        if (ok && my_blocks > 0 && mbar_wait(pv_done + 8 * t, (my_blocks - 1) & 1, status, 0x7a)) {
            tc_fence_after();
            float l_a, l_b;
            f32x2_unpack(l_ab, l_a, l_b);
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
            l_a += __shfl_xor_sync(0xffffffffu, l_a, 2); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
            const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
            uint32_t o[HD / 2];
            if constexpr (HD == 128) tmem_ld_16x256b_x16(o_addr, o); else tmem_ld_16x256b_x8(o_addr, o);
            tmem_ld_wait();
            T* out = reinterpret_cast<T*>(ap.out) + static_cast<size_t>(bh) * ap.seq * HD;
            uint32_t* row_a = reinterpret_cast<uint32_t*>(out + static_cast<size_t>(qa) * HD + c2);
            uint32_t* row_b = reinterpret_cast<uint32_t*>(out + static_cast<size_t>(qb) * HD + c2);
#pragma unroll
            for (int k = 0; k < HD / 8; ++k) {       // columns 8k + 2c, + 1: one 4-byte store per row and k
                if (qa < ap.seq) row_a[4 * k] = E::pack(__uint_as_float(o[4 * k]) * inv_a, __uint_as_float(o[4 * k + 1]) * inv_a);
                if (qb < ap.seq) row_b[4 * k] = E::pack(__uint_as_float(o[4 * k + 2]) * inv_b, __uint_as_float(o[4 * k + 3]) * inv_b);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        if (*reinterpret_cast<volatile int*>(status) != ST_OK) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Any-shape path (fp32, head sizes other than 64/128, unaligned pointers): one warp per
// query row, online softmax over the keys, lanes split the head dimension.
__device__ __forceinline__ float ald(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ald(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float ald(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void ast(float* p, float v) { *p = v; }
__device__ __forceinline__ void ast(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void ast(__half* p, float v) { *p = __float2half_rn(v); }

template <typename T, int MAXD>
__global__ void __launch_bounds__(128)
attention_rowwarp_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V, T* __restrict__ O,
                         int batch_heads, int seq, int d, float scale, int causal) {
    constexpr int PER = MAXD / 32;
    const int lane = threadIdx.x & 31;
    const size_t rows = static_cast<size_t>(batch_heads) * seq;
    for (size_t gr = blockIdx.x * 4 + (threadIdx.x >> 5); gr < rows; gr += static_cast<size_t>(gridDim.x) * 4) {
        const size_t bh = gr / seq;
        const int i = static_cast<int>(gr % seq);
        const T* q = Q + gr * d; const T* kb = K + bh * seq * d; const T* vb = V + bh * seq * d;
        float qv[PER], acc[PER];
#pragma unroll
        for (int t = 0; t < PER; ++t) { const int c = lane + 32 * t; qv[t] = c < d ? ald(q + c) * scale : 0.0f; acc[t] = 0.0f; }
        float m = -INFINITY, l = 0.0f;
        const int lim = causal ? i + 1 : seq;
        for (int j = 0; j < lim; ++j) {
            float s = 0.0f;
#pragma unroll
            for (int t = 0; t < PER; ++t) { const int c = lane + 32 * t; if (c < d) s = fmaf(qv[t], ald(kb + static_cast<size_t>(j) * d + c), s); }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            const float mn = fmaxf(m, s), a = expf(m - mn), p = expf(s - mn);
            l = l * a + p;
#pragma unroll
            for (int t = 0; t < PER; ++t) { const int c = lane + 32 * t; if (c < d) acc[t] = acc[t] * a + p * ald(vb + static_cast<size_t>(j) * d + c); }
            m = mn;
        }
#pragma unroll
        for (int t = 0; t < PER; ++t) { const int c = lane + 32 * t; if (c < d) ast(O + gr * d + c, acc[t] / l); }
    }
}

template <typename T>
int launch_rowwarp(const void* q, const void* k, const void* v, void* o, int bh, int seq, int d, float scale, int causal, cudaStream_t s) {
    const size_t rows = static_cast<size_t>(bh) * seq;
    size_t blocks = (rows + 3) / 4;
    const size_t cap = static_cast<size_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    if (d <= 128) attention_rowwarp_kernel<T, 128><<<static_cast<unsigned>(blocks), 128, 0, s>>>(static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(o), bh, seq, d, scale, causal);
    else if (d <= 512) attention_rowwarp_kernel<T, 512><<<static_cast<unsigned>(blocks), 128, 0, s>>>(static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(o), bh, seq, d, scale, causal);
    else { set_error("attention: d_head %d > 512 is not supported", d); return -1; }
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

template <int HD, int FMT>
int launch_attention_tc(pyc_dtype dt, int bh, int seq, const void* q, const void* k, const void* v, void* out, float scale, int causal,
                        cudaStream_t stream, int* status) {
    // PYC_B200_ATTENTION_KERNEL=1 selects the first kernel (128-key blocks, P through shared memory, one CTA per SM),
    // =2 the second (64-key blocks, P in TMEM, two CTAs per SM, one CTA per query block); the default is the third,
    // the second made persistent.
    const char* pick = getenv("PYC_B200_ATTENTION_KERNEL");
    const bool first = pick && pick[0] == '1';
    const bool fourth = pick && pick[0] == '4';
    // Without a choice from the environment: causal work up to 4096 keys (query blocks of very different length, many short
    // ones) goes to the persistent kernel, 2-13 % faster there; long or non-causal work, where every CTA runs the same long
    // loop, is 2-5 % faster with one CTA per query block (measured at 2048, 4096 and 8192 keys).
    const bool second = pick ? pick[0] == '2' : !(causal && seq <= 4096);
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    CUtensorMap tq, tk, tv;
    const uint64_t dims[3] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(seq), static_cast<uint64_t>(bh)};
    const uint64_t str[2] = {static_cast<uint64_t>(HD) * 2, static_cast<uint64_t>(seq) * HD * 2};
    const uint32_t box_q[3] = {64, 128, 1};
    const uint32_t box_kv[3] = {64, static_cast<uint32_t>(first || fourth ? BKV : BKV2), 1};
    if (encode_tmap(&tq, q, 2, 3, dims, str, box_q, true) != 0 || encode_tmap(&tk, k, 2, 3, dims, str, box_kv, true) != 0 ||
        encode_tmap(&tv, v, 2, 3, dims, str, box_kv, true) != 0) return -1;
    AttnParams ap;
    ap.seq = seq; ap.batch_heads = bh; ap.causal = causal ? 1 : 0; ap.scale_log2 = scale * 1.4426950408889634f; ap.out = out;
    dim3 grid((seq + BQ - 1) / BQ, bh);
    if (fourth) {
        const char* pe = getenv("PYC_B200_ATTENTION_POLY");
        const int poly = pe && pe[0] >= '0' && pe[0] <= '2' ? pe[0] - '0' : 0;
        constexpr size_t smem = AttnSmem4<HD>::BYTES > 120 * 1024 ? AttnSmem4<HD>::BYTES : 120 * 1024;   // one CTA per SM: it takes all 512 TMEM columns
        static std::atomic<bool> attr_set4[16][3];   // zero-initialised; set-once per device, a repeated set is harmless
        auto k0 = attention_tc4_kernel<HD, FMT, 0>;
        auto k1 = attention_tc4_kernel<HD, FMT, 1>;
        auto k2 = attention_tc4_kernel<HD, FMT, 2>;
        auto kernel = poly == 0 ? k0 : poly == 1 ? k1 : k2;
        if (dev < 16 && !attr_set4[dev][poly]) {
            B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            attr_set4[dev][poly] = true;
        }
        dim3 grid4((seq + 2 * BQ - 1) / (2 * BQ), bh);
        kernel<<<grid4, ATTN4_THREADS, smem, stream>>>(tq, tk, tv, ap, status);
    } else if (first) {
        auto kernel = attention_tc_kernel<HD, FMT>;
        // At least 120 KB so that two CTAs never share an SM: each one takes all 512 TMEM columns.
        constexpr size_t smem = AttnSmem<HD>::BYTES > 120 * 1024 ? AttnSmem<HD>::BYTES : 120 * 1024;
        static std::atomic<bool> attr_set[16];   // zero-initialised; set-once per device, a repeated set is harmless
        if (dev < 16 && !attr_set[dev]) {
            B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            attr_set[dev] = true;
        }
        kernel<<<grid, 192, smem, stream>>>(tq, tk, tv, ap, status);
    } else if (!second) {
        const char* pe = getenv("PYC_B200_ATTENTION_POLY");
        const bool poly = pe && pe[0] == '1';
        constexpr size_t smem = AttnSmem3<HD>::BYTES > 76 * 1024 ? AttnSmem3<HD>::BYTES : 76 * 1024;   // two CTAs per SM, 256 TMEM columns each
        static std::atomic<bool> attr_set3[16][2];   // zero-initialised; set-once per device, a repeated set is harmless
        auto k_poly = attention_tc3_kernel<HD, FMT, true>;
        auto k_mufu = attention_tc3_kernel<HD, FMT, false>;
        if (dev < 16 && !attr_set3[dev][poly]) {
            B200_CUDA_OK(cudaFuncSetAttribute(poly ? k_poly : k_mufu, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            attr_set3[dev][poly] = true;
        }
        const int num_qb = (seq + BQ - 1) / BQ;
        const long long units = static_cast<long long>(causal ? (num_qb + 1) / 2 : num_qb) * bh;
        const long long slots = 2ll * sm_count();
        const unsigned ctas = static_cast<unsigned>(units < slots ? units : slots);
        // work counter of this launch: one of 48 ints behind the status word (launches that overlap in time on different
        // streams get different ones), zeroed on the launching stream
        static std::atomic<unsigned> launch_seq{0};
        int* next_unit = status + 8 + (launch_seq.fetch_add(1) % 48u);
        B200_CUDA_OK(cudaMemsetAsync(next_unit, 0, sizeof(int), stream));
        if (poly) k_poly<<<ctas, 192, smem, stream>>>(tq, tk, tv, ap, status, next_unit);
        else k_mufu<<<ctas, 192, smem, stream>>>(tq, tk, tv, ap, status, next_unit);
    } else {
        // PYC_B200_ATTENTION_POLY=1 moves a quarter of the exp2 work to the FMA pipe (measured slightly slower on B200: the
        // softmax warps are bound by their dependency chains, not by the MUFU; kept as a switch).
        const char* pe = getenv("PYC_B200_ATTENTION_POLY");
        const bool poly = pe && pe[0] == '1';
        // Never less than 76 KB: at most two CTAs per SM, because each takes 256 of the 512 TMEM columns.
        constexpr size_t smem = AttnSmem2<HD>::BYTES > 76 * 1024 ? AttnSmem2<HD>::BYTES : 76 * 1024;
        static std::atomic<bool> attr_set2[16][2];   // zero-initialised; set-once per device, a repeated set is harmless
        auto k_poly = attention_tc2_kernel<HD, FMT, true>;
        auto k_mufu = attention_tc2_kernel<HD, FMT, false>;
        if (dev < 16 && !attr_set2[dev][poly]) {
            B200_CUDA_OK(cudaFuncSetAttribute(poly ? k_poly : k_mufu, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            attr_set2[dev][poly] = true;
        }
        if (poly) k_poly<<<grid, 192, smem, stream>>>(tq, tk, tv, ap, status);
        else k_mufu<<<grid, 192, smem, stream>>>(tq, tk, tv, ap, status);
    }
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

}  // namespace

int launch_attention(pyc_dtype dt, int batch_heads, int seq, int d, const void* q, const void* k, const void* v, void* out, float scale,
                     int causal, cudaStream_t s, int* status) {
    if (batch_heads <= 0 || seq <= 0 || d <= 0 || !q || !k || !v || !out) { set_error("attention: bad shape or NULL pointer"); return -1; }
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool tc = (dt == PYC_DTYPE_BF16 || dt == PYC_DTYPE_F16) && (d == 64 || d == 128) && scale > 0.0f && status && batch_heads <= 65535 &&
                    aligned(q) && aligned(k) && aligned(v) && aligned(out);
    if (tc) {
        const bool bf = dt == PYC_DTYPE_BF16;
        if (d == 128) return bf ? launch_attention_tc<128, 1>(dt, batch_heads, seq, q, k, v, out, scale, causal, s, status)
                                : launch_attention_tc<128, 0>(dt, batch_heads, seq, q, k, v, out, scale, causal, s, status);
        return bf ? launch_attention_tc<64, 1>(dt, batch_heads, seq, q, k, v, out, scale, causal, s, status)
                  : launch_attention_tc<64, 0>(dt, batch_heads, seq, q, k, v, out, scale, causal, s, status);
    }
    switch (dt) {
        case PYC_DTYPE_F32: return launch_rowwarp<float>(q, k, v, out, batch_heads, seq, d, scale, causal, s);
        case PYC_DTYPE_BF16: return launch_rowwarp<__nv_bfloat16>(q, k, v, out, batch_heads, seq, d, scale, causal, s);
        case PYC_DTYPE_F16: return launch_rowwarp<__half>(q, k, v, out, batch_heads, seq, d, scale, causal, s);
        default: set_error("attention: unsupported dtype %d", static_cast<int>(dt)); return -1;
    }
}

}  // namespace b200

extern "C" {

int pyc_b200_attention(pyc_dtype dtype, int batch_heads, int seq_len, int d_head, const void* Q, const void* K, const void* V, void* Out,
                       float scale, int causal, void* stream) {
    return b200::launch_attention(dtype, batch_heads, seq_len, d_head, Q, K, V, Out, scale, causal, static_cast<cudaStream_t>(stream),
                                  b200::device_status_word());
}

int pyc_cutlass_attention_dispatch(const char* symbol, int seq_len, int d_head, const void* Q, const void* K, const void* V, void* Out,
                                   float scale, void* stream) {
    if (!symbol) return -1;
    pyc_dtype dt; int causal = 0;
    if (!strcmp(symbol, "b200_attention_bf16") || !strcmp(symbol, "cutlass_attention_bf16")) dt = PYC_DTYPE_BF16;
    else if (!strcmp(symbol, "b200_attention_f16") || !strcmp(symbol, "cutlass_attention_f16")) dt = PYC_DTYPE_F16;
    else if (!strcmp(symbol, "b200_attention_bf16_causal")) { dt = PYC_DTYPE_BF16; causal = 1; }
    else if (!strcmp(symbol, "b200_attention_f16_causal")) { dt = PYC_DTYPE_F16; causal = 1; }
    else if (!strcmp(symbol, "b200_attention_f32")) dt = PYC_DTYPE_F32;
    else { b200::set_error("unknown attention symbol %s", symbol); return -1; }
    return pyc_b200_attention(dt, 1, seq_len, d_head, Q, K, V, Out, scale, causal, stream);
}

}  // extern "C"
