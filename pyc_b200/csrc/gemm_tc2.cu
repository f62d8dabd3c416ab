// bf16 / f16 GEMM with CTA pairs: two CTAs of a cluster share one tcgen05.mma
// (cta_group::2, 256 x 256 x 16 per instruction).  Same math, epilogue and C-level
// interface as gemm_tc.cu; what changes is the data movement per SM:
//   * a pair owns a 256 x 256 output tile; CTA r keeps rows r*128..+127 in its TMEM
//   * per k-block each CTA loads its own A rows (128 x 64) and only HALF of the B tile
//     (64 x 128), 32 KB instead of 48 KB, so the ring is 7 deep instead of 4 and the
//     B traffic per SM is halved
//   * loads of both CTAs are counted on the leader's (even CTA's) "full" barrier; the
//     leader's single MMA thread issues for the pair and commits completion to the
//     barriers of both CTAs; epilogue warps of both CTAs release the accumulator by
//     arriving on the leader's barrier
// No multicast of any kind is used: every CTA fetches its own operand halves.
// Replaces the same PyC code as gemm_tc.cu (cutlass_kernels/gemm/kernel.cu:48-84).
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include "internal.h"
#include "math.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BN = 256;          // columns per pair tile
constexpr int BNH = 128;         // B columns loaded by each CTA
constexpr int BK = 64;
constexpr int A_STAGE = BM * BK * 2;    // 16 KB
constexpr int B_STAGE = BNH * BK * 2;   // 16 KB
constexpr int GROUP_M = 8;              // in pair tiles (8 x 256 rows)
constexpr int EPI_STAGE_BYTES = 4 * 32 * 128;   // epilogue staging (6-stage form): 32 rows x 128 bytes per warp

struct Epi2 {
    void* D;
    const void* add;
    float alpha, add_scale;
    int add_mode, act, vec_ok;
    int l2_hints;   // 0: none; 1: A panel evict_last, B evict_first; 2: both evict_last; 3: A evict_last only
};

template <int FMT> struct El;
template <> struct El<1> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float to_f(T v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T from_f(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { __nv_bfloat162 p = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&p); }
    static __device__ __forceinline__ void unpack(uint32_t u, float& a, float& b) { a = __uint_as_float(u << 16); b = __uint_as_float(u & 0xffff0000u); }
};
template <> struct El<0> {
    using T = __half;
    static __device__ __forceinline__ float to_f(T v) { return __half2float(v); }
    static __device__ __forceinline__ T from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) { __half2 p = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&p); }
    static __device__ __forceinline__ void unpack(uint32_t u, float& a, float& b) { __half2 p = *reinterpret_cast<__half2*>(&u); float2 f = __half22float2(p); a = f.x; b = f.y; }
};

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int group = GROUP_M * tiles_n;
    const int g = tile / group;
    const int first = g * GROUP_M;
    const int gm = min(GROUP_M, tiles_m - first);
    const int local = tile - g * group;
    tm = first + local % gm;
    tn = local / gm;
}

template <int STAGES, bool B_KMAJOR, int FMT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(STAGES <= 6 ? 320 : 192, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Epi2 ep, int M, int N, int K, int* status) {
    constexpr uint32_t PAIR_TX = 2 * (A_STAGE + B_STAGE);  // bytes both CTAs deliver per stage
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = make_idesc(FMT, FMT, 0, B_KMAJOR ? 0 : 1, 2 * BM, BN);
    using E = El<FMT>;
    using T = typename E::T;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    // With 7 ring stages there is no room left; with 6, each epilogue warp gets 4 KB to park 64 columns of its 32 rows
    // and write them out as whole 128-byte row segments instead of 32 scattered pieces per store instruction.
    constexpr bool STAGED = STAGES <= 6;
    // The 6-stage form also runs eight epilogue warps (two per TMEM lane quarter, half of the tile's columns each): the epilogue's
    // stay beside the next tile's main loop is half as long.
    constexpr int EPI_WARPS = STAGED ? 8 : 4;
    uint8_t* sB = smem + STAGES * A_STAGE;
    uint8_t* sOut = sB + STAGES * B_STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + (STAGED ? EPI_WARPS * 4096 : 0));
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 2 * EPI_WARPS); }  // epilogue warps of both CTAs
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish_pair(); }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    // The two single-thread loops below share their scheduler with an epilogue warp each, and the MMA loop has to come
    // round once per 512 tensor-pipe cycles; everything that does not change per k-block (peer barrier addresses,
    // descriptor high words, shared-memory bases) is therefore computed once, and the per-stage values are stepped
    // with one add each instead of being rebuilt.
    if (warp == 0) {
        if (lane == 0) {  // each CTA loads its own halves; bytes are counted on the leader's barrier
            const uint32_t leader_full0 = map_to_cta(full0, 0);
            const uint32_t a_dst0 = smem_u32(sA), b_dst0 = smem_u32(sB);
            // The tile order keeps a panel of A rows and sweeps B across it: A is what the next wave wants to find in L2.
            const uint64_t pol_a = l2_policy_evict_last();
            const uint64_t pol_b = ep.l2_hints == 2 ? l2_policy_evict_last() : l2_policy_evict_first();
            uint32_t stage = 0, phase = 0, a_dst = a_dst0, b_dst = b_dst0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
                int tm, tn;
                pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
                const int n0 = tn * BN + static_cast<int>(rank) * BNH;
                for (int kb = 0, k0 = 0; kb < num_kb; ++kb, k0 += BK) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, status, 0x41)) { ok = false; break; }
                    const uint32_t leader_full = leader_full0 + 8 * stage;
                    if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * stage, PAIR_TX);
                    if (ep.l2_hints) {
                        tma_load_2d_pair_hint(a_dst, &tmA, leader_full, k0, m0, pol_a);
                        if (B_KMAJOR) {
                            if (ep.l2_hints == 3) tma_load_2d_pair(b_dst, &tmB, leader_full, k0, n0);
                            else tma_load_2d_pair_hint(b_dst, &tmB, leader_full, k0, n0, pol_b);
                        } else if (ep.l2_hints == 3) {
                            tma_load_2d_pair(b_dst, &tmB, leader_full, n0, k0);
                            tma_load_2d_pair(b_dst + BK * 128, &tmB, leader_full, n0 + 64, k0);
                        } else {
                            tma_load_2d_pair_hint(b_dst, &tmB, leader_full, n0, k0, pol_b);
                            tma_load_2d_pair_hint(b_dst + BK * 128, &tmB, leader_full, n0 + 64, k0, pol_b);
                        }
                    } else {
                        tma_load_2d_pair(a_dst, &tmA, leader_full, k0, m0);
                        if (B_KMAJOR) {
                            tma_load_2d_pair(b_dst, &tmB, leader_full, k0, n0);
                        } else {
                            tma_load_2d_pair(b_dst, &tmB, leader_full, n0, k0);
                            tma_load_2d_pair(b_dst + BK * 128, &tmB, leader_full, n0 + 64, k0);
                        }
                    }
                    a_dst += A_STAGE; b_dst += B_STAGE;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_dst = a_dst0; b_dst = b_dst0; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {  // the pair's single MMA issuer
            constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
            constexpr uint32_t A_STEP = A_STAGE >> 4, B_STEP = B_STAGE >> 4;
            constexpr uint32_t A_K16 = 32 >> 4, B_K16 = (B_KMAJOR ? 32 : 2048) >> 4;   // one 16-deep slice further along K
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), B_KMAJOR ? 16 : BK * 128);
            const uint32_t empty_peer0 = map_to_cta(empty0, 1), tfull_peer0 = map_to_cta(tfull0, 1);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0;
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++it) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, status, 0x42)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, status, 0x43)) { ok = false; break; }
                    tc_fence_after();
                    umma_f16_pair(d_tmem, smem_desc_join(a_lo, DESC_HI), smem_desc_join(b_lo, DESC_HI), IDESC, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k4 = 1; k4 < BK / 16; ++k4)
                        umma_f16_pair(d_tmem, smem_desc_join(a_lo + k4 * A_K16, DESC_HI), smem_desc_join(b_lo + k4 * B_K16, DESC_HI), IDESC, 1u);
                    umma_commit_pair(empty0 + 8 * stage);        // free the stage in both CTAs (own barrier: its shared::cta
                    umma_commit_pair(empty_peer0 + 8 * stage);   // address is also its cluster address)
                    a_lo += A_STEP; b_lo += B_STEP;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                }
                if (ok) {
                    umma_commit_pair(tfull0 + 8 * acc);          // accumulator ready in both CTAs
                    umma_commit_pair(tfull_peer0 + 8 * acc);
                }
            }
        }
    } else {
        const int wq = warp & 3;
        constexpr int CHUNKS_PER_WARP = (BN / 32) / (EPI_WARPS / 4);
        const int c_begin = ((warp - 2) >> 2) * CHUNKS_PER_WARP, c_end = c_begin + CHUNKS_PER_WARP;
        const uint32_t tempty_leader0 = map_to_cta(tempty0, 0);
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        const T* addp = reinterpret_cast<const T*>(ep.add);
        const float scalar_add = ep.add_mode == PYC_B200_ADD_SCALAR ? ep.add_scale * E::to_f(addp[0]) : 0.0f;
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            int tm, tn;
            pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int row = tm * 2 * BM + static_cast<int>(rank) * BM + wq * 32 + lane;
            const int n0 = tn * BN;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase, status, 0x44)) break;
            tc_fence_after();
            T* drow = reinterpret_cast<T*>(ep.D) + static_cast<size_t>(row) * N;
            const uint32_t acc_addr = lane_base + acc * BN;
            uint8_t* stage = sOut + (warp - 2) * 4096;
            const int row0 = row - lane;   // first row of this warp
            bool use_stage = false;
            // One 32-column chunk: scale, add, activation, 64 bytes out.  The next chunk's TMEM load is already in flight.
            auto chunk = [&](const uint32_t (&r)[32], int c) {
                const int col0 = n0 + c * 32;  // warp-uniform
                if (col0 >= N || row >= M) return;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = ep.alpha * __uint_as_float(r[j]) + scalar_add;
                const bool full_chunk = ep.vec_ok && (col0 + 32 <= N);
                if (ep.add_mode == PYC_B200_ADD_ROW_BIAS || ep.add_mode == PYC_B200_ADD_MATRIX) {
                    const T* src = ep.add_mode == PYC_B200_ADD_ROW_BIAS ? addp + col0 : addp + static_cast<size_t>(row) * N + col0;
                    if (full_chunk) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 u = __ldg(reinterpret_cast<const uint4*>(src) + q);
                            float a, b;
                            E::unpack(u.x, a, b); v[q * 8 + 0] += ep.add_scale * a; v[q * 8 + 1] += ep.add_scale * b;
                            E::unpack(u.y, a, b); v[q * 8 + 2] += ep.add_scale * a; v[q * 8 + 3] += ep.add_scale * b;
                            E::unpack(u.z, a, b); v[q * 8 + 4] += ep.add_scale * a; v[q * 8 + 5] += ep.add_scale * b;
                            E::unpack(u.w, a, b); v[q * 8 + 6] += ep.add_scale * a; v[q * 8 + 7] += ep.add_scale * b;
                        }
                    } else {
                        for (int j = 0; j < 32; ++j) if (col0 + j < N) v[j] += ep.add_scale * E::to_f(src[j]);
                    }
                }
                if (ep.act == PYC_B200_ACT_GELU) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) gelu_erf_x2_16bit(v[j], v[j + 1]);   // bf16 / f16 output
                } else if (ep.act == PYC_B200_ACT_RELU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
                }
                if (full_chunk) {
                    // 64 bytes of this row: two 32-byte stores when the row start allows it (whole sectors), else four 16-byte ones
                    uint32_t w[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) w[j] = E::pack(v[2 * j], v[2 * j + 1]);
                    if (STAGED && use_stage) {   // 16-byte chunk (c & 1) * 4 + q of this lane's row, at position chunk ^ (row & 7)
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            *reinterpret_cast<uint4*>(stage + lane * 128 + ((((c & 1) * 4 + q) ^ (lane & 7)) * 16)) =
                                make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    } else if (ep.vec_ok == 2) {
                        const uint32_t lo[8] = {w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]};
                        const uint32_t hi[8] = {w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]};
                        st_global_v8(drow + col0, lo);
                        st_global_v8(drow + col0 + 16, hi);
                    } else {
                        uint4* dst = reinterpret_cast<uint4*>(drow + col0);
#pragma unroll
                        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    }
                } else {
                    for (int j = 0; j < 32; ++j) if (col0 + j < N) drow[col0 + j] = E::from_f(v[j]);
                }
            };
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(acc_addr + c_begin * 32, r0);
#pragma unroll 1
            for (int c = c_begin; c < c_end; c += 2) {
                use_stage = STAGED && ep.vec_ok && n0 + c * 32 + 64 <= N;   // warp-uniform: all 64 columns exist
                tmem_ld_wait();
                tmem_ld_32x32(acc_addr + (c + 1) * 32, r1);
                chunk(r0, c);
                __syncwarp();
                tmem_ld_wait();
                if (c + 2 < c_end) tmem_ld_32x32(acc_addr + (c + 2) * 32, r0);
                chunk(r1, c + 1);
                __syncwarp();
                if (STAGED && use_stage) {
                    // store instruction i covers rows 4i .. 4i+3 of the warp, eight lanes (8 x 16 bytes) per row
                    const int colv = n0 + c * 32 + (lane & 7) * 8;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = 4 * i + (lane >> 3);
                        if (row0 + rr < M) {
                            const uint4 u = *reinterpret_cast<const uint4*>(stage + rr * 128 + (((lane & 7) ^ (rr & 7)) * 16));
                            *reinterpret_cast<uint4*>(reinterpret_cast<T*>(ep.D) + static_cast<size_t>(row0 + rr) * N + colv) = u;
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * acc);  // the leader's MMA thread waits for all 8 warps
        }
    }

    // Teardown: both CTAs meet here (also after a timed-out wait), so neither exits while the other may still
    // signal its barriers or read its shared memory.
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(status) != ST_OK) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <int STAGES, bool B_KMAJOR, int FMT>
int launch_pair_instance(const GemmProblem& p, cudaStream_t stream, int* status) {
    auto kernel = gemm_tc2_kernel<STAGES, B_KMAJOR, FMT>;
    constexpr size_t smem = 1024 + static_cast<size_t>(STAGES) * (A_STAGE + B_STAGE) + (STAGES <= 6 ? 8 * 4096 : 0) + (2 * STAGES + 4) * 8 + 16;
    static std::atomic<bool> attr_set[16];   // zero-initialised; set-once per device, a repeated set is harmless
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 16 && !attr_set[dev]) {
        B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_set[dev] = true;
    }
    CUtensorMap tmA, tmB;
    if (encode_tmap_2d(&tmA, p.A, 2, p.M, p.K, static_cast<uint64_t>(p.K) * 2, BM, BK) != 0) return -1;
    if (B_KMAJOR) { if (encode_tmap_2d(&tmB, p.B, 2, p.N, p.K, static_cast<uint64_t>(p.K) * 2, BNH, BK) != 0) return -1; }
    else { if (encode_tmap_2d(&tmB, p.B, 2, p.K, p.N, static_cast<uint64_t>(p.N) * 2, BK, 64) != 0) return -1; }
    Epi2 ep;
    ep.D = p.D; ep.add = p.add; ep.alpha = p.alpha; ep.add_scale = p.add_scale;
    ep.add_mode = p.add ? p.add_mode : PYC_B200_ADD_NONE; ep.act = p.act;
    ep.vec_ok = ((reinterpret_cast<uintptr_t>(p.D) % 16 == 0) && (p.N % 8 == 0) &&
                 (ep.add_mode == PYC_B200_ADD_NONE || ep.add_mode == PYC_B200_ADD_SCALAR || reinterpret_cast<uintptr_t>(p.add) % 16 == 0)) ? 1 : 0;
    if (ep.vec_ok && reinterpret_cast<uintptr_t>(p.D) % 32 == 0 && p.N % 16 == 0) ep.vec_ok = 2;   // rows start on 32-byte boundaries
    ep.l2_hints = 0;
    if (const char* h = getenv("PYC_B200_GEMM_L2_HINTS")) { const int v = atoi(h); if (v >= 0 && v <= 3) ep.l2_hints = v; }
    const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
    const int max_pairs = sm_count() / 2;
    const int grid = 2 * (tiles < max_pairs ? tiles : max_pairs);
    kernel<<<grid, STAGES <= 6 ? 320 : 192, smem, stream>>>(tmA, tmB, ep, p.M, p.N, p.K, status);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

}  // namespace

int launch_gemm_tc_pair(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream, int* status) {
    const bool bf16 = p.dtype == PYC_DTYPE_BF16;
    if (cfg.stages == 6) {   // six ring stages + staged epilogue stores
        if (p.b_col_major) return bf16 ? launch_pair_instance<6, true, 1>(p, stream, status) : launch_pair_instance<6, true, 0>(p, stream, status);
        return bf16 ? launch_pair_instance<6, false, 1>(p, stream, status) : launch_pair_instance<6, false, 0>(p, stream, status);
    }
    if (p.b_col_major) return bf16 ? launch_pair_instance<7, true, 1>(p, stream, status) : launch_pair_instance<7, true, 0>(p, stream, status);
    return bf16 ? launch_pair_instance<7, false, 1>(p, stream, status) : launch_pair_instance<7, false, 0>(p, stream, status);
}

}  // namespace b200
