// fp8 (e4m3) x fp8 (e4m3) GEMM on the tcgen05 tensor cores (kind::f8f6f4), fp32
// accumulation in TMEM, with dequantisation fused into the epilogue:
//     D[m,n] = act( acc[m,n] * row_scale[m] * col_scale[n] + bias[n] )   -> bf16
// row_scale is the per-token scale of the quantised activations, col_scale the
// per-output-channel scale of the quantised weights.
//
// PyC has no fp8 dtype or kernel (include/pyc/ir.h:16-23 stops at I8); this is the
// weight path of the transformer-FFN benchmark configuration, reached through the
// additive entry points only.  Structure identical to gemm_tc.cu (persistent CTA,
// TMA ring, single-thread MMA issuer, double-buffered TMEM accumulators, four
// epilogue warps); what changes is the element size: a 128-byte swizzle row holds
// 128 k-values, one MMA consumes K = 32, B stored [K,N] row-major is the MN-major
// operand with 128-column slabs (LBO = 16 KB, SBO = 1 KB).
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdlib.h>

#include <algorithm>

#include "internal.h"
#include "math.cuh"
#include "ptx_sm100.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;                      // fp8 elements per stage row = 128 bytes
constexpr int A_STAGE_BYTES = BM * BK;
constexpr int GROUP_M = 16;
constexpr int EPI_STAGE_BYTES = 4 * 32 * 128;   // epilogue staging: 32 rows x 128 bytes per warp

struct Fp8Epilogue {
    __nv_bfloat16* D;
    const float* row_scale;   // [M] or null
    const float* col_scale;   // [N] or null
    const __nv_bfloat16* bias;  // [N] or null
    int act;
    // Row scatter for tensor parallelism (world > 0): row r of D belongs to rank r / rows_per_rank and is stored at
    // dst[owner] + (src_rank * rows_per_rank + r % rows_per_rank) * N, i.e. straight into the owner's receive slot for this
    // rank (its own memory or a peer's, mapped into this process); D is unused then.
    __nv_bfloat16* dst[PYC_B200_TP_MAX_RANKS];
    int world, rows_per_rank, src_rank;
    // In-switch all-reduce fused into the CTA-pair kernel (sw_world > 0): D is this rank's copy of a buffer bound to an
    // NVLink multicast object, sw_mc its multicast address.
    char* sw_mc;
    uint32_t* sw_flags[PYC_B200_TP_MAX_RANKS];
    uint32_t* sw_fin[PYC_B200_TP_MAX_RANKS];
    uint32_t* sw_epochs;
    int sw_world, sw_rank;
};

__device__ __forceinline__ void fp8_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int group = GROUP_M * tiles_n;
    const int g = tile / group;
    const int first = g * GROUP_M;
    const int gm = min(GROUP_M, tiles_m - first);
    const int local = tile - g * group;
    tm = first + local % gm;
    tn = local / gm;
}

// Epilogue of one accumulator tile for one thread (= one row): BN columns from TMEM at `acc_addr`, dequantise, bias,
// activation, bf16 out.  Shared by the single-CTA and the CTA-pair kernel.
// Where row `row` of the result starts: in D, or (tensor parallel) in the owning rank's receive slot for this rank.
__device__ __forceinline__ __nv_bfloat16* fp8_out_row(const Fp8Epilogue& ep, int row, int N) {
    if (ep.world > 0) {
        const int owner = row / ep.rows_per_rank;
        return ep.dst[owner] + (static_cast<size_t>(ep.src_rank) * ep.rows_per_rank + (row - owner * ep.rows_per_rank)) * N;
    }
    return ep.D + static_cast<size_t>(row) * N;
}

// `stage`: 4 KB of shared memory private to the calling warp (32 rows x 128 bytes).  With vec_ok the results of 64
// columns are parked there, one row per lane, and written out with every store instruction covering four whole
// 128-byte row segments: full lines instead of 32 scattered 16-byte pieces, which matters most when the rows go to
// another GPU over NVLink.  16-byte chunk c of row r sits at chunk position c ^ (r & 7), so neither side conflicts.
template <int BN>
__device__ __forceinline__ void fp8_epilogue_tile(const Fp8Epilogue& ep, uint32_t acc_addr, int row, int n0, int M, int N, bool vec_ok,
                                                  uint8_t* stage) {
    const int lane = threadIdx.x & 31;
    const int row0 = row - lane;   // first row of this warp
    const float rs = (ep.row_scale && row < M) ? ep.row_scale[row] : 1.0f;
    __nv_bfloat16* drow = row < M ? fp8_out_row(ep, row, N) : ep.D;
    bool use_stage = false;
    // One 32-column chunk; the next chunk's TMEM load is already in flight while this one is computed.
    auto chunk = [&](const uint32_t (&r)[32], int c) {
        const int col0 = n0 + c * 32;  // warp-uniform
        if (col0 >= N || row >= M) return;
        {
            float v[32];
            const bool full_chunk = vec_ok && col0 + 32 <= N;
            if (full_chunk) {  // scales and bias as 16-byte loads: every lane reads the same 128 / 64 bytes (broadcast)
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * rs;
                if (ep.col_scale) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const float4 c4 = __ldg(reinterpret_cast<const float4*>(ep.col_scale + col0) + q);
                        v[q * 4 + 0] *= c4.x; v[q * 4 + 1] *= c4.y; v[q * 4 + 2] *= c4.z; v[q * 4 + 3] *= c4.w;
                    }
                }
                if (ep.bias) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 u = __ldg(reinterpret_cast<const uint4*>(ep.bias + col0) + q);
                        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                        for (int t = 0; t < 4; ++t) { v[q * 8 + 2 * t] += __uint_as_float(w[t] << 16); v[q * 8 + 2 * t + 1] += __uint_as_float(w[t] & 0xffff0000u); }
                    }
                }
                if (ep.act == PYC_B200_ACT_GELU) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) gelu_erf_x2_16bit(v[j], v[j + 1]);   // bf16 output
                } else if (ep.act == PYC_B200_ACT_RELU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = col0 + j;
                    float x = __uint_as_float(r[j]) * rs;
                    if (col < N) {
                        if (ep.col_scale) x *= __ldg(ep.col_scale + col);
                        if (ep.bias) x += __bfloat162float(ep.bias[col]);
                    }
                    v[j] = apply_activation(x, ep.act);
                }
            }
            if (full_chunk) {
                uint4* dst = reinterpret_cast<uint4*>(drow + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]), p1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]), p3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
                    uint4 u;
                    u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
                    u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
                    if (use_stage) {   // chunk (c & 1) * 4 + q of this lane's row
                        const int cc = ((c & 1) * 4 + q) ^ (lane & 7);
                        *reinterpret_cast<uint4*>(stage + lane * 128 + cc * 16) = u;
                    } else {
                        dst[q] = u;
                    }
                }
            } else {
                for (int j = 0; j < 32; ++j) if (col0 + j < N) drow[col0 + j] = __float2bfloat16_rn(v[j]);
            }
        }
    };
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(acc_addr, r0);
#pragma unroll 1
    for (int c = 0; c < BN / 32; c += 2) {
        use_stage = stage != nullptr && vec_ok && n0 + c * 32 + 64 <= N;   // warp-uniform: all 64 columns exist
        tmem_ld_wait();
        tmem_ld_32x32(acc_addr + (c + 1) * 32, r1);
        chunk(r0, c);
        __syncwarp();
        tmem_ld_wait();
        if (c + 2 < BN / 32) tmem_ld_32x32(acc_addr + (c + 2) * 32, r0);
        chunk(r1, c + 1);
        __syncwarp();
        if (use_stage) {
            // 64 columns of 32 rows are parked: store instruction i covers rows 4i .. 4i+3, eight lanes per row
            const int colv = n0 + c * 32 + (lane & 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int rr = 4 * i + (lane >> 3);
                const int grow = row0 + rr;
                if (grow < M && colv + 8 <= N) {
                    const uint4 u = *reinterpret_cast<const uint4*>(stage + rr * 128 + (((lane & 7) ^ (rr & 7)) * 16));
                    *reinterpret_cast<uint4*>(fp8_out_row(ep, grow, N) + colv) = u;
                }
            }
            __syncwarp();
        }
    }
}

template <int BN, int STAGES, bool B_KMAJOR>
__global__ void __launch_bounds__(192, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Fp8Epilogue ep, int M, int N, int K, int* status) {
    constexpr int B_STAGE_BYTES = BN * BK;
    constexpr uint32_t STAGE_TX = A_STAGE_BYTES + B_STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = make_idesc(0, 0, 0, B_KMAJOR ? 0 : 1, BM, BN);  // e4m3 x e4m3 -> f32

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint8_t* sOut = sB + STAGES * B_STAGE_BYTES;                     // 4 epilogue warps x 4 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + EPI_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
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

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t a_dst0 = smem_u32(sA), b_dst0 = smem_u32(sB);
            uint32_t stage = 0, phase = 0, adst = a_dst0, bdst = b_dst0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn;
                fp8_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, status, 0x31)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * stage;
                    mbar_arrive_expect_tx(fb, STAGE_TX);
                    tma_load_2d(adst, &tmA, fb, kb * BK, m0);
                    if (B_KMAJOR) {
                        tma_load_2d(bdst, &tmB, fb, kb * BK, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 128; ++j) tma_load_2d(bdst + j * (BK * 128), &tmB, fb, n0 + j * 128, kb * BK);
                    }
                    adst += A_STAGE_BYTES; bdst += B_STAGE_BYTES;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; adst = a_dst0; bdst = b_dst0; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // Constant descriptor high word, stepped low words: the loop must come round once per k-block of tensor time
            // while an epilogue warp competes for the same scheduler.
            constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
            constexpr uint32_t A_STEP = A_STAGE_BYTES >> 4, B_STEP = B_STAGE_BYTES >> 4;
            constexpr uint32_t A_K32 = 32 >> 4, B_K32 = (B_KMAJOR ? 32 : 32 * 128) >> 4;   // 32 k-values further along K
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), B_KMAJOR ? 16 : BK * 128);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, status, 0x32)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, status, 0x33)) { ok = false; break; }
                    tc_fence_after();
                    umma_f8(d_tmem, smem_desc_join(a_lo, DESC_HI), smem_desc_join(b_lo, DESC_HI), IDESC, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k4 = 1; k4 < BK / 32; ++k4)  // one MMA = 32 k-values = 32 bytes of a K-major row
                        umma_f8(d_tmem, smem_desc_join(a_lo + k4 * A_K32, DESC_HI), smem_desc_join(b_lo + k4 * B_K32, DESC_HI), IDESC, 1u);
                    umma_commit(empty0 + 8 * stage);
                    a_lo += A_STEP; b_lo += B_STEP;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                }
                if (ok) umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int wq = warp & 3;
        int it = 0;
        const bool vec_ok = (N % 8 == 0) && (reinterpret_cast<uintptr_t>(ep.D) % 16 == 0) &&
                            (reinterpret_cast<uintptr_t>(ep.col_scale) % 16 == 0) && (reinterpret_cast<uintptr_t>(ep.bias) % 16 == 0);
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            int tm, tn;
            fp8_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int row = tm * BM + wq * 32 + lane;
            const int n0 = tn * BN;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase, status, 0x34)) break;
            tc_fence_after();
            fp8_epilogue_tile<BN>(ep, tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + acc * BN, row, n0, M, N, vec_ok, sOut + wq * 4096);
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

template <int BN, int STAGES, bool B_KMAJOR>
int launch_fp8_instance(int M, int N, int K, const void* A, const void* B, const Fp8Epilogue& ep, cudaStream_t stream, int* status) {
    auto kernel = gemm_fp8_kernel<BN, STAGES, B_KMAJOR>;
    constexpr size_t smem = 1024 + static_cast<size_t>(STAGES) * (A_STAGE_BYTES + BN * BK) + EPI_STAGE_BYTES + (2 * STAGES + 4) * 8 + 16;
    static std::atomic<bool> attr_set[16];   // zero-initialised; set-once per device, a repeated set is harmless
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 16 && !attr_set[dev]) {
        B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_set[dev] = true;
    }
    CUtensorMap tmA, tmB;
    if (encode_tmap_2d(&tmA, A, 1, M, K, static_cast<uint64_t>(K), BM, BK) != 0) return -1;
    if (B_KMAJOR) { if (encode_tmap_2d(&tmB, B, 1, N, K, static_cast<uint64_t>(K), BN, BK) != 0) return -1; }
    else { if (encode_tmap_2d(&tmB, B, 1, K, N, static_cast<uint64_t>(N), BK, 128) != 0) return -1; }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    kernel<<<tiles < sm_count() ? tiles : sm_count(), 192, smem, stream>>>(tmA, tmB, ep, M, N, K, status);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}


// ---------------------------------------------------------------------------------------
// CTA-pair form (cta_group::2, 256 x 256 x 32 per instruction), the fp8 twin of the bf16 pair
// kernel: a pair owns a 256 x 256 tile, each CTA loads its 128 A rows and HALF of the B tile
// (32 KB per stage instead of 48 KB, ring 6 deep plus 16 KB of epilogue staging), the leader's single thread issues for both
// tensor cores, loads of both CTAs count on the leader's "full" barrier, epilogue warps of both
// CTAs release the accumulator on the leader's barrier.  No multicast of any kind.
// ---------------------------------------------------------------------------------------
constexpr int PBN = 256, PBNH = 128;
constexpr int PB_STAGE_BYTES = PBNH * BK;     // 16 KB
constexpr int P_GROUP_M = 8;                  // in pair tiles (8 x 256 rows)
constexpr int PAIR_EPI_WARPS = 8;
constexpr int PAIR_THREADS = 64 + 32 * PAIR_EPI_WARPS;

__device__ __forceinline__ void fp8_pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int group = P_GROUP_M * tiles_n;
    const int g = tile / group;
    const int first = g * P_GROUP_M;
    const int gm = min(P_GROUP_M, tiles_m - first);
    const int local = tile - g * group;
    tm = first + local % gm;
    tn = local / gm;
}

// ---- all-reduce of D inside the NVSwitch, fused into the pair kernel ---------------------------------------------------
// Tensor-parallel use: every rank computes a partial sum of the SAME [M][N] result (its slice of K) into its own copy of a
// buffer bound to one NVLink multicast object.  The unit of exchange is a CTA's part of a tile, 128 rows x 256 columns,
// slot = tile * 2 + cta.  Two extra warps per CTA do the exchange; the epilogue warps only count themselves on a
// shared-memory barrier after their stores, so the accumulators are released as fast as without it.
//   publisher warp: whenever all eight epilogue warps have stored further units (a shared-memory counter) -> one
//                   system-scope fence -> one 32-bit epoch per rank and unit into flags[rank][slot][me] (single writer per word);
//   reducer warp:   same tile order; when all ranks have published the unit it reduces this rank's 128 / world rows with
//                   multimem.ld_reduce (the switch fetches the rows from every rank and adds them in fp32) and writes the
//                   sums into every rank's copy with multimem.st, eight 512-byte rows in flight.
// The exchange of tile i thus runs while the tensor cores work on tiles i+1, i+2, ...  At the end every reducer warp
// meets the reducer warps of the same CTA index on the other ranks (fin flags): when the kernel has finished on a rank,
// every rank's sums have landed in its D.  All waits are bounded and report through the status word.
// Measured with the fence in the epilogue warps instead: each fence stalls its warp ~8 us, the epilogue falls behind
// the tensor cores and the GEMM takes 0.23 ms instead of 0.09 (4 GPUs, 8192 x 4096 x 4096).
// Needs M % 256 == 0, N % 256 == 0, world in {2, 4, 8}.
__device__ __forceinline__ bool sw_poll(const Fp8Epilogue& ep, const uint32_t* words, uint32_t epoch) {
    const int lane = threadIdx.x & 31;
    bool ok = true;
    if (lane < ep.sw_world) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(words + lane) : "memory");
        ok = static_cast<int32_t>(v - epoch) >= 0;
    }
    return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ bool sw_wait(const Fp8Epilogue& ep, const uint32_t* words, uint32_t epoch, int* status, int site) {
    const long long t0 = clock64();
    while (!sw_poll(ep, words, epoch)) {
        if (clock64() - t0 > 4000000000ll) { if ((threadIdx.x & 31) == 0) atomicCAS(status, ST_OK, (site << 8) | 1); return false; }
    }
    return true;
}
// every lane's earlier global stores -> visible at system scope, then the epoch into word [slot][me] of every rank
__device__ __forceinline__ void sw_publish(const Fp8Epilogue& ep, uint32_t* const* table, size_t slot, uint32_t epoch) {
    const int lane = threadIdx.x & 31;
    __syncwarp();
    if (lane < ep.sw_world) {
        __threadfence_system();
        uint32_t* w = table[lane] + slot * PYC_B200_TP_MAX_RANKS + ep.sw_rank;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(w), "r"(epoch) : "memory");
    }
}
__device__ __forceinline__ void sw_ld_reduce(char* addr, uint32_t (&v)[4]) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(addr) : "memory");
}
__device__ __forceinline__ void sw_st(char* addr, const uint32_t (&v)[4]) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
}
template <int STAGES, bool B_KMAJOR, bool SWITCH_REDUCE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SWITCH_REDUCE ? PAIR_THREADS + 64 : PAIR_THREADS, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Fp8Epilogue ep, int M, int N, int K, int* status) {
    constexpr uint32_t PAIR_TX = 2 * (A_STAGE_BYTES + PB_STAGE_BYTES);
    constexpr uint32_t TMEM_COLS = 2 * PBN;
    constexpr uint32_t IDESC = make_idesc(0, 0, 0, B_KMAJOR ? 0 : 1, 2 * BM, PBN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint8_t* sOut = sB + STAGES * PB_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + PAIR_EPI_WARPS * 4096);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 6);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16, stored0 = tempty0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + PBN - 1) / PBN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 2 * PAIR_EPI_WARPS); }  // epilogue warps of both CTAs
        *reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4) = 0u;   // at stored0: how many (epilogue warp, tile) parts this CTA has stored
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) { tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish_pair(); }
    tc_fence_before();
    cluster_sync_all();   // barriers of both CTAs exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leader_full0 = map_to_cta(full0, 0);
            const uint32_t a_dst0 = smem_u32(sA), b_dst0 = smem_u32(sB);
            uint32_t stage = 0, phase = 0, a_dst = a_dst0, b_dst = b_dst0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
                int tm, tn;
                fp8_pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * 2 * BM + static_cast<int>(rank) * BM;
                const int n0 = tn * PBN + static_cast<int>(rank) * PBNH;
                for (int kb = 0, k0 = 0; kb < num_kb; ++kb, k0 += BK) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, status, 0x35)) { ok = false; break; }
                    const uint32_t leader_full = leader_full0 + 8 * stage;
                    if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * stage, PAIR_TX);
                    tma_load_2d_pair(a_dst, &tmA, leader_full, k0, m0);
                    if (B_KMAJOR) tma_load_2d_pair(b_dst, &tmB, leader_full, k0, n0);
                    else tma_load_2d_pair(b_dst, &tmB, leader_full, n0, k0);
                    a_dst += A_STAGE_BYTES; b_dst += PB_STAGE_BYTES;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_dst = a_dst0; b_dst = b_dst0; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {  // the pair's single MMA issuer
            constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
            constexpr uint32_t A_STEP = A_STAGE_BYTES >> 4, B_STEP = PB_STAGE_BYTES >> 4;
            constexpr uint32_t A_K32 = 32 >> 4, B_K32 = (B_KMAJOR ? 32 : 32 * 128) >> 4;
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), B_KMAJOR ? 16 : BK * 128);
            const uint32_t empty_peer0 = map_to_cta(empty0, 1), tfull_peer0 = map_to_cta(tfull0, 1);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0;
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++it) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, status, 0x36)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * PBN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, status, 0x37)) { ok = false; break; }
                    tc_fence_after();
                    umma_f8_pair(d_tmem, smem_desc_join(a_lo, DESC_HI), smem_desc_join(b_lo, DESC_HI), IDESC, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k4 = 1; k4 < BK / 32; ++k4)
                        umma_f8_pair(d_tmem, smem_desc_join(a_lo + k4 * A_K32, DESC_HI), smem_desc_join(b_lo + k4 * B_K32, DESC_HI), IDESC, 1u);
                    umma_commit_pair(empty0 + 8 * stage);
                    umma_commit_pair(empty_peer0 + 8 * stage);
                    a_lo += A_STEP; b_lo += B_STEP;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                }
                if (ok) {
                    umma_commit_pair(tfull0 + 8 * acc);
                    umma_commit_pair(tfull_peer0 + 8 * acc);
                }
            }
        }
    } else if (warp < 2 + PAIR_EPI_WARPS) {
        // Eight epilogue warps: two per TMEM lane quarter, each taking half of the tile's columns.  With fp8 the main loop of a
        // tile is half as long as with bf16 while the epilogue (dequantise, bias, GELU, pack) is the same work, so four warps
        // could not keep up at K = 4096.
        const int wq = warp & 3;
        const int half = (warp - 2) >> 2;
        const uint32_t tempty_leader0 = map_to_cta(tempty0, 0);
        const bool vec_ok = (N % 8 == 0) && (reinterpret_cast<uintptr_t>(ep.D) % 16 == 0) &&
                            (reinterpret_cast<uintptr_t>(ep.col_scale) % 16 == 0) && (reinterpret_cast<uintptr_t>(ep.bias) % 16 == 0);
        int it = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            int tm, tn;
            fp8_pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int row = tm * 2 * BM + static_cast<int>(rank) * BM + wq * 32 + lane;
            const int n0 = tn * PBN;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase, status, 0x38)) break;
            tc_fence_after();
            fp8_epilogue_tile<PBN / 2>(ep, tmem_base + (static_cast<uint32_t>(wq * 32) << 16) + acc * PBN + half * (PBN / 2), row, n0 + half * (PBN / 2), M, N,
                                       vec_ok, sOut + (warp - 2) * 4096);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (SWITCH_REDUCE) asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(stored0) : "memory");
                mbar_arrive_cluster(tempty_leader0 + 8 * acc);
            }
        }
    } else if (SWITCH_REDUCE && warp == 2 + PAIR_EPI_WARPS) {
        // Publisher warp.  The epilogue warps count every part they have stored on a shared-memory counter (a counter, not
        // a phase barrier: the publisher may fall several tiles behind, its fence costs ~8 us and a tile can be shorter).
        // Whenever whole tiles have been stored since the last look: ONE system-scope fence, then one epoch word per rank
        // and tile.
        const uint32_t sw_epoch = ep.sw_epochs[blockIdx.x] + 1;
        const int my_tiles = pair < num_tiles ? (num_tiles - pair + pairs - 1) / pairs : 0;
        int published = 0;
        const long long t0 = clock64();
        while (published < my_tiles) {
            uint32_t c;
            asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(c) : "r"(stored0) : "memory");
            const int done = static_cast<int>(c / PAIR_EPI_WARPS);
            if (done > published) {
                if (lane < ep.sw_world) {
                    __threadfence_system();
                    for (int i = published; i < done; ++i) {
                        const int tile = pair + i * pairs;
                        uint32_t* w = ep.sw_flags[lane] + static_cast<size_t>(tile * 2 + static_cast<int>(rank)) * PYC_B200_TP_MAX_RANKS + ep.sw_rank;
                        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(w), "r"(sw_epoch) : "memory");
                    }
                }
                __syncwarp();
                published = done;
            } else if (clock64() - t0 > 4000000000ll) {
                if (lane == 0) atomicCAS(status, ST_OK, (0x39 << 8) | 1);
                break;
            }
        }
    } else if (SWITCH_REDUCE && warp == 3 + PAIR_EPI_WARPS) {
        // Reducer warp: follows the same tile order, waits until all ranks have published their 128 x 256 part and reduces
        // this rank's 128 / world rows of it in the switch, one 512-byte row per instruction, eight rows in flight.
        const uint32_t sw_epoch = ep.sw_epochs[blockIdx.x] + 1;
        const int share = 2 * BM / 2 / ep.sw_world;          // rows of a CTA's 128 that this rank reduces
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
            int tm, tn;
            fp8_pair_tile_coords(tile, tiles_m, tiles_n, tm, tn);
            ok = sw_wait(ep, ep.sw_flags[ep.sw_rank] + static_cast<size_t>(tile * 2 + static_cast<int>(rank)) * PYC_B200_TP_MAX_RANKS, sw_epoch, status, 0x3a);
            if (!ok) break;
            char* base = ep.sw_mc + (static_cast<size_t>(tm * 2 * BM + static_cast<int>(rank) * BM + ep.sw_rank * share) * N + tn * PBN + lane * 8) * 2;
            const size_t row_bytes = static_cast<size_t>(N) * 2;
            for (int j0 = 0; j0 < share; j0 += 8) {      // eight rows (4 KB) in flight; sixteen were slower (0.219 against 0.197 ms at 4 GPUs)
                uint32_t v[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) sw_ld_reduce(base + (j0 + j) * row_bytes, v[j]);
#pragma unroll
                for (int j = 0; j < 8; ++j) sw_st(base + (j0 + j) * row_bytes, v[j]);
            }
        }
        // this rank's sums have been written everywhere; leave only when the reducer warps of all ranks say the same
        sw_publish(ep, ep.sw_fin, static_cast<size_t>(blockIdx.x), sw_epoch);
        sw_wait(ep, ep.sw_fin[ep.sw_rank] + static_cast<size_t>(blockIdx.x) * PYC_B200_TP_MAX_RANKS, sw_epoch, status, 0x3c);
    }

    // Both CTAs meet here (also after a timed-out wait): neither exits while the other may still signal its barriers
    // or read its shared memory.
    tc_fence_before();
    cluster_sync_all();
    if (SWITCH_REDUCE && threadIdx.x == 0) ep.sw_epochs[blockIdx.x] += 1;   // every epilogue thread read it before the loop
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(status) != ST_OK) for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <int STAGES, bool B_KMAJOR, bool SWITCH_REDUCE = false>
int launch_fp8_pair_instance(int M, int N, int K, const void* A, const void* B, const Fp8Epilogue& ep, cudaStream_t stream, int* status) {
    auto kernel = gemm_fp8_pair_kernel<STAGES, B_KMAJOR, SWITCH_REDUCE>;
    constexpr size_t smem = 1024 + static_cast<size_t>(STAGES) * (A_STAGE_BYTES + PB_STAGE_BYTES) + PAIR_EPI_WARPS * 4096 + (2 * STAGES + 6) * 8 + 16;
    static std::atomic<bool> attr_set[16];   // zero-initialised; set-once per device, a repeated set is harmless
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 16 && !attr_set[dev]) {
        B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_set[dev] = true;
    }
    CUtensorMap tmA, tmB;
    if (encode_tmap_2d(&tmA, A, 1, M, K, static_cast<uint64_t>(K), BM, BK) != 0) return -1;
    if (B_KMAJOR) { if (encode_tmap_2d(&tmB, B, 1, N, K, static_cast<uint64_t>(K), PBNH, BK) != 0) return -1; }
    else { if (encode_tmap_2d(&tmB, B, 1, K, N, static_cast<uint64_t>(N), BK, 128) != 0) return -1; }
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + PBN - 1) / PBN);
    const int max_pairs = sm_count() / 2;
    const int grid = 2 * (tiles < max_pairs ? tiles : max_pairs);
    kernel<<<grid, SWITCH_REDUCE ? PAIR_THREADS + 64 : PAIR_THREADS, smem, stream>>>(tmA, tmB, ep, M, N, K, status);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

}  // namespace

int launch_gemm_fp8(int M, int N, int K, const void* A, const void* B, int b_col_major, const float* row_scale, const float* col_scale,
                    const void* bias, int act, void* D, cudaStream_t stream, int* status, const Fp8Scatter* scatter, const Fp8SwitchReduce* sw) {
    if (M <= 0 || N <= 0 || K <= 0 || !A || !B || (!D && !scatter) || !status) { set_error("fp8 gemm: bad shape or NULL pointer"); return -1; }
    if (scatter && (scatter->world < 1 || scatter->world > PYC_B200_TP_MAX_RANKS || scatter->rank < 0 || scatter->rank >= scatter->world ||
                    M % scatter->world != 0)) { set_error("fp8 gemm: bad scatter description (world %d, rank %d, M %d)", scatter->world, scatter->rank, M); return -1; }
    if (K % 16 != 0 || (!b_col_major && N % 16 != 0) || reinterpret_cast<uintptr_t>(A) % 16 || reinterpret_cast<uintptr_t>(B) % 16) {
        set_error("fp8 gemm: needs K %% 16 == 0, N %% 16 == 0 for row-major B and 16-byte aligned operands (TMA)"); return -1;
    }
    Fp8Epilogue ep;
    ep.D = static_cast<__nv_bfloat16*>(D); ep.row_scale = row_scale; ep.col_scale = col_scale;
    ep.bias = static_cast<const __nv_bfloat16*>(bias); ep.act = act;
    ep.world = 0; ep.rows_per_rank = 0; ep.src_rank = 0;
    for (int i = 0; i < PYC_B200_TP_MAX_RANKS; ++i) ep.dst[i] = nullptr;
    ep.sw_mc = nullptr; ep.sw_epochs = nullptr; ep.sw_world = 0; ep.sw_rank = 0;
    for (int i = 0; i < PYC_B200_TP_MAX_RANKS; ++i) { ep.sw_flags[i] = nullptr; ep.sw_fin[i] = nullptr; }
    if (sw) {
        const int w = sw->world;
        if (scatter || b_col_major || !D || (w != 2 && w != 4 && w != 8) || sw->rank < 0 || sw->rank >= w || M % 256 || N % 256 || !sw->multicast_d || !sw->epochs ||
            reinterpret_cast<uintptr_t>(sw->multicast_d) % 16 || reinterpret_cast<uintptr_t>(D) % 16) {
            set_error("fp8 gemm with in-switch reduce: needs row-major B, M %% 256 == 0, N %% 256 == 0, 2, 4 or 8 ranks, a 16-byte aligned D and its multicast address");
            return -1;
        }
        if (2 * std::min(static_cast<long long>(M / 256) * (N / 256), static_cast<long long>(sm_count() / 2)) > PYC_B200_TP_FUSED_EPOCH_SLOTS) {
            set_error("fp8 gemm with in-switch reduce: more CTAs than PYC_B200_TP_FUSED_EPOCH_SLOTS"); return -1;
        }
        ep.sw_mc = static_cast<char*>(sw->multicast_d); ep.sw_epochs = static_cast<uint32_t*>(sw->epochs); ep.sw_world = w; ep.sw_rank = sw->rank;
        for (int i = 0; i < w; ++i) {
            if (!sw->flags[i] || !sw->fin[i]) { set_error("fp8 gemm with in-switch reduce: flag buffer %d is NULL", i); return -1; }
            ep.sw_flags[i] = static_cast<uint32_t*>(sw->flags[i]); ep.sw_fin[i] = static_cast<uint32_t*>(sw->fin[i]);
        }
        return launch_fp8_pair_instance<6, false, true>(M, N, K, A, B, ep, stream, status);
    }
    if (scatter) {
        ep.world = scatter->world; ep.rows_per_rank = M / scatter->world; ep.src_rank = scatter->rank;
        for (int i = 0; i < scatter->world; ++i) {
            if (!scatter->dst[i] || reinterpret_cast<uintptr_t>(scatter->dst[i]) % 16) { set_error("fp8 gemm: scatter slot %d is NULL or not 16-byte aligned", i); return -1; }
            ep.dst[i] = static_cast<__nv_bfloat16*>(scatter->dst[i]);
        }
        if (!ep.D) ep.D = ep.dst[scatter->rank];   // only its alignment is looked at
    }
    const int sms = sm_count();
    const long long t256 = static_cast<long long>((M + 127) / 128) * ((N + 255) / 256), t128 = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
    const bool use256 = ((t256 + sms - 1) / sms) * 256 <= ((t128 + sms - 1) / sms) * 128 * 1.15;
    // CTA pairs once there is at least a wave of 256 x 256 tiles (PYC_B200_FP8_PAIR=0: never, =1: always)
    const char* pe = getenv("PYC_B200_FP8_PAIR");
    const long long pair_tiles = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256);
    if (pe && (pe[0] == '0' || pe[0] == '1') ? pe[0] == '1' : pair_tiles >= sms / 2)
        return b_col_major ? launch_fp8_pair_instance<6, true>(M, N, K, A, B, ep, stream, status) : launch_fp8_pair_instance<6, false>(M, N, K, A, B, ep, stream, status);
    if (use256) return b_col_major ? launch_fp8_instance<256, 4, true>(M, N, K, A, B, ep, stream, status) : launch_fp8_instance<256, 4, false>(M, N, K, A, B, ep, stream, status);
    return b_col_major ? launch_fp8_instance<128, 6, true>(M, N, K, A, B, ep, stream, status) : launch_fp8_instance<128, 6, false>(M, N, K, A, B, ep, stream, status);
}

}  // namespace b200
