// bf16 / f16 GEMM on the 5th-generation tensor cores (tcgen05) with a fused
// epilogue: D = act(alpha * A*B + add_scale * add).
//
// Replaces the tensor-core lane of PyC's CUDA backend: the CUTLASS sm80
// mma.sync kernels of src/compiler/cutlass_kernels/gemm/kernel.cu:48-84 and the
// cublasGemmEx bf16/f16 path of src/compiler/runtime/cuda_backend.c:849-896,
// plus the host-side add/relu loops of cuda_backend.c:1697-1742, which here run
// in the kernel's epilogue.
//
// One persistent CTA per SM, 192 threads, warp-specialised:
//   warp 0      TMA producer: A [128 x 64] and B [64 x BN] tiles, 128-byte
//               swizzled, STAGES-deep ring, per-CTA loads only
//   warp 1      allocates TMEM, one lane issues tcgen05.mma (128 x BN x 16)
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns, bias / activation,
//               convert, 16-byte global stores
// Two fp32 accumulators of 128 x BN live in TMEM (2*BN columns), so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Data layout: A row-major [M,K] (K-major operand).  B row-major [K,N] is an
// MN-major operand: each TMA box is 64 n-values (128 B) by 64 k-rows, boxes for
// consecutive 64-column chunks sit 8 KB apart (descriptor LBO), 8-row groups
// 1 KB apart (SBO).  B stored [N,K] is the K-major form.
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include <mutex>

#include "internal.h"
#include "math.cuh"
#include "ptx_sm100.cuh"

namespace b200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int GROUP_M = 16;

struct Epilogue {
    void* D;
    const void* add;
    float alpha, add_scale;
    int add_mode, act, vec_ok;
    int group_m;     // M-tiles per rasterisation group
    int l2_hints;    // 0 none, 1 A evict_last + B evict_first, 2 both evict_last
};

template <int FMT> struct Elem;
template <> struct Elem<1> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float to_f(T v) { return __bfloat162float(v); }
    static __device__ __forceinline__ T from_f(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&p);
    }
    static __device__ __forceinline__ void unpack(uint32_t u, float& a, float& b) {
        a = __uint_as_float(u << 16); b = __uint_as_float(u & 0xffff0000u);
    }
};
template <> struct Elem<0> {
    using T = __half;
    static __device__ __forceinline__ float to_f(T v) { return __half2float(v); }
    static __device__ __forceinline__ T from_f(float v) { return __float2half_rn(v); }
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 p = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&p);
    }
    static __device__ __forceinline__ void unpack(uint32_t u, float& a, float& b) {
        __half2 p = *reinterpret_cast<__half2*>(&u);
        float2 f = __half22float2(p); a = f.x; b = f.y;
    }
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
    const int group = group_m * tiles_n;
    const int g = tile / group;
    const int first = g * group_m;
    const int gm = min(group_m, tiles_m - first);
    const int local = tile - g * group;
    tm = first + local % gm;
    tn = local / gm;
}

template <int BN, int STAGES, bool B_KMAJOR, int FMT>
__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               Epilogue ep, int M, int N, int K, int* status) {
    constexpr int B_STAGE_BYTES = BN * BK * 2;
    constexpr uint32_t STAGE_TX = A_STAGE_BYTES + B_STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = make_idesc(FMT, FMT, 0, B_KMAJOR ? 0 : 1, BM, BN);
    using E = Elem<FMT>;
    using T = typename E::T;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;
    uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * B_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES;
    const uint32_t tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM;
    const int tiles_n = (N + BN - 1) / BN;
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
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t a_dst0 = smem_u32(sA), b_dst0 = smem_u32(sB);
            uint32_t stage = 0, phase = 0, adst = a_dst0, bdst = b_dst0;
            bool ok = true;
            const uint64_t pol_a = l2_policy_evict_last();
            const uint64_t pol_b = ep.l2_hints == 2 ? l2_policy_evict_last() : l2_policy_evict_first();
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, ep.group_m, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, status, 1)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * stage;
                    mbar_arrive_expect_tx(fb, STAGE_TX);
                    if (ep.l2_hints == 1 || ep.l2_hints == 2) {
                        tma_load_2d_hint(adst, &tmA, fb, kb * BK, m0, pol_a);
                        if (B_KMAJOR) {
                            tma_load_2d_hint(bdst, &tmB, fb, kb * BK, n0, pol_b);
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / 64; ++j) tma_load_2d_hint(bdst + j * (BK * 128), &tmB, fb, n0 + j * 64, kb * BK, pol_b);
                        }
                    } else {
                        tma_load_2d(adst, &tmA, fb, kb * BK, m0);
                        if (B_KMAJOR) {
                            tma_load_2d(bdst, &tmB, fb, kb * BK, n0);
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / 64; ++j) tma_load_2d(bdst + j * (BK * 128), &tmB, fb, n0 + j * 64, kb * BK);
                        }
                    }
                    adst += A_STAGE_BYTES; bdst += B_STAGE_BYTES;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; adst = a_dst0; bdst = b_dst0; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // This loop has to come round once per k-block of tensor-pipe time while sharing its scheduler with an
            // epilogue warp: descriptor high words are constants and the low words are stepped, not rebuilt.
            constexpr uint32_t DESC_HI = smem_desc_hi_sw128(1024);
            constexpr uint32_t A_STEP = A_STAGE_BYTES >> 4, B_STEP = B_STAGE_BYTES >> 4;
            constexpr uint32_t A_K16 = 32 >> 4, B_K16 = (B_KMAJOR ? 32 : 2048) >> 4;
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA), 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_u32(sB), B_KMAJOR ? 16 : BK * 128);
            uint32_t stage = 0, phase = 0, a_lo = a_lo0, b_lo = b_lo0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, status, 2)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase, status, 3)) { ok = false; break; }
                    tc_fence_after();
                    umma_f16(d_tmem, smem_desc_join(a_lo, DESC_HI), smem_desc_join(b_lo, DESC_HI), IDESC, kb != 0 ? 1u : 0u);
#pragma unroll
                    for (uint32_t k4 = 1; k4 < BK / 16; ++k4)
                        umma_f16(d_tmem, smem_desc_join(a_lo + k4 * A_K16, DESC_HI), smem_desc_join(b_lo + k4 * B_K16, DESC_HI), IDESC, 1u);
                    umma_commit(empty0 + 8 * stage);
                    a_lo += A_STEP; b_lo += B_STEP;
                    if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
                }
                if (ok) umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int wq = warp & 3;  // TMEM lane quarter this warp may read
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        const T* addp = reinterpret_cast<const T*>(ep.add);
        const float scalar_add = ep.add_mode == PYC_B200_ADD_SCALAR ? ep.add_scale * E::to_f(addp[0]) : 0.0f;
        int it = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, ep.group_m, tm, tn);
            const int row = tm * BM + wq * 32 + lane;
            const int n0 = tn * BN;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase, status, 4)) break;
            tc_fence_after();
            T* drow = reinterpret_cast<T*>(ep.D) + static_cast<size_t>(row) * N;
            const uint32_t acc_addr = lane_base + acc * BN;
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
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < N) v[j] += ep.add_scale * E::to_f(src[j]);
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
                    if (ep.vec_ok == 2) {
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
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < N) drow[col0 + j] = E::from_f(v[j]);
                }
            };
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(acc_addr, r0);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c += 2) {
                tmem_ld_wait();
                tmem_ld_32x32(acc_addr + (c + 1) * 32, r1);
                chunk(r0, c);
                __syncwarp();
                tmem_ld_wait();
                if (c + 2 < BN / 32) tmem_ld_32x32(acc_addr + (c + 2) * 32, r0);
                chunk(r1, c + 1);
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        }
    }

    // Teardown: every role falls through to here, also after a timed-out wait.
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(status) != ST_OK) {
            // A wait gave up: give copies and MMAs in flight time to land before the CTA's
            // shared memory and TMEM go away.
            for (int i = 0; i < 2000; ++i) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Tile rasterisation knobs: PYC_B200_GEMM_GROUP_M (M-tiles per group) and PYC_B200_GEMM_L2_HINTS (0, 1, 2) override the defaults.
inline void tile_order_from_env(int* group_m, int* l2_hints) {
    *group_m = GROUP_M;
    *l2_hints = 0;
    if (const char* g = getenv("PYC_B200_GEMM_GROUP_M")) { const int v = atoi(g); if (v >= 1 && v <= 1024) *group_m = v; }
    if (const char* h = getenv("PYC_B200_GEMM_L2_HINTS")) { const int v = atoi(h); if (v >= 0 && v <= 2) *l2_hints = v; }
}

template <int BN, int STAGES>
constexpr size_t tc_smem_bytes() {
    return 1024 + static_cast<size_t>(STAGES) * (A_STAGE_BYTES + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16;
}

template <int BN, int STAGES, bool B_KMAJOR, int FMT>
int launch_instance(const GemmProblem& p, cudaStream_t stream, int* status) {
    auto kernel = gemm_tc_kernel<BN, STAGES, B_KMAJOR, FMT>;
    constexpr size_t smem = tc_smem_bytes<BN, STAGES>();
    static std::atomic<bool> attr_set[16];   // zero-initialised; set-once per device, a repeated set is harmless
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 16 && !attr_set[dev]) {
        B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_set[dev] = true;
    }
    CUtensorMap tmA, tmB;
    if (encode_tmap_2d(&tmA, p.A, 2, p.M, p.K, static_cast<uint64_t>(p.K) * 2, BM, BK) != 0) return -1;
    if (B_KMAJOR) {
        if (encode_tmap_2d(&tmB, p.B, 2, p.N, p.K, static_cast<uint64_t>(p.K) * 2, BN, BK) != 0) return -1;
    } else {
        if (encode_tmap_2d(&tmB, p.B, 2, p.K, p.N, static_cast<uint64_t>(p.N) * 2, BK, 64) != 0) return -1;
    }
    Epilogue ep;
    ep.D = p.D; ep.add = p.add; ep.alpha = p.alpha; ep.add_scale = p.add_scale;
    ep.add_mode = p.add ? p.add_mode : PYC_B200_ADD_NONE; ep.act = p.act;
    const bool aligned = (reinterpret_cast<uintptr_t>(p.D) % 16 == 0) && (p.N % 8 == 0) &&
                         (ep.add_mode == PYC_B200_ADD_NONE || ep.add_mode == PYC_B200_ADD_SCALAR ||
                          reinterpret_cast<uintptr_t>(p.add) % 16 == 0);
    ep.vec_ok = aligned ? ((reinterpret_cast<uintptr_t>(p.D) % 32 == 0 && p.N % 16 == 0) ? 2 : 1) : 0;   // 2: rows start on 32-byte boundaries
    tile_order_from_env(&ep.group_m, &ep.l2_hints);
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    kernel<<<grid, 192, smem, stream>>>(tmA, tmB, ep, p.M, p.N, p.K, status);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

template <int BN, int STAGES>
int launch_by_layout(const GemmProblem& p, cudaStream_t stream, int* status) {
    const bool bf16 = p.dtype == PYC_DTYPE_BF16;
    if (p.b_col_major) return bf16 ? launch_instance<BN, STAGES, true, 1>(p, stream, status) : launch_instance<BN, STAGES, true, 0>(p, stream, status);
    return bf16 ? launch_instance<BN, STAGES, false, 1>(p, stream, status) : launch_instance<BN, STAGES, false, 0>(p, stream, status);
}

}  // namespace

int launch_gemm_tc(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream, int* status) {
    if (cfg.bn == 256 && cfg.stages == 4) return launch_by_layout<256, 4>(p, stream, status);
    if (cfg.bn == 128 && cfg.stages == 6) return launch_by_layout<128, 6>(p, stream, status);
    if (cfg.bn == 64 && cfg.stages == 8) return launch_by_layout<64, 8>(p, stream, status);
    set_error("no tensor-core GEMM instance for tile %dx%dx%d stages %d", cfg.bm, cfg.bn, cfg.bk, cfg.stages);
    return -1;
}

// ---------------------------------------------------------------------------
// pyc_b200_gemm_static: the same tensor-core GEMM for callers that must not
// allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they
// need a GEMM: a serving loop that has already handed all device memory to its
// own pool (PyC's Rust runtime keeps such a pool), code running while a stream
// capture is open elsewhere in the process, or a latency-critical thread that
// cannot afford the device-wide synchronisation an allocation implies.  The
// ordinary entry points create a per-device context on first use (stream,
// status word, pinned mirror).  This one touches none of that: the only scratch
// the kernel needs -- the status block its bounded waits report into -- lives
// in the file-scope device array below, which every GPU that loads the library
// holds (256 bytes) until the process exits.
//
// The first call on each device resolves the array's device address with
// cudaGetSymbolAddress (the name below is only a host-side handle, not a device
// pointer), raises the kernel's dynamic shared-memory limit and reads the SM
// count.  Make that first call before any stream capture begins.  Every call
// shares the one block and clears it on `stream` before launching, so two calls
// whose kernels overlap on the GPU (different streams) race on it: keep calls
// on one stream, or order them with events.
// ---------------------------------------------------------------------------
namespace {

constexpr int kStaticScratchBytes = 256;
constexpr int kStaticMaxDim = 1 << 20;  // largest M, N or K accepted; the kernel's 32-bit tile arithmetic is checked up to here
static __device__ __align__(256) int g_static_scratch[kStaticScratchBytes / sizeof(int)];

struct StaticDeviceSetup {
    bool ready = false;
    int* scratch = nullptr;  // device address of g_static_scratch on this device
    int sms = 0;
    bool attr[3][2][2] = {};
};
StaticDeviceSetup g_static_setup[16];

template <int BN, int STAGES, bool B_KMAJOR, int FMT>
int launch_static_instance(const GemmProblem& p, cudaStream_t stream, StaticDeviceSetup& sd, int bn_index) {
    auto kernel = gemm_tc_kernel<BN, STAGES, B_KMAJOR, FMT>;
    constexpr size_t smem = tc_smem_bytes<BN, STAGES>();
    if (!sd.attr[bn_index][B_KMAJOR ? 1 : 0][FMT]) {
        B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        sd.attr[bn_index][B_KMAJOR ? 1 : 0][FMT] = true;
    }
    CUtensorMap tmA, tmB;
    if (encode_tmap_2d(&tmA, p.A, 2, p.M, p.K, static_cast<uint64_t>(p.K) * 2, BM, BK) != 0) return -1;
    if (B_KMAJOR) {
        if (encode_tmap_2d(&tmB, p.B, 2, p.N, p.K, static_cast<uint64_t>(p.K) * 2, BN, BK) != 0) return -1;
    } else {
        if (encode_tmap_2d(&tmB, p.B, 2, p.K, p.N, static_cast<uint64_t>(p.N) * 2, BK, 64) != 0) return -1;
    }
    Epilogue ep;
    ep.D = p.D; ep.add = p.add; ep.alpha = p.alpha; ep.add_scale = p.add_scale;
    ep.add_mode = p.add ? p.add_mode : PYC_B200_ADD_NONE; ep.act = p.act;
    ep.vec_ok = ((reinterpret_cast<uintptr_t>(p.D) % 16 == 0) && (p.N % 8 == 0) &&
                 (ep.add_mode == PYC_B200_ADD_NONE || ep.add_mode == PYC_B200_ADD_SCALAR || reinterpret_cast<uintptr_t>(p.add) % 16 == 0)) ? 1 : 0;
    if (ep.vec_ok && reinterpret_cast<uintptr_t>(p.D) % 32 == 0 && p.N % 16 == 0) ep.vec_ok = 2;   // rows start on 32-byte boundaries
    tile_order_from_env(&ep.group_m, &ep.l2_hints);
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    // The block keeps whatever the previous call left: the status word must start at zero.
    B200_CUDA_OK(cudaMemsetAsync(sd.scratch, 0, kStaticScratchBytes, stream));
    kernel<<<tiles < sd.sms ? tiles : sd.sms, 192, smem, stream>>>(tmA, tmB, ep, p.M, p.N, p.K, sd.scratch);
    B200_CUDA_OK(cudaGetLastError());
    count_launch();
    return 0;
}

template <int BN, int STAGES>
int launch_static_layout(const GemmProblem& p, cudaStream_t stream, StaticDeviceSetup& sd, int bn_index) {
    const bool bf16 = p.dtype == PYC_DTYPE_BF16;
    if (p.b_col_major) return bf16 ? launch_static_instance<BN, STAGES, true, 1>(p, stream, sd, bn_index) : launch_static_instance<BN, STAGES, true, 0>(p, stream, sd, bn_index);
    return bf16 ? launch_static_instance<BN, STAGES, false, 1>(p, stream, sd, bn_index) : launch_static_instance<BN, STAGES, false, 0>(p, stream, sd, bn_index);
}

}  // namespace
}  // namespace b200

extern "C" int pyc_b200_gemm_static(const pyc_b200_gemm_args* a, void* stream) {
    using namespace b200;
    if (!a || !a->A || !a->B || !a->D) { set_error("pyc_b200_gemm_static: NULL argument"); return -1; }
    if (a->dtype != PYC_DTYPE_BF16 && a->dtype != PYC_DTYPE_F16) { set_error("pyc_b200_gemm_static: only bf16 and f16 (the tensor-core kernel)"); return -1; }
    if (a->M <= 0 || a->N <= 0 || a->K <= 0) { set_error("pyc_b200_gemm_static: M, N, K must be positive"); return -1; }
    if (a->M > kStaticMaxDim || a->N > kStaticMaxDim || a->K > kStaticMaxDim) {
        set_error("pyc_b200_gemm_static: %dx%dx%d exceeds the supported maximum of %d per dimension", a->M, a->N, a->K, kStaticMaxDim);
        return -1;
    }
    if (a->K % 8 != 0 || (!a->b_col_major && a->N % 8 != 0) || reinterpret_cast<uintptr_t>(a->A) % 16 || reinterpret_cast<uintptr_t>(a->B) % 16) {
        set_error("pyc_b200_gemm_static: needs K %% 8 == 0, N %% 8 == 0 for row-major B, and 16-byte aligned A and B (TMA)");
        return -1;
    }
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) { set_error("pyc_b200_gemm_static: device index %d out of range", dev); return -1; }
    StaticDeviceSetup& sd = g_static_setup[dev];
    static std::mutex* setup_mu = new std::mutex();
    std::lock_guard<std::mutex> setup_lock(*setup_mu);  // set-up and the shared block's clear+launch pair stay ordered per process
    if (!sd.ready) {
        // Once per device, with that device current.  The symbol name is a host-side stand-in; the kernel
        // needs the address the driver reports for this device.
        int major = 0, sms = 0;
        B200_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        B200_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (major != 10) { set_error("pyc_b200_gemm_static: needs an sm_100 device, found compute capability major %d", major); return -1; }
        void* ptr = nullptr;
        B200_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) { set_error("pyc_b200_gemm_static: cudaGetSymbolAddress returned NULL"); return -1; }
        sd.scratch = static_cast<int*>(ptr);
        sd.sms = sms;
        sd.ready = true;
    }
    GemmProblem p;
    p.dtype = a->dtype; p.M = a->M; p.N = a->N; p.K = a->K; p.A = a->A; p.B = a->B; p.D = a->D;
    p.b_col_major = a->b_col_major != 0; p.alpha = a->alpha; p.add_mode = a->add_mode; p.add = a->add; p.act = a->act;
    // Tile width by the same wave-count estimate the allocating path uses.
    int best_bn = 256;
    double best_cost = 0.0;
    const int bns[3] = {256, 128, 64};
    const double eff[3] = {1.0, 0.85, 0.6};
    for (int i = 0; i < 3; ++i) {
        const double tiles = static_cast<double>((p.M + 127) / 128) * ((p.N + bns[i] - 1) / bns[i]);
        const double waves = static_cast<double>(static_cast<long long>((tiles + sd.sms - 1) / sd.sms));
        const double cost = waves * 128 * bns[i] / eff[i];
        if (i == 0 || cost < best_cost) { best_cost = cost; best_bn = bns[i]; }
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (best_bn == 256) return launch_static_layout<256, 4>(p, s, sd, 0);
    if (best_bn == 128) return launch_static_layout<128, 6>(p, s, sd, 1);
    return launch_static_layout<64, 8>(p, s, sd, 2);
}

// Allocation-free reader of the static block's status word.  The kernel's bounded waits record a code there when they
// give up; without this a caller of pyc_b200_gemm_static could not tell a timed-out GEMM from a good one, because the
// ordinary status call reads the per-device context (and creating that context allocates).
extern "C" int pyc_b200_gemm_static_status(int* host_out, void* stream) {
    using namespace b200;
    if (!host_out) { set_error("pyc_b200_gemm_static_status: NULL destination"); return -1; }
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16 || !g_static_setup[dev].ready) {
        // Nothing has been launched through the static entry on this device: there is nothing to report.
        *host_out = 0;
        return 0;
    }
    B200_CUDA_OK(cudaMemcpyAsync(host_out, g_static_setup[dev].scratch, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return 0;
}
