// Internal interfaces between the dispatch layer and the kernel files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <string>

#include "pyc_b200.h"

namespace b200 {

// ---- errors ---------------------------------------------------------------
void set_error(const char* fmt, ...);
const char* last_error();
#define B200_CUDA_OK(expr)                                                         \
    do {                                                                           \
        cudaError_t e__ = (expr);                                                  \
        if (e__ != cudaSuccess) {                                                  \
            ::b200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
            return -1;                                                             \
        }                                                                          \
    } while (0)

inline size_t dtype_size(pyc_dtype d) {
    switch (d) { case PYC_DTYPE_F32: case PYC_DTYPE_I32: return 4; case PYC_DTYPE_F16: case PYC_DTYPE_BF16: return 2; case PYC_DTYPE_I8: return 1; default: return 0; }
}

// Counts every kernel this library enqueues (telemetry; also the benchmark's
// launch count).
void count_launch(size_t n = 1);
size_t launches_total();

// Device status word of the current device's context: kernels write a non-zero
// code when a bounded wait runs out.  Zeroed when the context is created.
int* device_status_word();
// Synchronise nothing; read the status word with a blocking copy on `stream`.
int read_device_status(cudaStream_t stream);

// ---- tensor maps ------------------------------------------------------------
// Encode a 2D tiled tensor map over a row-major [rows, cols] matrix of 1-, 2- or
// 4-byte elements: box = box_rows x box_cols, 128-byte swizzle (box_cols * elem
// must be 128 bytes), out-of-bounds reads fill with zero.  Returns 0 / -1.
int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                   uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols);
// General form: up to 5 dims, innermost first; strides in bytes for dims 1..n-1.
int encode_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

// ---- GEMM -------------------------------------------------------------------
struct GemmProblem {
    pyc_dtype dtype = PYC_DTYPE_UNKNOWN;
    int M = 0, N = 0, K = 0;
    const void* A = nullptr;   // [M,K] row-major
    const void* B = nullptr;   // [K,N] row-major, or [N,K] when b_col_major
    void* D = nullptr;         // [M,N] row-major
    bool b_col_major = false;
    float alpha = 1.0f;
    int add_mode = PYC_B200_ADD_NONE;
    const void* add = nullptr;
    float add_scale = 1.0f;    // D = act(alpha*A*B + add_scale*add)
    int act = PYC_B200_ACT_NONE;
};

enum GemmKind { GEMM_TC = 0, GEMM_SIMT = 1, GEMM_TC_PAIR = 2 };
struct GemmConfig {
    const char* symbol;
    GemmKind kind;
    int dtype_mask;            // bit (1 << pyc_dtype)
    int bm, bn, bk, stages;
    int priority;
    size_t smem_bytes;
    pyc_kernel_workload_family workload;
};
const GemmConfig* gemm_configs(int* count);
const GemmConfig* find_gemm_config(const char* symbol);
// Current choice for (dtype, shape): autotune winner if one was measured, else
// the registry's promoted symbol, else a shape heuristic.
const GemmConfig* choose_gemm_config(const GemmProblem& p);
void remember_gemm_winner(pyc_dtype dtype, int M, int N, int K, const GemmConfig* cfg);
bool gemm_config_supports(const GemmConfig& cfg, const GemmProblem& p);
// Who made the last choose_gemm_config() decision of this thread: "autotune", "env", "promoted", "registry" or "model".
const char* last_selection_source();
// Bumped whenever a per-shape winner changes; part of the dispatch layer's graph-cache key.
uint64_t selection_epoch();
// PyC's workload classes for a matmul shape (compiler_api.c:1141-1170).
pyc_kernel_workload_family matmul_workload_family(size_t m, size_t n, size_t k);
// Load persisted timings / per-shape winners (path NULL: PYC_AUTOTUNE_DB_PATH).  Returns winners installed, -1 without a path.
int autotune_db_load(const char* path);

int launch_gemm(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream);
// kernel-file entry points
int launch_gemm_tc(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream, int* status);
int launch_gemm_simt(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream);
int launch_gemm_tc_pair(const GemmConfig& cfg, const GemmProblem& p, cudaStream_t stream, int* status);

// ---- elementwise / reductions ------------------------------------------------
int launch_add(pyc_dtype dt, const void* a, const void* b, void* out, size_t n, cudaStream_t s);
int launch_bias_act(pyc_dtype dt, const void* x, const void* add, int add_mode, int act, void* out,
                    size_t rows, size_t cols, cudaStream_t s);
int launch_layernorm(pyc_dtype dt, const void* x, const void* gamma, const void* beta, void* out,
                     size_t rows, size_t cols, float eps, cudaStream_t s);
int launch_softmax(pyc_dtype dt, const void* x, void* out, size_t rows, size_t cols, cudaStream_t s);
int launch_reduce_sum(pyc_dtype dt, const void* x, void* out, size_t rows, size_t cols, cudaStream_t s);

// ---- attention / conv ----------------------------------------------------------
int launch_attention(pyc_dtype dt, int batch_heads, int seq, int d, const void* q, const void* k, const void* v,
                     void* out, float scale, int causal, cudaStream_t s, int* status);
int launch_conv2d(pyc_dtype dt, int N, int H, int W, int C, int K, int R, int S, int pad_h, int pad_w,
                  int stride_h, int stride_w, const void* in, const void* filt, const void* bias, int relu,
                  void* out, cudaStream_t s, int* status);

// ---- fp8 GEMM (+ row scatter for tensor parallelism) / row quantisers --------------
struct Fp8Scatter {
    void* dst[PYC_B200_TP_MAX_RANKS];   // receive buffer of every rank: [world][M / world][N] bf16
    int world, rank;
};
// In-switch all-reduce of D fused into the GEMM (CTA-pair kernel only): see gemm_fp8.cu.
struct Fp8SwitchReduce {
    void* multicast_d;                       // multicast address of D (every rank's D bound to one NVLink multicast object)
    void* flags[PYC_B200_TP_MAX_RANKS];      // per rank: [(M/256) * (N/256) * 2][PYC_B200_TP_MAX_RANKS] uint32
    void* fin[PYC_B200_TP_MAX_RANKS];        // per rank: [PYC_B200_TP_FUSED_EPOCH_SLOTS][PYC_B200_TP_MAX_RANKS] uint32
    void* epochs;                            // local: [PYC_B200_TP_FUSED_EPOCH_SLOTS] uint32
    int world, rank;
};
int launch_gemm_fp8(int M, int N, int K, const void* A, const void* B, int b_col_major, const float* row_scale, const float* col_scale,
                    const void* bias, int act, void* D, cudaStream_t stream, int* status, const Fp8Scatter* scatter = nullptr,
                    const Fp8SwitchReduce* switch_reduce = nullptr);

// ---- registry -------------------------------------------------------------------
void registry_init_once();
int registry_count(const char* op_key);
bool registry_promoted_symbol(const char* op_key, std::string* out);
void registry_report_ms(const char* op_key, const char* symbol, double ms);

int sm_count();

}  // namespace b200
