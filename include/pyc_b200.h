/*
 * pyc_b200.h -- C-ABI of the B200-native execution backend for PyC's
 * compiler-next runtime (libpyc_b200.so).
 *
 * Part 1 declares the eight symbols that PyC's own GPU half exports
 * (src/compiler/runtime/cuda_backend.c + src/compiler/cutlass_kernels/) with
 * identical names, argument meaning and return conventions, so that PyC's
 * compiler_api.c, its Rust FFI (src/runtime/vortex_core/src/ffi/mod.rs:161-186)
 * and its Python ctypes layer (python/pyc/compiler/__init__.py:187-190) bind to
 * this library without change.
 *
 * Part 2 is additive: entry points for work PyC's IR cannot express (batched
 * attention, conv2d with a bias/ReLU epilogue, fp8-weight FFN block) and for
 * GPU-aware callers (caller-owned stream, measured autotune).  Nothing in part
 * 2 changes the meaning of part 1.
 *
 * All pointers named "device" must be CUDA device (or managed) addresses on the
 * current device.  All functions are thread-safe per device; work on one device
 * is serialised behind that device's context lock.
 */
#ifndef PYC_B200_H
#define PYC_B200_H

#include "pyc_b200_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ======================================================================= *
 * Part 1 -- drop-in symbols                                                *
 * ======================================================================= */

/* Replaces pyc_cuda_dispatch_trace_init (include/pyc/cuda_backend.h:61,
 * src/compiler/runtime/cuda_backend.c:235-247): zero the trace, reason = "". */
void pyc_cuda_dispatch_trace_init(pyc_cuda_dispatch_trace* trace);

/* Replaces pyc_cuda_current_hardware_family (cuda_backend.h:62,
 * cuda_backend.c:249-301).  The PyC enum has no Blackwell member; as in PyC,
 * compute capability >= 9 reports PYC_KERNEL_HARDWARE_HOPPER, so a B200 gets
 * the "hopper" scoring affinity.  PYC_CUDA_FORCE_HARDWARE_FAMILY=
 * hopper|ada|generic overrides.  No device => GENERIC. */
pyc_kernel_hardware_family pyc_cuda_current_hardware_family(void);

/* Replaces pyc_cuda_dispatch (cuda_backend.h:87-96, cuda_backend.c:2808-2928):
 * run one compiled IR module.  inputs[]/outputs[] follow the module's
 * INPUT/OUTPUT op order.  Each pyc_tensor.data may be a host pointer (staged
 * through pinned memory, as PyC does) or a device pointer (zero copy).
 * Supported op kinds: INPUT, MATMUL, ADD (same shape, row bias [N], scalar [1]),
 * RELU, GELU (erf), REDUCE_SUM (trailing axis), LAYERNORM (last axis, eps 1e-5,
 * optional gamma/beta as input_ids[1..2]), OUTPUT; dtypes F32, BF16, F16.
 * The op sequence is fused (matmul+bias+activation), placed in one device
 * arena by lifetime, captured once as a CUDA graph and replayed afterwards.
 * Returns OK (ran on the GPU), FALLBACK (cpu_executor ran: no device, an env
 * switch, or an op kind the GPU path does not know) or ERROR (NULL argument,
 * PYC_CUDA_FORCE_ERROR, a CUDA failure, or the fallback failed too).
 * Env switches honoured: PYC_CUDA_DISABLE, PYC_CUDA_FORCE_ERROR,
 * PYC_CUDA_FORCE_FALLBACK, PYC_CUDA_SIMULATE_AVAILABLE,
 * PYC_CUDA_ENABLE_GRAPH_REPLAY, PYC_CUDA_ASSUME_STATIC_LHS/RHS,
 * PYC_CUDA_SKIP_HOST_OUTPUT_COPY.  trace->reason is always NUL-terminated. */
pyc_cuda_dispatch_status pyc_cuda_dispatch(
    const pyc_ir_module* module, const pyc_tensor* inputs, size_t input_count,
    pyc_tensor* outputs, size_t output_count,
    pyc_cpu_executor_fn cpu_executor, void* executor_ctx, pyc_cuda_dispatch_trace* trace);

/* Replaces pyc_cutlass_gemm_dispatch (cuda_backend.h:105-114,
 * cutlass_kernels/gemm/kernel.cu:151-203): C[M,N] = alpha*A[M,K]*B + beta*C on
 * device pointers, row-major, leading dimensions K / N / N, enqueued on
 * `stream` (cudaStream_t) without synchronising.  `symbol` picks dtype and
 * tile configuration; PyC's four legacy names are accepted as aliases
 * (cutlass_gemm_tensorcore_bf16: B row-major [K,N]; cutlass_gemm_tensorcore_f16:
 * B column-major as in kernel.cu:161-174; cutlass_gemm_simt_f32 and
 * ada_gemm_k64_warp32_async_f32: fp32).  Returns 0, or -1 for an unknown symbol,
 * a bad shape or a launch failure. */
int pyc_cutlass_gemm_dispatch(const char* symbol, int M, int N, int K,
                              const void* A, const void* B, void* C,
                              float alpha, float beta, void* stream);

/* Replaces pyc_cutlass_conv2d_dispatch (cuda_backend.h:116-126,
 * cutlass_kernels/conv2d/kernel.cu:80-111): NHWC forward convolution, filter
 * KRSC, cross-correlation, dilation 1, groups 1, output [N,P,Q,K] with
 * P=(H-R+2*pad_h)/stride_h+1.  Symbols: b200_conv2d_fprop_bf16 /
 * b200_conv2d_fprop_f16 and PyC's cutlass_conv2d_fprop_{f16,bf16}. */
int pyc_cutlass_conv2d_dispatch(const char* symbol, int N, int H, int W, int C_in,
                                int K, int R, int S, int pad_h, int pad_w,
                                int stride_h, int stride_w,
                                const void* input, const void* filter, void* output, void* stream);

/* Replaces pyc_cutlass_attention_dispatch (cuda_backend.h:128-138,
 * cutlass_kernels/attention/kernel.cu:95-122): one head,
 * Out[seq_len,d_head] = softmax(scale * Q K^T) V, as the header comment at
 * attention/kernel.cu:6-8 defines it (PyC's own kernel body is an identity
 * copy).  Symbols: b200_attention_bf16, b200_attention_bf16_causal,
 * b200_attention_f16[_causal], and PyC's cutlass_attention_{f16,bf16}
 * (non-causal). */
int pyc_cutlass_attention_dispatch(const char* symbol, int seq_len, int d_head,
                                   const void* Q, const void* K, const void* V, void* Out,
                                   float scale, void* stream);

/* Replaces pyc_cutlass_kernel_count (cuda_backend.h:143, registry/init.cu:88-91):
 * number of CUDA kernels registered under op_key ("matmul", "conv2d",
 * "attention"). */
int pyc_cutlass_kernel_count(const char* op_key);

/* Replaces pyc_cutlass_registry_init (registry/init.cu:32-78): register every
 * kernel of this library in PyC's kernel registry (when PyC's
 * kernel_registry.c is linked in the same process) and in the library's own
 * symbol table; honours PYC_PROMOTED_GEMM_SYMBOL.  Idempotent. */
void pyc_cutlass_registry_init(void);

/* ======================================================================= *
 * Part 2 -- additive entry points (no counterpart in PyC)                  *
 * ======================================================================= */

typedef enum { PYC_B200_ACT_NONE = 0, PYC_B200_ACT_RELU = 1, PYC_B200_ACT_GELU = 2 } pyc_b200_activation;
typedef enum { PYC_B200_ADD_NONE = 0, PYC_B200_ADD_MATRIX = 1, PYC_B200_ADD_ROW_BIAS = 2, PYC_B200_ADD_SCALAR = 3 } pyc_b200_add_mode;

/* Fused GEMM: D = act(alpha * A*B + add), device pointers, row-major.
 * dtype is the storage type of A, B, add and D (F32, BF16 or F16); the
 * accumulator is fp32.  b_col_major != 0 means B is stored [N,K].
 * symbol may be NULL (the registry's current choice for dtype/shape). */
typedef struct {
    const char* symbol;
    pyc_dtype dtype;
    int M, N, K;
    const void* A;
    const void* B;
    void* D;
    int b_col_major;
    float alpha;
    pyc_b200_add_mode add_mode;
    const void* add;              /* [M,N], [N] or [1] of dtype */
    pyc_b200_activation act;
} pyc_b200_gemm_args;
int pyc_b200_gemm(const pyc_b200_gemm_args* args, void* stream);

/* No counterpart in PyC.  The same tensor-core GEMM (bf16 / f16 only) for callers
 * that cannot allocate device memory when they need it: hosts that have given
 * all of HBM to their own pool, threads that must not trigger the device-wide
 * synchronisation of an allocation, code that runs while a capture is open.
 * It creates no context, stream or buffer and calls no allocator; the kernel's
 * only scratch (its status block) is a 256-byte array compiled into the library
 * and resident on every GPU that loads it.  Limits: M, N, K <= 1048576 each,
 * K % 8 == 0, N % 8 == 0 for row-major B, A and B 16-byte aligned; anything
 * else returns -1 with a message in pyc_b200_last_error().  The first call on a
 * device does one-time set-up (address of the array, kernel attributes): make it
 * before any stream capture.  All calls share the array and clear it on
 * `stream` before launching, so calls whose kernels overlap on the GPU race on
 * it: issue them on one stream or order them with events.  args->symbol is
 * ignored (the tile width is chosen from the shape). */
int pyc_b200_gemm_static(const pyc_b200_gemm_args* args, void* stream);

/* No counterpart in PyC.  Status of the static entry point's kernels, also without
 * any allocation: enqueues one 4-byte copy of the shared block's status word into
 * *host_out on `stream` (use pinned memory for a truly asynchronous copy) and
 * returns; after the caller has synchronised that stream, *host_out is 0 when every
 * wait of the preceding pyc_b200_gemm_static kernels completed, otherwise
 * (site << 8) | 1 for the first wait that ran out -- the output of that GEMM is then
 * not valid.  The word is cleared by the next pyc_b200_gemm_static call, so read it
 * before issuing another one.  pyc_b200_device_status() does NOT see this word (it
 * reads the per-device context that the allocating entry points create).  Before
 * the first static call on a device *host_out is set to 0 directly. */
int pyc_b200_gemm_static_status(int* host_out, void* stream);

/* Elementwise / reduction ops on device pointers (HBM-bound kernels). */
int pyc_b200_add(pyc_dtype dtype, const void* a, const void* b, void* out, size_t elems, void* stream);
int pyc_b200_bias_act(pyc_dtype dtype, const void* x, const void* add, pyc_b200_add_mode add_mode,
                      pyc_b200_activation act, void* out, size_t rows, size_t cols, void* stream);
int pyc_b200_layernorm(pyc_dtype dtype, const void* x, const void* gamma, const void* beta,
                       void* out, size_t rows, size_t cols, float eps, void* stream);
int pyc_b200_softmax(pyc_dtype dtype, const void* x, void* out, size_t rows, size_t cols, void* stream);
int pyc_b200_reduce_sum(pyc_dtype dtype, const void* x, void* out, size_t rows, size_t cols, void* stream);

/* Batched attention: Q,K,V,Out are [batch_heads, seq_len, d_head] contiguous. */
int pyc_b200_attention(pyc_dtype dtype, int batch_heads, int seq_len, int d_head,
                       const void* Q, const void* K, const void* V, void* Out,
                       float scale, int causal, void* stream);

/* conv2d forward with fused bias[K] (may be NULL) and optional ReLU. */
int pyc_b200_conv2d(pyc_dtype dtype, int N, int H, int W, int C_in, int K, int R, int S,
                    int pad_h, int pad_w, int stride_h, int stride_w,
                    const void* input, const void* filter, const void* bias, int relu,
                    void* output, void* stream);

/* ---- fp8 (e4m3) weight path: the transformer-FFN configuration ------------ *
 * No counterpart in PyC (its dtype enum has no fp8).                          */

/* Per-token quantisation of bf16 rows: q = round_e4m3(x / scale), scale[row] = amax(row) / 448
 * (cols % 8 == 0, cols <= 16384).  The second form applies LayerNorm (last axis, eps, optional
 * gamma/beta [cols] bf16) first, in the same pass over the row. */
int pyc_b200_quantize_rows(const void* x_bf16, void* q_e4m3, float* row_scale, size_t rows, size_t cols, void* stream);
int pyc_b200_layernorm_quantize(const void* x_bf16, const void* gamma, const void* beta, void* q_e4m3, float* row_scale,
                                size_t rows, size_t cols, float eps, void* stream);

/* D[M,N] (bf16) = act(acc * row_scale[m] * col_scale[n] + bias[n]); A [M,K] e4m3, B [K,N] e4m3 row-major
 * (or [N,K] when b_col_major); scales and bias may be NULL.  K % 16 == 0, N % 16 == 0. */
int pyc_b200_gemm_fp8(int M, int N, int K, const void* A_e4m3, const void* B_e4m3, int b_col_major, const float* row_scale,
                      const float* col_scale, const void* bias_bf16, pyc_b200_activation act, void* D_bf16, void* stream);

/* One FFN block: out = W2^T-form( GELU( LN(x) * W1 + b1 ) ) * ... i.e.
 *   out[T,H] = (gelu(layernorm(x)[T,H] . W1[H,I] + b1[I]) . W2[I,H]) + b2[H]
 * x, out, biases bf16; W1, W2 e4m3 row-major with one fp32 scale per OUTPUT channel (w1_scale[I], w2_scale[H]);
 * activations are quantised per token to e4m3 in front of each GEMM, both GEMMs run on the fp8 tensor-core path.
 * Tensor parallel use: give each rank its column slice of W1 / b1 / w1_scale and row slice of W2 (inner = I / ranks),
 * b2 on one rank only; `out` is then a partial sum to be all-reduced by the caller.
 * The caller provides the scratch: pyc_b200_ffn_workspace_bytes(tokens, hidden, inner) bytes, 256-byte aligned. */
typedef struct {
    int tokens, hidden, inner;
    const void* x;
    const void* ln_gamma;   /* may be NULL */
    const void* ln_beta;    /* may be NULL */
    float eps;              /* <= 0: 1e-5 */
    const void* w1; const float* w1_scale; const void* b1;   /* b1 may be NULL */
    const void* w2; const float* w2_scale; const void* b2;   /* b2 may be NULL */
    void* out;
} pyc_b200_ffn_args;
size_t pyc_b200_ffn_workspace_bytes(int tokens, int hidden, int inner);
int pyc_b200_ffn_block(const pyc_b200_ffn_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* Per-phase timing of the FFN block for profiling callers: events5 points to five cudaEvent_t (created by the caller with
 * timing enabled) that every following pyc_b200_ffn_block / _tp / _scatter call OF THIS THREAD records on its stream: [0]
 * at the start, [1] after LayerNorm+quantise, [2] after the first GEMM (+GELU), [3] after the re-quantise, [4] after the
 * second GEMM.  NULL switches it off again.  Nothing is allocated or synchronised. */
int pyc_b200_ffn_phase_events(void* const* events5);

/* Tensor-parallel FFN through PyC's collective interface.  Each rank calls this with its shard (as described above:
 * column slice of W1 / b1 / w1_scale, row slice of W2, b2 on one rank) and the vtable of a loaded collective backend
 * (pyc_collective_comm, include/pyc/collective_comm.h:30-101; PyC's loader is pyc_load_comm_backend,
 * src/compiler/runtime/comm_backend_loader.c) plus the communicator handle its launcher created (PyC hands it around as
 * "comm_handle", src/compiler/runtime/distributed_runtime.c:16-42).  The block runs, then ONE all_reduce (sum) of the
 * [tokens, hidden] partial sums is issued through comm->all_reduce with PYC_DTYPE_BF16, in place on args->out, on `stream`.
 * PyC's own NCCL shim has no bf16 mapping (src/compiler/runtime/comm_backend_nccl.c:139-150 knows I8/I32/F16/F32);
 * libpyc_b200_comm_nccl.so in this package is a backend for the same interface that has it.  world == 1 needs no vtable.
 * Returns 0, or -1 (message in pyc_b200_last_error()) for bad arguments or a collective status other than PYC_COMM_OK.
 * PyC's own pyc_run_model never calls a collective (its options only carry world_size / rank). */
int pyc_b200_ffn_block_tp(const pyc_b200_ffn_args* args, const pyc_collective_comm* comm, pyc_comm_handle_t comm_handle,
                          int world, int rank, void* workspace, size_t workspace_bytes, void* stream);

/* Tensor-parallel FFN without a library collective: the reduce-scatter is done by the second GEMM's epilogue and the
 * all-gather by the reduction kernel, both with plain stores into peer memory over NVLink.
 *   - every rank owns tokens / world consecutive rows of the result and a receive buffer [world][tokens/world][hidden]
 *     bf16 that the other ranks can write (pyc_b200_symm_alloc + pyc_b200_symm_open, or any peer-mapped memory);
 *   - pyc_b200_ffn_block_scatter is pyc_b200_ffn_block whose last GEMM stores row r of this rank's partial sum into slot
 *     `rank` of the receive buffer of the rank that owns r (recv_slots[owner]); args->out is not written and may be NULL;
 *   - after ALL ranks have finished that call (a barrier of the caller: an NCCL barrier on the stream, for instance),
 *     pyc_b200_tp_reduce_broadcast adds the world slots of the local receive buffer in fp32 and stores the owned rows,
 *     rounded to bf16, into the [tokens][hidden] output of every rank (outs[0..world-1]); after a second barrier every
 *     rank holds the full result.
 * No kernel waits on another GPU; ordering between ranks is the caller's two barriers.  world <= PYC_B200_TP_MAX_RANKS.
 * PyC has no counterpart: its options carry world_size/rank (include/pyc/compiler_api.h:53-62) but pyc_run_model never
 * exchanges data between ranks. */
#define PYC_B200_TP_MAX_RANKS 8
int pyc_b200_ffn_block_scatter(const pyc_b200_ffn_args* args, void* workspace, size_t workspace_bytes, void* const* recv_slots,
                               int world, int rank, void* stream);
int pyc_b200_tp_reduce_broadcast(const void* recv_local, void* const* outs, int world, int rank, int rows_per_rank, int hidden,
                                 void* stream);
/* All-reduce (sum) of a [rows][hidden] bf16 tensor inside the NVSwitch, for the tensor-parallel FFN's partial sums: the
 * third way to do the exchange that pyc_b200_ffn_block_tp does through comm->all_reduce (include/pyc/collective_comm.h:49-58).
 * Every rank's copy of the tensor sits at the same offset of a buffer bound to ONE NVLink multicast object (cuMulticast*;
 * torch.distributed._symmetric_memory does the allocation and hands out the address) and `multicast_ptr` is the multicast
 * address of the tensor.  Each rank reduces 1/world of the 16-byte pieces with multimem.ld_reduce (fp32 accumulation in
 * the switch, one rounding) and broadcasts them with multimem.st; in place, on `stream`, one kernel of
 * PYC_B200_TP_MULTIMEM_BLOCKS blocks that must be co-resident (nothing else may hold the GPU's SMs for long).
 *   flag_ptrs[r]   : rank r's flag words, PYC_B200_TP_MULTIMEM_BLOCKS * PYC_B200_TP_MAX_RANKS uint32, zeroed once before the
 *                    first call, writable from every rank (own pointer at [rank], peer mappings elsewhere);
 *   epoch_counters : PYC_B200_TP_MULTIMEM_BLOCKS uint32 in local device memory, zeroed once; the kernel advances them, so the
 *                    call can be captured in a CUDA graph and replayed.
 * Every rank must make the same sequence of calls.  The two cross-GPU rendezvous inside the kernel are bounded waits
 * (~2 s); one that runs out shows as ((40 | 41) << 8) | 1 in pyc_b200_device_status().  The producer of the partial sums
 * must be earlier work on the same stream.  PyC has no counterpart (its NCCL shim calls ncclAllReduce). */
#define PYC_B200_TP_MULTIMEM_BLOCKS 128
int pyc_b200_tp_allreduce_multimem(void* multicast_ptr, void* const* flag_ptrs, void* epoch_counters, int world, int rank,
                                   size_t rows, size_t hidden, void* stream);
/* The tensor-parallel FFN block with the all-reduce fused into its last GEMM: the fourth form of the exchange, and the one
 * where the transfer overlaps the GEMM tile by tile.  args->out must be this rank's copy of a [tokens][hidden] bf16 buffer
 * bound to an NVLink multicast object and `multicast_out` that buffer's multicast address (as for
 * pyc_b200_tp_allreduce_multimem).  In the last GEMM (CTA-pair kernel) a publisher warp per CTA announces every 128 x 256
 * part of the partial sum once it is stored (one system-scope fence, one epoch word per rank) and a reducer warp, walking
 * the same tile order, reduces this rank's 128 / world rows of each part in the switch (multimem.ld_reduce, fp32
 * accumulation, one rounding) and writes the sums into every rank's copy (multimem.st) while the tensor cores work on the
 * following tiles; when the call's kernels have finished on a rank, its `out` holds the all-reduced result.  No
 * communicator, no caller barrier.
 *   flag_ptrs[r] : rank r's flag words, (tokens/256) * (hidden/256) * 2 * PYC_B200_TP_MAX_RANKS uint32, zeroed once, writable
 *                  from every rank;   fin_ptrs[r] : likewise, PYC_B200_TP_FUSED_EPOCH_SLOTS * PYC_B200_TP_MAX_RANKS uint32;
 *   epoch_counters : PYC_B200_TP_FUSED_EPOCH_SLOTS uint32 of local memory, zeroed once (the kernel advances them: the call
 *                  can be captured in a CUDA graph and replayed).
 * tokens and hidden multiples of 256, world 2, 4 or 8, every rank makes the same sequence of calls, and one set of flag /
 * counter buffers serves ONE problem shape (the epochs are per CTA, the flags per tile).  Waits are bounded
 * (~2 s; sites 0x39-0x3c in pyc_b200_device_status()).  PyC has no counterpart. */
#define PYC_B200_TP_FUSED_EPOCH_SLOTS 256
int pyc_b200_ffn_block_switch_reduce(const pyc_b200_ffn_args* args, void* workspace, size_t workspace_bytes, void* multicast_out,
                                     void* const* flag_ptrs, void* const* fin_ptrs, void* epoch_counters, int world, int rank,
                                     void* stream);
/* Device memory that other processes on the same node can map: allocate + export a 64-byte handle, open a peer's handle,
 * close it again, free the own allocation.  (cudaMalloc + CUDA IPC; the handle is sent by whatever channel the caller has.) */
int pyc_b200_symm_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
int pyc_b200_symm_open(const unsigned char handle[64], void** ptr);
int pyc_b200_symm_close(void* ptr);
int pyc_b200_symm_free(void* ptr);

/* Time every registered tile configuration for (dtype, M, N, K) with CUDA
 * events, feed the measured milliseconds to PyC's registry
 * (pyc_kernel_benchmark_update_symbol) when it is linked, remember the winner
 * for later NULL-symbol calls, and write its name to best_symbol.
 * Returns the number of configurations timed, or -1. */
int pyc_b200_autotune_gemm(pyc_dtype dtype, int M, int N, int K, int iters,
                           char* best_symbol, size_t best_symbol_size, double* best_ms);

/* Persisted autotune results, in the line format of PyC's autotune DB ("op|backend|symbol|best_ms",
 * src/compiler/compiler_api.c:2145-2305, path rule :2124-2143: PYC_AUTOTUNE_DB_PATH).  pyc_b200_autotune_gemm and the
 * PYC_B200_AUTOTUNE=1 dispatch path append every timing under flock("<path>.lock") and compact the file as PyC does.
 * Lines with op "matmul" are the per-symbol timings PyC's own loader reads; lines with op "matmul@<dtype>:<M>x<N>x<K>"
 * carry the same timings per shape, and the fastest symbol of a shape becomes that shape's choice in the next process.
 * The DB is read once when the library registers its kernels; this call reads `path` (NULL: PYC_AUTOTUNE_DB_PATH) again.
 * Returns the number of per-shape winners installed, 0 when the file does not exist, -1 without a path. */
int pyc_b200_autotune_db_load(const char* path);

/* The plan of the most recent GPU run of `module` in this process (NULL: of the most recent run of any module): one text
 * line per step, "step <i>: <kernel symbol> [<who chose it>] <- <op>#<id> + <op>#<id> ...", naming the IR ops each kernel
 * absorbed.  PyC's own fusion pass renames ops and drops the epilogue (src/compiler/passes/pass_manager.c:241-267) and its
 * "matmul_fused" catalog holds placeholders (src/compiler/compiler_api.c:2094-2122), so
 * pyc_run_stats.selected_kernel_symbol cannot name the kernel that ran; this does, without touching a PyC header.
 * "who chose it" is autotune | env | promoted | registry | model (see pyc_cuda_dispatch's selection order in runtime.cu).
 * Returns the length of the full text (copy truncated to out_size - 1), or -1 if that module has not run. */
int pyc_b200_last_plan(const pyc_ir_module* module, char* out, size_t out_size);

/* The device-arena plan pyc_cuda_dispatch would use for this module and these tensor descriptors, without running
 * anything (host-only; works without a GPU): one pyc_alloc_request per arena-resident tensor -- tensor_id = IR op id,
 * size, alignment 1024, start/end = first and last step that touches it -- in placement order, the offset each got, and
 * the peak.  The placement is the first-fit reuse rule of PyC's planner (src/compiler/runtime/runtime_allocator.c:123-187):
 * feeding the same requests to pyc_alloc_plan_build_with_mode gives the same offsets and peak.  tensors_on_device != 0
 * plans as if every tensor were a device pointer (no staging copies), 0 as if all were host memory.
 * Writes at most `capacity` entries, *count_out = number of arena tensors.  Returns 0 / -1. */
int pyc_b200_plan_arena(const pyc_ir_module* module, const pyc_tensor* inputs, size_t input_count,
                        pyc_tensor* outputs, size_t output_count, int tensors_on_device,
                        pyc_alloc_request* requests_out, size_t* offsets_out, size_t capacity,
                        size_t* count_out, size_t* peak_bytes_out);

/* Device arena / graph cache telemetry for the last pyc_cuda_dispatch on the
 * current device. */
typedef struct {
    size_t arena_bytes;           /* size of the device arena */
    size_t plan_peak_bytes;       /* peak of the lifetime plan */
    size_t plan_total_bytes;      /* sum of all intermediate tensors */
    size_t graphs_cached;
    size_t graph_replays;
    size_t kernels_per_graph;
    size_t kernel_launches_total; /* kernels this library has launched so far */
} pyc_b200_runtime_info;
int pyc_b200_get_runtime_info(pyc_b200_runtime_info* out);

/* GPU-aware callers: make pyc_cuda_dispatch enqueue on `stream` and, when
 * async != 0 and every tensor is a device pointer, return without
 * synchronising.  Pass NULL/0 to restore the default (private stream, sync). */
int pyc_b200_set_stream(void* stream, int async);

/* Kernels never spin without a limit: a wait that runs out writes a code to a
 * per-device status word and the kernel returns.  This reads that word
 * (synchronising the library's stream): 0 = fine, otherwise
 * (site << 8) | 1, or -1 if no device. */
int pyc_b200_device_status(void);

/* Self-test of the bounded waits: enqueue on `stream` a one-CTA kernel that waits, for at most about limit_us
 * microseconds (1 .. 1000000), on a barrier nobody arrives at.  The wait runs out by itself, the kernel records
 * (0x7f << 8) | 1 in the device status word and returns; pyc_b200_device_status() then reports that value once, and a
 * pyc_cuda_dispatch that runs before the word has been read returns PYC_CUDA_DISPATCH_ERROR with the reason
 * "b200_kernel_wait_timeout:0x7f01".  Nothing hangs, traps or faults.  Returns 0 / -1. */
int pyc_b200_selftest_wait_timeout(int limit_us, void* stream);

/* Last error text of the calling thread ("" when none). */
const char* pyc_b200_last_error(void);

/* Free every device allocation, graph and stream the library owns on the
 * current device. */
void pyc_b200_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* PYC_B200_H */
