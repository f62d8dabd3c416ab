/*
 * pyc_b200_abi.h -- binary layout of the PyC compiler-next types that cross the
 * backend seam.
 *
 * The B200 backend is a drop-in for the GPU half of PyC's compiler-next runtime,
 * so every struct here must have the exact size, field order and enum values of
 * the PyC public headers it stands in for:
 *
 *   pyc_dtype, pyc_shape, pyc_ir_op, pyc_ir_module   include/pyc/ir.h:12-53
 *   pyc_tensor                                       include/pyc/compiler_api.h:82-87
 *   pyc_backend, pyc_kernel_*_family, pyc_kernel_desc include/pyc/kernel_registry.h:16-51
 *   pyc_alloc_request, pyc_alloc_plan                include/pyc/runtime_allocator.h:14-36
 *   pyc_cuda_dispatch_trace, status codes            include/pyc/cuda_backend.h:28-55
 *   pyc_collective_comm, pyc_reduce_op, pyc_comm_status include/pyc/collective_comm.h:13-101
 *
 * When this header is compiled inside the PyC tree (the maintainer defines
 * PYC_B200_WITH_PYC_HEADERS), the PyC headers provide the types and this file
 * only checks their layout.  Stand-alone (this repository, ctypes users) the
 * types are declared here.  Either way the _Static_asserts at the bottom pin
 * the sizes the kernels and the dispatch code rely on.
 */
#ifndef PYC_B200_ABI_H
#define PYC_B200_ABI_H

#include <stddef.h>
#include <stdint.h>

#if defined(PYC_B200_WITH_PYC_HEADERS)

#include "pyc/compiler_api.h"
#include "pyc/cuda_backend.h"
#include "pyc/runtime_allocator.h"
#include "pyc/collective_comm.h"

#else /* stand-alone declarations */

#ifdef __cplusplus
extern "C" {
#endif

/* ---- IR (ir.h) --------------------------------------------------------- */
enum { PYC_IR_MAX_DIMS = 8, PYC_IR_MAX_OPS = 1024, PYC_IR_MAX_INPUTS = 8, PYC_IR_MAX_NAME = 64 };

typedef enum { PYC_DTYPE_UNKNOWN = 0, PYC_DTYPE_F32 = 1, PYC_DTYPE_F16 = 2, PYC_DTYPE_BF16 = 3,
               PYC_DTYPE_I32 = 4, PYC_DTYPE_I8 = 5 } pyc_dtype;

typedef struct { size_t rank; int64_t dims[PYC_IR_MAX_DIMS]; } pyc_shape;

typedef enum { PYC_IR_OP_INPUT = 0, PYC_IR_OP_CONST = 1, PYC_IR_OP_MATMUL = 2, PYC_IR_OP_ADD = 3,
               PYC_IR_OP_RELU = 4, PYC_IR_OP_GELU = 5, PYC_IR_OP_REDUCE_SUM = 6,
               PYC_IR_OP_LAYERNORM = 7, PYC_IR_OP_OUTPUT = 8 } pyc_ir_op_kind;

typedef struct {
    pyc_ir_op_kind kind;            /* @0   */
    char name[PYC_IR_MAX_NAME];     /* @4   */
    pyc_dtype dtype;                /* @68  */
    pyc_shape shape;                /* @72  */
    int input_ids[PYC_IR_MAX_INPUTS]; /* @144 */
    size_t input_count;             /* @176 */
} pyc_ir_op;                        /* 184 bytes */

typedef struct { pyc_ir_op ops[PYC_IR_MAX_OPS]; size_t op_count; } pyc_ir_module;

/* ---- run-time tensor descriptor (compiler_api.h) ------------------------ */
typedef struct { void* data; size_t size_bytes; pyc_dtype dtype; pyc_shape shape; } pyc_tensor;

/* ---- kernel registry (kernel_registry.h) -------------------------------- */
enum { PYC_KERNEL_MAX = 512, PYC_KERNEL_OP_KEY_MAX = 64, PYC_KERNEL_SYMBOL_MAX = 128 };

typedef enum { PYC_BACKEND_CPU = 0, PYC_BACKEND_CUDA = 1 } pyc_backend;
typedef enum { PYC_MODE_BALANCED = 0, PYC_MODE_MEMORY_FIRST = 1, PYC_MODE_UTILIZATION_FIRST = 2 } pyc_objective_mode;

typedef enum { PYC_KERNEL_WORKLOAD_ANY = 0, PYC_KERNEL_WORKLOAD_SMALL, PYC_KERNEL_WORKLOAD_SQUARE,
               PYC_KERNEL_WORKLOAD_LARGE_SQUARE, PYC_KERNEL_WORKLOAD_TALL_SKINNY,
               PYC_KERNEL_WORKLOAD_WIDE_SKINNY } pyc_kernel_workload_family;

typedef enum { PYC_KERNEL_HARDWARE_ANY = 0, PYC_KERNEL_HARDWARE_GENERIC, PYC_KERNEL_HARDWARE_ADA,
               PYC_KERNEL_HARDWARE_HOPPER } pyc_kernel_hardware_family;

typedef struct {
    char op_key[PYC_KERNEL_OP_KEY_MAX];
    pyc_backend backend;
    char symbol[PYC_KERNEL_SYMBOL_MAX];
    int priority;
    double estimated_occupancy;
    int tensor_core_eligible;
    size_t shared_mem_bytes;
    int reg_pressure_class;
    pyc_kernel_workload_family preferred_workload_family;
    pyc_kernel_hardware_family preferred_hardware_family;
} pyc_kernel_desc;                  /* 240 bytes */

/* selection trace and context of pyc_kernel_coselect_with_context (kernel_registry.h:53-76) */
typedef struct {
    double selected_score, selected_estimated_utilization, pressure_penalty, allocator_penalty, reuse_bonus;
    size_t candidates_considered;
} pyc_kernel_selection_trace;       /* 48 bytes */

typedef struct {
    double pressure_score;
    size_t pressure_events, rematerialized_tensors, reused_allocations, total_requested_bytes, peak_bytes, memory_budget_bytes;
    pyc_kernel_workload_family workload_family;
    pyc_kernel_hardware_family hardware_family;
} pyc_kernel_coselect_context;      /* 64 bytes */

/* ---- allocation plan (runtime_allocator.h) ------------------------------ */
enum { PYC_ALLOC_MAX_REQUESTS = 2048 };
typedef struct { int tensor_id; size_t size_bytes; size_t alignment; int start_step; int end_step; } pyc_alloc_request;
typedef struct {
    pyc_alloc_request requests[PYC_ALLOC_MAX_REQUESTS];
    size_t request_count;
    size_t offsets[PYC_ALLOC_MAX_REQUESTS];
    size_t peak_bytes, reused_allocations, allocation_events, overlap_pairs_observed;
    size_t largest_allocation_bytes, rematerialized_tensors, rematerialized_bytes, pressure_events;
    double pressure_score;
} pyc_alloc_plan;

/* ---- dispatch seam (cuda_backend.h) ------------------------------------- */
typedef enum { PYC_CUDA_DISPATCH_OK = 0, PYC_CUDA_DISPATCH_FALLBACK = 1, PYC_CUDA_DISPATCH_ERROR = 2 } pyc_cuda_dispatch_status;
enum { PYC_CUDA_REASON_MAX = 128 };

typedef struct {
    int cuda_requested, cuda_available, fallback_to_cpu, graph_replayed;
    double copy_in_ms, kernel_ms, copy_out_ms, sync_ms;
    char reason[PYC_CUDA_REASON_MAX];
} pyc_cuda_dispatch_trace;          /* 176 bytes */

typedef int (*pyc_cpu_executor_fn)(const pyc_ir_module* module, const pyc_tensor* inputs, size_t input_count,
                                   pyc_tensor* outputs, size_t output_count, void* executor_ctx);

/* ---- collective interface (collective_comm.h:13-101) --------------------- */
typedef enum { PYC_REDUCE_SUM = 0, PYC_REDUCE_PROD = 1, PYC_REDUCE_MIN = 2, PYC_REDUCE_MAX = 3, PYC_REDUCE_AVG = 4 } pyc_reduce_op;
typedef enum { PYC_COMM_OK = 0, PYC_COMM_ERR_TIMEOUT = 1, PYC_COMM_ERR_HARDWARE = 2, PYC_COMM_ERR_INVALID = 3 } pyc_comm_status;
typedef void* pyc_comm_handle_t;
typedef struct pyc_collective_comm {
    void* backend_ctx;
    pyc_comm_status (*all_reduce)(void* backend_ctx, pyc_comm_handle_t comm, const void* send_buf, void* recv_buf, size_t count,
                                  pyc_dtype dtype, pyc_reduce_op op, void* stream);
    pyc_comm_status (*all_gather)(void* backend_ctx, pyc_comm_handle_t comm, const void* send_buf, void* recv_buf, size_t count,
                                  pyc_dtype dtype, void* stream);
    pyc_comm_status (*reduce_scatter)(void* backend_ctx, pyc_comm_handle_t comm, const void* send_buf, void* recv_buf, size_t count,
                                      pyc_dtype dtype, pyc_reduce_op op, void* stream);
    pyc_comm_status (*broadcast)(void* backend_ctx, pyc_comm_handle_t comm, const void* send_buf, void* recv_buf, size_t count,
                                 pyc_dtype dtype, int root_rank, void* stream);
    pyc_comm_status (*send)(void* backend_ctx, pyc_comm_handle_t comm, const void* send_buf, size_t count, pyc_dtype dtype,
                            int peer_rank, void* stream);
    pyc_comm_status (*recv)(void* backend_ctx, pyc_comm_handle_t comm, void* recv_buf, size_t count, pyc_dtype dtype,
                            int peer_rank, void* stream);
    pyc_comm_status (*barrier)(void* backend_ctx, pyc_comm_handle_t comm, void* stream);
} pyc_collective_comm;              /* 64 bytes: context + seven entry points */

#ifdef __cplusplus
}
#endif

#endif /* PYC_B200_WITH_PYC_HEADERS */

#ifdef __cplusplus
#define PYC_B200_STATIC_ASSERT(c, m) static_assert(c, m)
#else
#define PYC_B200_STATIC_ASSERT(c, m) _Static_assert(c, m)
#endif

PYC_B200_STATIC_ASSERT(sizeof(pyc_shape) == 72, "pyc_shape layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_ir_op) == 184, "pyc_ir_op layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_ir_module) == 188424, "pyc_ir_module layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_tensor) == 96, "pyc_tensor layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_kernel_desc) == 240, "pyc_kernel_desc layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_cuda_dispatch_trace) == 176, "pyc_cuda_dispatch_trace layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_kernel_coselect_context) == 64, "pyc_kernel_coselect_context layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_kernel_selection_trace) == 48, "pyc_kernel_selection_trace layout");
PYC_B200_STATIC_ASSERT(sizeof(pyc_collective_comm) == 64, "pyc_collective_comm layout");
PYC_B200_STATIC_ASSERT(offsetof(pyc_ir_op, dtype) == 68 && offsetof(pyc_ir_op, input_ids) == 144, "pyc_ir_op offsets");

#endif /* PYC_B200_ABI_H */
