"""ctypes mirror of the PyC structs that cross the backend seam.

Field order and sizes follow include/pyc_b200_abi.h, which in turn restates
PyC's include/pyc/ir.h:12-53, compiler_api.h:82-87, kernel_registry.h:16-51 and
cuda_backend.h:28-55.  The size assertions at the bottom are the same ones the
C header makes.
"""
import ctypes as C

PYC_IR_MAX_DIMS = 8
PYC_IR_MAX_OPS = 1024
PYC_IR_MAX_INPUTS = 8
PYC_IR_MAX_NAME = 64
PYC_KERNEL_OP_KEY_MAX = 64
PYC_KERNEL_SYMBOL_MAX = 128
PYC_CUDA_REASON_MAX = 128

# pyc_dtype
DTYPE_UNKNOWN, DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_I32, DTYPE_I8 = range(6)
DTYPE_SIZE = {DTYPE_F32: 4, DTYPE_F16: 2, DTYPE_BF16: 2, DTYPE_I32: 4, DTYPE_I8: 1}
DTYPE_NAME = {DTYPE_F32: "f32", DTYPE_F16: "f16", DTYPE_BF16: "bf16", DTYPE_I32: "i32", DTYPE_I8: "i8"}

# pyc_ir_op_kind
(OP_INPUT, OP_CONST, OP_MATMUL, OP_ADD, OP_RELU, OP_GELU, OP_REDUCE_SUM, OP_LAYERNORM, OP_OUTPUT) = range(9)

# pyc_backend / dispatch status
BACKEND_CPU, BACKEND_CUDA = 0, 1
DISPATCH_OK, DISPATCH_FALLBACK, DISPATCH_ERROR = 0, 1, 2

# pyc_b200 extension enums
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2
ADD_NONE, ADD_MATRIX, ADD_ROW_BIAS, ADD_SCALAR = 0, 1, 2, 3


class Shape(C.Structure):
    _fields_ = [("rank", C.c_size_t), ("dims", C.c_int64 * PYC_IR_MAX_DIMS)]

    @classmethod
    def of(cls, dims):
        s = cls()
        s.rank = len(dims)
        for i, d in enumerate(dims):
            s.dims[i] = int(d)
        return s

    def tolist(self):
        return [int(self.dims[i]) for i in range(self.rank)]


class IrOp(C.Structure):
    _fields_ = [("kind", C.c_int), ("name", C.c_char * PYC_IR_MAX_NAME), ("dtype", C.c_int),
                ("shape", Shape), ("input_ids", C.c_int * PYC_IR_MAX_INPUTS), ("input_count", C.c_size_t)]


class IrModule(C.Structure):
    _fields_ = [("ops", IrOp * PYC_IR_MAX_OPS), ("op_count", C.c_size_t)]


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("size_bytes", C.c_size_t), ("dtype", C.c_int), ("shape", Shape)]


class KernelDesc(C.Structure):
    _fields_ = [("op_key", C.c_char * PYC_KERNEL_OP_KEY_MAX), ("backend", C.c_int),
                ("symbol", C.c_char * PYC_KERNEL_SYMBOL_MAX), ("priority", C.c_int),
                ("estimated_occupancy", C.c_double), ("tensor_core_eligible", C.c_int),
                ("shared_mem_bytes", C.c_size_t), ("reg_pressure_class", C.c_int),
                ("preferred_workload_family", C.c_int), ("preferred_hardware_family", C.c_int)]


class DispatchTrace(C.Structure):
    _fields_ = [("cuda_requested", C.c_int), ("cuda_available", C.c_int), ("fallback_to_cpu", C.c_int),
                ("graph_replayed", C.c_int), ("copy_in_ms", C.c_double), ("kernel_ms", C.c_double),
                ("copy_out_ms", C.c_double), ("sync_ms", C.c_double), ("reason", C.c_char * PYC_CUDA_REASON_MAX)]


CPU_EXECUTOR_FN = C.CFUNCTYPE(C.c_int, C.POINTER(IrModule), C.POINTER(Tensor), C.c_size_t,
                              C.POINTER(Tensor), C.c_size_t, C.c_void_p)


class GemmArgs(C.Structure):
    _fields_ = [("symbol", C.c_char_p), ("dtype", C.c_int), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int),
                ("A", C.c_void_p), ("B", C.c_void_p), ("D", C.c_void_p), ("b_col_major", C.c_int),
                ("alpha", C.c_float), ("add_mode", C.c_int), ("add", C.c_void_p), ("act", C.c_int)]


class FfnArgs(C.Structure):
    _fields_ = [("tokens", C.c_int), ("hidden", C.c_int), ("inner", C.c_int), ("x", C.c_void_p), ("ln_gamma", C.c_void_p),
                ("ln_beta", C.c_void_p), ("eps", C.c_float), ("w1", C.c_void_p), ("w1_scale", C.c_void_p), ("b1", C.c_void_p),
                ("w2", C.c_void_p), ("w2_scale", C.c_void_p), ("b2", C.c_void_p), ("out", C.c_void_p)]


class RuntimeInfo(C.Structure):
    _fields_ = [("arena_bytes", C.c_size_t), ("plan_peak_bytes", C.c_size_t), ("plan_total_bytes", C.c_size_t),
                ("graphs_cached", C.c_size_t), ("graph_replays", C.c_size_t), ("kernels_per_graph", C.c_size_t),
                ("kernel_launches_total", C.c_size_t)]


assert C.sizeof(Shape) == 72
assert C.sizeof(IrOp) == 184
assert C.sizeof(IrModule) == 188424
assert C.sizeof(Tensor) == 96
assert C.sizeof(KernelDesc) == 240
assert C.sizeof(DispatchTrace) == 176
