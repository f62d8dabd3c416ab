"""ctypes binding of libpyc_b200.so: the calls a PyC host makes at the backend seam.

`dispatch()` is pyc_cuda_dispatch (include/pyc/cuda_backend.h:87-96 in PyC);
`gemm_by_symbol()` is pyc_cutlass_gemm_dispatch (cuda_backend.h:105-114); the
rest are the additive pyc_b200_* entry points.  There is no CPU path here: if
the library is missing, or a call does not run on the GPU, these raise.
"""
import ctypes as C
import os

from . import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpyc_b200.so")

EXPORTS = [
    # drop-in symbols (PyC names)
    "pyc_cuda_dispatch_trace_init", "pyc_cuda_current_hardware_family", "pyc_cuda_dispatch",
    "pyc_cutlass_gemm_dispatch", "pyc_cutlass_conv2d_dispatch", "pyc_cutlass_attention_dispatch",
    "pyc_cutlass_kernel_count", "pyc_cutlass_registry_init",
    # additive
    "pyc_b200_gemm", "pyc_b200_gemm_static", "pyc_b200_gemm_static_status", "pyc_b200_add", "pyc_b200_bias_act", "pyc_b200_layernorm", "pyc_b200_softmax",
    "pyc_b200_reduce_sum", "pyc_b200_quantize_rows", "pyc_b200_layernorm_quantize", "pyc_b200_gemm_fp8",
    "pyc_b200_ffn_workspace_bytes", "pyc_b200_ffn_block", "pyc_b200_ffn_block_tp", "pyc_b200_ffn_phase_events", "pyc_b200_ffn_block_scatter", "pyc_b200_tp_reduce_broadcast", "pyc_b200_tp_allreduce_multimem", "pyc_b200_ffn_block_switch_reduce",
    "pyc_b200_symm_alloc", "pyc_b200_symm_open", "pyc_b200_symm_close", "pyc_b200_symm_free", "pyc_b200_attention", "pyc_b200_conv2d", "pyc_b200_autotune_gemm", "pyc_b200_autotune_db_load", "pyc_b200_last_plan", "pyc_b200_plan_arena",
    "pyc_b200_get_runtime_info", "pyc_b200_set_stream", "pyc_b200_device_status", "pyc_b200_selftest_wait_timeout", "pyc_b200_last_error",
    "pyc_b200_shutdown",
]

_lib = None


class BackendError(RuntimeError):
    pass


def load():
    """Load the CUDA library; fail loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BackendError(f"{LIB_PATH} is missing: run `python -m pyc_b200.build` (needs nvcc); there is no CPU fallback")
    L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    vp, i, sz, f = C.c_void_p, C.c_int, C.c_size_t, C.c_float
    L.pyc_cuda_dispatch_trace_init.argtypes = [C.POINTER(abi.DispatchTrace)]
    L.pyc_cuda_dispatch_trace_init.restype = None
    L.pyc_cuda_current_hardware_family.restype = i
    L.pyc_cuda_dispatch.argtypes = [C.POINTER(abi.IrModule), C.POINTER(abi.Tensor), sz, C.POINTER(abi.Tensor), sz,
                                    abi.CPU_EXECUTOR_FN, vp, C.POINTER(abi.DispatchTrace)]
    L.pyc_cuda_dispatch.restype = i
    L.pyc_cutlass_gemm_dispatch.argtypes = [C.c_char_p, i, i, i, vp, vp, vp, f, f, vp]
    L.pyc_cutlass_conv2d_dispatch.argtypes = [C.c_char_p] + [i] * 11 + [vp, vp, vp, vp]
    L.pyc_cutlass_attention_dispatch.argtypes = [C.c_char_p, i, i, vp, vp, vp, vp, f, vp]
    L.pyc_cutlass_kernel_count.argtypes = [C.c_char_p]
    L.pyc_cutlass_registry_init.restype = None
    L.pyc_b200_gemm.argtypes = [C.POINTER(abi.GemmArgs), vp]
    L.pyc_b200_gemm_static.argtypes = [C.POINTER(abi.GemmArgs), vp]
    L.pyc_b200_gemm_static_status.argtypes = [C.POINTER(C.c_int), vp]
    L.pyc_b200_add.argtypes = [i, vp, vp, vp, sz, vp]
    L.pyc_b200_bias_act.argtypes = [i, vp, vp, i, i, vp, sz, sz, vp]
    L.pyc_b200_layernorm.argtypes = [i, vp, vp, vp, vp, sz, sz, f, vp]
    L.pyc_b200_softmax.argtypes = [i, vp, vp, sz, sz, vp]
    L.pyc_b200_reduce_sum.argtypes = [i, vp, vp, sz, sz, vp]
    L.pyc_b200_quantize_rows.argtypes = [vp, vp, vp, sz, sz, vp]
    L.pyc_b200_layernorm_quantize.argtypes = [vp, vp, vp, vp, vp, sz, sz, f, vp]
    L.pyc_b200_gemm_fp8.argtypes = [i, i, i, vp, vp, i, vp, vp, vp, i, vp, vp]
    L.pyc_b200_ffn_workspace_bytes.argtypes = [i, i, i]
    L.pyc_b200_ffn_workspace_bytes.restype = sz
    L.pyc_b200_ffn_block.argtypes = [C.POINTER(abi.FfnArgs), vp, sz, vp]
    L.pyc_b200_ffn_block_tp.argtypes = [C.POINTER(abi.FfnArgs), vp, vp, i, i, vp, sz, vp]
    L.pyc_b200_autotune_db_load.argtypes = [C.c_char_p]
    L.pyc_b200_last_plan.argtypes = [C.POINTER(abi.IrModule), C.c_char_p, sz]
    L.pyc_b200_ffn_block_scatter.argtypes = [C.POINTER(abi.FfnArgs), vp, sz, C.POINTER(vp), i, i, vp]
    L.pyc_b200_tp_reduce_broadcast.argtypes = [vp, C.POINTER(vp), i, i, i, i, vp]
    L.pyc_b200_ffn_block_switch_reduce.argtypes = [C.POINTER(abi.FfnArgs), vp, sz, vp, C.POINTER(vp), C.POINTER(vp), vp, i, i, vp]
    L.pyc_b200_tp_allreduce_multimem.argtypes = [vp, C.POINTER(vp), vp, i, i, sz, sz, vp]
    L.pyc_b200_symm_alloc.argtypes = [sz, C.POINTER(vp), C.c_char_p]
    L.pyc_b200_symm_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    L.pyc_b200_symm_close.argtypes = [vp]
    L.pyc_b200_symm_free.argtypes = [vp]
    L.pyc_b200_attention.argtypes = [i, i, i, i, vp, vp, vp, vp, f, i, vp]
    L.pyc_b200_conv2d.argtypes = [i] * 12 + [vp, vp, vp, i, vp, vp]
    L.pyc_b200_autotune_gemm.argtypes = [i, i, i, i, i, C.c_char_p, sz, C.POINTER(C.c_double)]
    L.pyc_b200_get_runtime_info.argtypes = [C.POINTER(abi.RuntimeInfo)]
    L.pyc_b200_set_stream.argtypes = [vp, i]
    L.pyc_b200_last_error.restype = C.c_char_p
    L.pyc_b200_shutdown.restype = None
    _lib = L
    return L


def last_error():
    return (load().pyc_b200_last_error() or b"").decode()


def _check(rc, what):
    if rc != 0:
        raise BackendError(f"{what} failed (rc={rc}): {last_error()}")


@abi.CPU_EXECUTOR_FN
def _refuse_cpu(module, inputs, n_in, outputs, n_out, ctx):
    # The seam requires a cpu_executor argument (PyC rejects NULL); this one
    # makes any attempt to leave the GPU an error instead of a silent fallback.
    return -1


def make_tensor(ptr, nbytes, dtype, shape):
    t = abi.Tensor()
    t.data = ptr
    t.size_bytes = nbytes
    t.dtype = dtype
    t.shape = abi.Shape.of(shape)
    return t


def dispatch(module, inputs, outputs, cpu_executor=None, require_gpu=True):
    """pyc_cuda_dispatch.  inputs/outputs: lists of abi.Tensor (host or device pointers).
    Returns (status, trace).  With require_gpu (default) anything but a GPU run raises."""
    L = load()
    ins = (abi.Tensor * len(inputs))(*inputs)
    outs = (abi.Tensor * len(outputs))(*outputs)
    trace = abi.DispatchTrace()
    st = L.pyc_cuda_dispatch(C.byref(module), ins, len(inputs), outs, len(outputs),
                             cpu_executor or _refuse_cpu, None, C.byref(trace))
    if require_gpu and (st != abi.DISPATCH_OK or trace.fallback_to_cpu or not trace.reason.startswith(b"b200_")):
        raise BackendError(f"pyc_cuda_dispatch did not run on the GPU: status={st} reason={trace.reason.decode()!r} {last_error()}")
    return st, trace


def gemm_by_symbol(symbol, M, N, K, A, B, Cptr, alpha=1.0, beta=0.0, stream=0):
    _check(load().pyc_cutlass_gemm_dispatch(symbol.encode(), M, N, K, A, B, Cptr, alpha, beta, stream), f"pyc_cutlass_gemm_dispatch({symbol})")


def gemm(dtype, M, N, K, A, B, D, add=None, add_mode=abi.ADD_NONE, act=abi.ACT_NONE, alpha=1.0,
         b_col_major=False, symbol=None, stream=0):
    a = abi.GemmArgs()
    a.symbol = symbol.encode() if symbol else None
    a.dtype, a.M, a.N, a.K = dtype, M, N, K
    a.A, a.B, a.D = A, B, D
    a.b_col_major = int(b_col_major)
    a.alpha = alpha
    a.add_mode = add_mode if add else abi.ADD_NONE
    a.add = add
    a.act = act
    _check(load().pyc_b200_gemm(C.byref(a), stream), "pyc_b200_gemm")


def gemm_static(dtype, M, N, K, A, B, D, add=None, add_mode=abi.ADD_NONE, act=abi.ACT_NONE, alpha=1.0, b_col_major=False, stream=0):
    """pyc_b200_gemm_static: the tensor-core GEMM without any allocation (see include/pyc_b200.h)."""
    a = abi.GemmArgs()
    a.symbol = None
    a.dtype, a.M, a.N, a.K = dtype, M, N, K
    a.A, a.B, a.D = A, B, D
    a.b_col_major = int(b_col_major)
    a.alpha = alpha
    a.add_mode = add_mode if add else abi.ADD_NONE
    a.add = add
    a.act = act
    _check(load().pyc_b200_gemm_static(C.byref(a), stream), "pyc_b200_gemm_static")


def gemm_static_status(host_int_ptr, stream=0):
    """pyc_b200_gemm_static_status: enqueue the copy of the static block's status word into the int at `host_int_ptr`
    (an address; pinned memory for an asynchronous copy).  Read the int after synchronising `stream`."""
    _check(load().pyc_b200_gemm_static_status(C.cast(host_int_ptr, C.POINTER(C.c_int)), stream), "pyc_b200_gemm_static_status")


def add(dtype, a, b, out, elems, stream=0):
    _check(load().pyc_b200_add(dtype, a, b, out, elems, stream), "pyc_b200_add")


def bias_act(dtype, x, addp, add_mode, act, out, rows, cols, stream=0):
    _check(load().pyc_b200_bias_act(dtype, x, addp, add_mode, act, out, rows, cols, stream), "pyc_b200_bias_act")


def layernorm(dtype, x, gamma, beta, out, rows, cols, eps=1e-5, stream=0):
    _check(load().pyc_b200_layernorm(dtype, x, gamma, beta, out, rows, cols, eps, stream), "pyc_b200_layernorm")


def softmax(dtype, x, out, rows, cols, stream=0):
    _check(load().pyc_b200_softmax(dtype, x, out, rows, cols, stream), "pyc_b200_softmax")


def reduce_sum(dtype, x, out, rows, cols, stream=0):
    _check(load().pyc_b200_reduce_sum(dtype, x, out, rows, cols, stream), "pyc_b200_reduce_sum")


def quantize_rows(x, q, scale, rows, cols, stream=0):
    _check(load().pyc_b200_quantize_rows(x, q, scale, rows, cols, stream), "pyc_b200_quantize_rows")


def layernorm_quantize(x, gamma, beta, q, scale, rows, cols, eps=1e-5, stream=0):
    _check(load().pyc_b200_layernorm_quantize(x, gamma, beta, q, scale, rows, cols, eps, stream), "pyc_b200_layernorm_quantize")


def gemm_fp8(M, N, K, A, B, D, row_scale=None, col_scale=None, bias=None, act=abi.ACT_NONE, b_col_major=False, stream=0):
    _check(load().pyc_b200_gemm_fp8(M, N, K, A, B, int(b_col_major), row_scale, col_scale, bias, act, D, stream), "pyc_b200_gemm_fp8")


def ffn_workspace_bytes(tokens, hidden, inner):
    return int(load().pyc_b200_ffn_workspace_bytes(tokens, hidden, inner))


def ffn_block(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, out, workspace, workspace_bytes,
              ln_gamma=None, ln_beta=None, b1=None, b2=None, eps=1e-5, stream=0):
    a = abi.FfnArgs()
    a.tokens, a.hidden, a.inner = tokens, hidden, inner
    a.x, a.ln_gamma, a.ln_beta, a.eps = x, ln_gamma, ln_beta, eps
    a.w1, a.w1_scale, a.b1 = w1, w1_scale, b1
    a.w2, a.w2_scale, a.b2 = w2, w2_scale, b2
    a.out = out
    _check(load().pyc_b200_ffn_block(C.byref(a), workspace, workspace_bytes, stream), "pyc_b200_ffn_block")


def _ffn_args(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, out, ln_gamma, ln_beta, b1, b2, eps):
    a = abi.FfnArgs()
    a.tokens, a.hidden, a.inner = tokens, hidden, inner
    a.x, a.ln_gamma, a.ln_beta, a.eps = x, ln_gamma, ln_beta, eps
    a.w1, a.w1_scale, a.b1 = w1, w1_scale, b1
    a.w2, a.w2_scale, a.b2 = w2, w2_scale, b2
    a.out = out
    return a


def ffn_block_tp(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, out, workspace, workspace_bytes, comm, comm_handle, world, rank,
                 ln_gamma=None, ln_beta=None, b1=None, b2=None, eps=1e-5, stream=0):
    """pyc_b200_ffn_block_tp: this rank's shard, then one bf16 all-reduce through the pyc_collective_comm vtable at address `comm`."""
    a = _ffn_args(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, out, ln_gamma, ln_beta, b1, b2, eps)
    _check(load().pyc_b200_ffn_block_tp(C.byref(a), comm, comm_handle, world, rank, workspace, workspace_bytes, stream), "pyc_b200_ffn_block_tp")


def last_plan(module=None):
    """Text plan of the most recent GPU run of `module` (None: of any module); None if it has not run."""
    buf = C.create_string_buffer(16384)
    n = load().pyc_b200_last_plan(C.byref(module) if module is not None else None, buf, len(buf))
    return None if n < 0 else buf.value.decode()


def autotune_db_load(path=None):
    return load().pyc_b200_autotune_db_load(path.encode() if path else None)


def ffn_phase_events(event_handles):
    """Five cudaEvent_t handles (ints) recorded by the following FFN block calls of this thread, or None to stop.
    Returns the ctypes table, which must stay alive while the hook is set."""
    L = load()
    L.pyc_b200_ffn_phase_events.argtypes = [C.POINTER(C.c_void_p)]
    if event_handles is None:
        L.pyc_b200_ffn_phase_events(None)
        return None
    table = (C.c_void_p * 5)(*event_handles)
    L.pyc_b200_ffn_phase_events(table)
    return table


def ffn_block_scatter(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, workspace, workspace_bytes, recv_slots, rank,
                      ln_gamma=None, ln_beta=None, b1=None, b2=None, eps=1e-5, stream=0):
    """The FFN block whose last GEMM stores every row into slot `rank` of the owning rank's receive buffer (recv_slots[owner])."""
    a = _ffn_args(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, None, ln_gamma, ln_beta, b1, b2, eps)
    world = len(recv_slots)
    table = (C.c_void_p * world)(*recv_slots)
    _check(load().pyc_b200_ffn_block_scatter(C.byref(a), workspace, workspace_bytes, table, world, rank, stream), "pyc_b200_ffn_block_scatter")


def tp_reduce_broadcast(recv_local, outs, rank, rows_per_rank, hidden, stream=0):
    world = len(outs)
    table = (C.c_void_p * world)(*outs)
    _check(load().pyc_b200_tp_reduce_broadcast(recv_local, table, world, rank, rows_per_rank, hidden, stream), "pyc_b200_tp_reduce_broadcast")


TP_MULTIMEM_BLOCKS, TP_MAX_RANKS = 128, 8     # PYC_B200_TP_MULTIMEM_BLOCKS, PYC_B200_TP_MAX_RANKS


TP_FUSED_EPOCH_SLOTS = 256     # PYC_B200_TP_FUSED_EPOCH_SLOTS


def ffn_block_switch_reduce(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, out, workspace, workspace_bytes, multicast_out,
                            flag_ptrs, fin_ptrs, epoch_counters, rank, ln_gamma=None, ln_beta=None, b1=None, b2=None, eps=1e-5, stream=0):
    """The FFN block whose last GEMM all-reduces its result inside the NVSwitch while it runs (out: this rank's copy of the
    multicast-bound buffer, multicast_out: its multicast address)."""
    a = _ffn_args(tokens, hidden, inner, x, w1, w1_scale, w2, w2_scale, out, ln_gamma, ln_beta, b1, b2, eps)
    world = len(flag_ptrs)
    _check(load().pyc_b200_ffn_block_switch_reduce(C.byref(a), workspace, workspace_bytes, multicast_out, (C.c_void_p * world)(*flag_ptrs),
                                                   (C.c_void_p * world)(*fin_ptrs), epoch_counters, world, rank, stream),
           "pyc_b200_ffn_block_switch_reduce")


def tp_allreduce_multimem(multicast_ptr, flag_ptrs, epoch_counters, rank, rows, hidden, stream=0):
    """In-switch all-reduce (sum, bf16, in place) of the [rows, hidden] tensor at `multicast_ptr`; flag_ptrs: one per rank."""
    world = len(flag_ptrs)
    table = (C.c_void_p * world)(*flag_ptrs)
    _check(load().pyc_b200_tp_allreduce_multimem(multicast_ptr, table, epoch_counters, world, rank, rows, hidden, stream),
           "pyc_b200_tp_allreduce_multimem")


def symm_alloc(nbytes):
    """(device pointer, 64-byte handle another process of this node can open)"""
    ptr = C.c_void_p()
    handle = C.create_string_buffer(64)
    _check(load().pyc_b200_symm_alloc(nbytes, C.byref(ptr), handle), "pyc_b200_symm_alloc")
    return ptr.value, handle.raw


def symm_open(handle):
    ptr = C.c_void_p()
    _check(load().pyc_b200_symm_open(handle, C.byref(ptr)), "pyc_b200_symm_open")
    return ptr.value


def symm_close(ptr):
    _check(load().pyc_b200_symm_close(ptr), "pyc_b200_symm_close")


def symm_free(ptr):
    _check(load().pyc_b200_symm_free(ptr), "pyc_b200_symm_free")


def attention(dtype, batch_heads, seq, d, q, k, v, out, scale, causal, stream=0):
    _check(load().pyc_b200_attention(dtype, batch_heads, seq, d, q, k, v, out, scale, int(causal), stream), "pyc_b200_attention")


def conv2d(dtype, N, H, W, Cin, K, R, S, pad, stride, x, w, bias, relu, out, stream=0):
    _check(load().pyc_b200_conv2d(dtype, N, H, W, Cin, K, R, S, pad[0], pad[1], stride[0], stride[1], x, w, bias, int(relu), out, stream), "pyc_b200_conv2d")


def autotune_gemm(dtype, M, N, K, iters=5):
    buf = C.create_string_buffer(abi.PYC_KERNEL_SYMBOL_MAX)
    ms = C.c_double()
    n = load().pyc_b200_autotune_gemm(dtype, M, N, K, iters, buf, len(buf), C.byref(ms))
    if n < 0:
        raise BackendError(f"pyc_b200_autotune_gemm failed: {last_error()}")
    return buf.value.decode(), ms.value, n


def runtime_info():
    info = abi.RuntimeInfo()
    load().pyc_b200_get_runtime_info(C.byref(info))
    return info


def kernel_count(op_key):
    return load().pyc_cutlass_kernel_count(op_key.encode())


def set_stream(stream, async_=False):
    _check(load().pyc_b200_set_stream(stream, int(async_)), "pyc_b200_set_stream")


def selftest_wait_timeout(limit_us=50, stream=0):
    _check(load().pyc_b200_selftest_wait_timeout(limit_us, stream), "pyc_b200_selftest_wait_timeout")


def device_status():
    return load().pyc_b200_device_status()
