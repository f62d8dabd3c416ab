"""CPU: the C-ABI library loads without a GPU, exports every symbol the header
declares, and honours the dispatch contract PyC's own tests pin
(tests/compiler_next/test_cuda_backend.c, test_production_cuda_contracts.c):
reason strings, status codes, env switches.  No kernel runs here.
"""
import ctypes as C
import os
import re

import numpy as np
import pytest

from pyc_b200 import abi, backend, ir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV_KEYS = ["PYC_CUDA_DISABLE", "PYC_CUDA_FORCE_ERROR", "PYC_CUDA_FORCE_FALLBACK", "PYC_CUDA_SIMULATE_AVAILABLE"]


@pytest.fixture
def clean_env():
    saved = {k: os.environ.get(k) for k in ENV_KEYS}
    for k in ENV_KEYS:
        os.environ.pop(k, None)
    yield os.environ
    for k, v in saved.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


def header_functions():
    text = open(os.path.join(ROOT, "include", "pyc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pyc_(?:cuda|cutlass|b200)_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = backend.load()
    declared = header_functions()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/pyc_b200.h but not exported"
    assert sorted(declared) == sorted(backend.EXPORTS)


def test_pyc_drop_in_symbol_names_present():
    # The eight symbols PyC's cuda_backend.c + cutlass_kernels export (nm of PyC's own archive).
    lib = backend.load()
    for name in ["pyc_cuda_dispatch", "pyc_cuda_dispatch_trace_init", "pyc_cuda_current_hardware_family",
                 "pyc_cutlass_gemm_dispatch", "pyc_cutlass_conv2d_dispatch", "pyc_cutlass_attention_dispatch",
                 "pyc_cutlass_kernel_count", "pyc_cutlass_registry_init"]:
        assert hasattr(lib, name)


def test_registry_counts_and_unknown_symbol():
    assert backend.kernel_count("matmul") >= 9
    assert backend.kernel_count("conv2d") >= 2
    assert backend.kernel_count("attention") >= 2
    assert backend.kernel_count("nonexistent") == 0
    lib = backend.load()
    assert lib.pyc_cutlass_gemm_dispatch(b"no_such_kernel", 8, 8, 8, None, None, None, 1.0, 0.0, None) == -1
    assert "unknown GEMM symbol" in backend.last_error()


def _host_tensors(arrays, dtype=abi.DTYPE_F32):
    return [backend.make_tensor(a.ctypes.data, a.nbytes, dtype, a.shape) for a in arrays]


def _kat():
    lhs = np.array([[1, -2], [3, 4]], np.float32); rhs = np.array([[2, 1], [-1, 3]], np.float32)
    bias = np.array([0.5, -1.5], np.float32); out = np.zeros((2, 2), np.float32)
    return ir.matmul_bias_act(abi.DTYPE_F32, 2, 2, 2, bias="row", act="relu"), [lhs, rhs, bias], out


def test_null_arguments_are_errors(clean_env):
    lib = backend.load()
    trace = abi.DispatchTrace()
    assert lib.pyc_cuda_dispatch(None, None, 0, None, 0, backend._refuse_cpu, None, C.byref(trace)) == abi.DISPATCH_ERROR
    lib.pyc_cuda_dispatch_trace_init(C.byref(trace))
    assert trace.reason == b"" and trace.cuda_requested == 0


def test_in_switch_all_reduce_rejects_bad_arguments_before_touching_a_device(clean_env):
    lib = backend.load()
    flags = (C.c_void_p * 2)(0x1000, 0x2000)
    call = lambda mc, fl, ep, world, rank, rows, hidden: lib.pyc_b200_tp_allreduce_multimem(mc, fl, ep, world, rank, rows, hidden, None)
    assert call(None, flags, 0x3000, 2, 0, 8, 64) == -1                      # no multicast address
    assert call(0x4000, flags, 0x3000, 1, 0, 8, 64) == -1                    # one rank has nothing to exchange
    assert call(0x4000, flags, 0x3000, 9, 0, 8, 64) == -1                    # more than PYC_B200_TP_MAX_RANKS
    assert call(0x4000, flags, 0x3000, 2, 2, 8, 64) == -1                    # rank out of range
    assert call(0x4000, flags, 0x3000, 2, 0, 8, 60) == -1                    # hidden not a multiple of 8 (16-byte pieces)
    assert call(0x4008, flags, 0x3000, 2, 0, 8, 64) == -1                    # misaligned tensor
    assert b"multimem" in lib.pyc_b200_last_error()


def test_fused_switch_reduce_rejects_bad_arguments_before_touching_a_device(clean_env):
    lib = backend.load()
    args = abi.FfnArgs()
    ptrs = (C.c_void_p * 2)(0x1000, 0x2000)
    call = lambda a, mc, fl, fin, ep, world, rank: lib.pyc_b200_ffn_block_switch_reduce(a, 0x5000, 1 << 20, mc, fl, fin, ep, world, rank, None)
    assert call(None, 0x4000, ptrs, ptrs, 0x3000, 2, 0) == -1                      # no arguments
    assert call(C.byref(args), None, ptrs, ptrs, 0x3000, 2, 0) == -1               # no multicast address
    assert call(C.byref(args), 0x4000, None, ptrs, 0x3000, 2, 0) == -1             # no flag table
    assert call(C.byref(args), 0x4000, ptrs, ptrs, None, 2, 0) == -1               # no epoch counters
    assert call(C.byref(args), 0x4000, ptrs, ptrs, 0x3000, 1, 0) == -1             # one rank has nothing to exchange
    assert call(C.byref(args), 0x4000, ptrs, ptrs, 0x3000, 2, 5) == -1             # rank out of range
    assert b"switch reduce" in lib.pyc_b200_last_error()


def test_forced_error(clean_env):
    clean_env["PYC_CUDA_FORCE_ERROR"] = "1"
    mod, ins, out = _kat()
    st, trace = backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]), require_gpu=False)
    assert st == abi.DISPATCH_ERROR and trace.reason == b"forced_error" and trace.fallback_to_cpu == 0


def test_disabled_by_env_falls_back_to_callers_executor(clean_env):
    clean_env["PYC_CUDA_DISABLE"] = "1"
    calls = []

    @abi.CPU_EXECUTOR_FN
    def executor(module, inputs, n_in, outputs, n_out, ctx):
        calls.append((n_in, n_out))
        return 0

    mod, ins, out = _kat()
    st, trace = backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]), cpu_executor=executor, require_gpu=False)
    assert st == abi.DISPATCH_FALLBACK and trace.fallback_to_cpu == 1 and trace.reason == b"disabled_by_env"
    assert calls == [(3, 1)] and trace.cuda_available == 0
    # and when that executor fails, the dispatch is an error
    st, trace = backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]), require_gpu=False)
    assert st == abi.DISPATCH_ERROR and trace.reason == b"cpu_fallback_failed"


def test_forced_fallback_reason(clean_env):
    clean_env["PYC_CUDA_SIMULATE_AVAILABLE"] = "1"
    clean_env["PYC_CUDA_FORCE_FALLBACK"] = "1"

    @abi.CPU_EXECUTOR_FN
    def executor(module, inputs, n_in, outputs, n_out, ctx):
        return 0

    mod, ins, out = _kat()
    st, trace = backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]), cpu_executor=executor, require_gpu=False)
    assert st == abi.DISPATCH_FALLBACK and trace.reason == b"cuda_forced_fallback" and trace.cuda_available == 1


def _no_gpu():
    import torch
    return not torch.cuda.is_available()


@pytest.mark.skipif(not _no_gpu(), reason="the host stand-in only answers when no device exists")
def test_simulated_device_contract(clean_env):
    # tests/compiler_next/test_cuda_backend.c:84-89 and :252-312 on a machine without CUDA.
    clean_env["PYC_CUDA_SIMULATE_AVAILABLE"] = "1"
    mod, ins, out = _kat()
    for _ in range(2):
        out[:] = 0
        st, trace = backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]), require_gpu=False)
        assert st == abi.DISPATCH_OK and trace.fallback_to_cpu == 0 and trace.reason == b"cuda_native_simulated"
        assert out.reshape(-1).tolist() == [4.5, 0.0, 2.5, 13.5]
    bits = np.array([0x3F80, 0x4000, 0x4040, 0x4080], np.uint16); got = np.zeros(4, np.uint16)
    b = ir.ModuleBuilder(); b.output(b.input("input0", abi.DTYPE_BF16, [4]))
    st, trace = backend.dispatch(b.module, _host_tensors([bits], abi.DTYPE_BF16), _host_tensors([got], abi.DTYPE_BF16), require_gpu=False)
    assert st == abi.DISPATCH_OK and got.tolist() == bits.tolist()


@pytest.mark.skipif(not _no_gpu(), reason="needs a machine without a device")
def test_no_device_is_loud_not_silent(clean_env):
    mod, ins, out = _kat()
    with pytest.raises(backend.BackendError):
        backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]))  # require_gpu defaults to True
    st, trace = backend.dispatch(mod, _host_tensors(ins), _host_tensors([out]), require_gpu=False)
    assert st == abi.DISPATCH_ERROR  # the refusing executor fails, nothing computed on the CPU
    assert out.sum() == 0


def test_hardware_family_override(clean_env):
    lib = backend.load()
    os.environ["PYC_CUDA_FORCE_HARDWARE_FAMILY"] = "ada"
    try:
        assert lib.pyc_cuda_current_hardware_family() == 2
        os.environ["PYC_CUDA_FORCE_HARDWARE_FAMILY"] = "hopper"
        assert lib.pyc_cuda_current_hardware_family() == 3
    finally:
        os.environ.pop("PYC_CUDA_FORCE_HARDWARE_FAMILY", None)
