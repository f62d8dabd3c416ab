"""GPU: pyc_b200_gemm_static, the GEMM entry point for callers that cannot
allocate device memory (a host that owns all of HBM through its own pool, a
thread that must not stall the device with an allocation).  Its scratch is a
small array built into the library instead of a context created on first use.

Checked through the C-ABI against the ordinary entry point (pyc_b200_gemm, same
math: results must agree within the 2e-2 bf16 tolerance the other tests use) and against the CPU oracle, on two calls in a row -- the second call
reuses the shared scratch block the first one left behind.  Collected last on
purpose (file name), so a failure here cannot hide another test's result.
"""
import numpy as np
import pytest

from pyc_b200 import abi, workloads

pytestmark = pytest.mark.gpu


def test_static_scratch_gemm_matches_allocating_entry_point_twice(backend, oracle_lib):
    from gpu_util import TOL, empty_device, rel_err, round_to, to_device, to_host_f32
    import torch
    dtype = abi.DTYPE_BF16
    cases = [(384, 512, 1024, abi.ADD_ROW_BIAS, abi.ACT_GELU), (200, 264, 328, abi.ADD_MATRIX, abi.ACT_RELU)]
    for call, (M, K, N, mode, act) in enumerate(cases):   # two calls in a row, different shapes and epilogues
        a_s, a_r = round_to(dtype, workloads.normal((M, K), 500 + call)); b_s, b_r = round_to(dtype, workloads.normal((K, N), 600 + call))
        c_s, c_r = round_to(dtype, workloads.normal((N,) if mode == abi.ADD_ROW_BIAS else (M, N), 700 + call, 4.0))
        d_a, d_b, d_c = to_device(a_s), to_device(b_s), to_device(c_s)
        out_static, out_ref = empty_device(dtype, (M, N)), empty_device(dtype, (M, N))
        backend.gemm_static(dtype, M, N, K, d_a.data_ptr(), d_b.data_ptr(), out_static.data_ptr(), add=d_c.data_ptr(), add_mode=mode, act=act)
        torch.cuda.synchronize()
        backend.gemm(dtype, M, N, K, d_a.data_ptr(), d_b.data_ptr(), out_ref.data_ptr(), add=d_c.data_ptr(), add_mode=mode, act=act)
        torch.cuda.synchronize()
        got, ref = to_host_f32(dtype, out_static), to_host_f32(dtype, out_ref)
        assert rel_err(got, ref) <= TOL[dtype]
        # (the ordinary entry point may pick another tile configuration for the shape, so equality is not required)
        want = oracle_lib.add(oracle_lib.matmul(a_r, b_r), c_r)
        want = oracle_lib.gelu(want) if act == abi.ACT_GELU else oracle_lib.relu(want)
        assert rel_err(got, want) <= TOL[dtype]


def test_static_scratch_gemm_rejects_what_it_cannot_take(backend):
    import torch
    x = torch.zeros(64, dtype=torch.int16, device="cuda")
    p = x.data_ptr()
    for kwargs, text in [(dict(M=(1 << 20) + 1, N=8, K=8), "exceeds the supported maximum"),
                         (dict(M=8, N=8, K=12), "K % 8"),
                         (dict(M=8, N=12, K=8), "N % 8")]:
        with pytest.raises(backend.BackendError, match=text.replace("%", "%")):
            backend.gemm_static(abi.DTYPE_BF16, kwargs["M"], kwargs["N"], kwargs["K"], p, p, p)
    with pytest.raises(backend.BackendError, match="only bf16 and f16"):
        backend.gemm_static(abi.DTYPE_F32, 8, 8, 8, p, p, p)
