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
    status = torch.full((1,), -7, dtype=torch.int32).pin_memory()
    for call, (M, K, N, mode, act) in enumerate(cases):   # two calls in a row, different shapes and epilogues
        a_s, a_r = round_to(dtype, workloads.normal((M, K), 500 + call)); b_s, b_r = round_to(dtype, workloads.normal((K, N), 600 + call))
        c_s, c_r = round_to(dtype, workloads.normal((N,) if mode == abi.ADD_ROW_BIAS else (M, N), 700 + call, 4.0))
        d_a, d_b, d_c = to_device(a_s), to_device(b_s), to_device(c_s)
        out_static, out_ref = empty_device(dtype, (M, N)), empty_device(dtype, (M, N))
        backend.gemm_static(dtype, M, N, K, d_a.data_ptr(), d_b.data_ptr(), out_static.data_ptr(), add=d_c.data_ptr(), add_mode=mode, act=act)
        backend.gemm_static_status(status.data_ptr())          # no allocation either: one 4-byte copy on the same stream
        torch.cuda.synchronize()
        assert int(status[0]) == 0, f"a bounded wait of the static GEMM gave up: 0x{int(status[0]):x}"
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


@pytest.mark.parametrize("case", ["f16_colmajor_b", "narrow_n64", "scalar_add", "unaligned_d"])
def test_static_scratch_gemm_other_instances(backend, oracle_lib, case):
    """The template instances only this entry point reaches: f16 with B stored [N,K], the 64-wide tile, the scalar add,
    and an output that is not 16-byte aligned (element-wise stores).  Each against the CPU oracle, status word checked."""
    from gpu_util import TOL, rel_err, round_to, to_device, to_host_f32
    import torch
    dtype = abi.DTYPE_F16 if case == "f16_colmajor_b" else abi.DTYPE_BF16
    M, K, N = {"f16_colmajor_b": (256, 320, 384), "narrow_n64": (96, 256, 64), "scalar_add": (128, 128, 256), "unaligned_d": (128, 192, 136)}[case]
    a_s, a_r = round_to(dtype, workloads.normal((M, K), 811)); b_s, b_r = round_to(dtype, workloads.normal((K, N), 812))
    colmajor = case == "f16_colmajor_b"
    d_a, d_b = to_device(a_s), to_device(np.ascontiguousarray(b_s.T) if colmajor else b_s)
    want = oracle_lib.matmul(a_r, b_r)
    add = mode = None
    if case == "scalar_add":
        c_s, c_r = round_to(dtype, np.array([1.25], np.float32))
        d_c = to_device(c_s); add, mode = d_c.data_ptr(), abi.ADD_SCALAR
        want = oracle_lib.add(want, c_r)
    pad = 1 if case == "unaligned_d" else 0               # output starts 2 bytes past a 16-byte boundary
    raw = torch.zeros(M * N + 8, dtype=torch.int16, device="cuda")
    out = raw[pad:pad + M * N]
    status = torch.full((1,), -7, dtype=torch.int32).pin_memory()
    for _ in range(2):
        backend.gemm_static(dtype, M, N, K, d_a.data_ptr(), d_b.data_ptr(), out.data_ptr(), add=add, add_mode=mode or abi.ADD_NONE,
                            act=abi.ACT_NONE, b_col_major=colmajor)
        backend.gemm_static_status(status.data_ptr())
        torch.cuda.synchronize()
        assert int(status[0]) == 0
    got = to_host_f32(dtype, out.reshape(M, N))
    assert rel_err(got, want) <= TOL[dtype]
    assert int(raw[M * N + pad:].abs().max()) == 0 and (pad == 0 or int(raw[0]) == 0)   # nothing written outside D
