"""GPU parity: HBM-bound kernels (add, bias+activation, layernorm, softmax,
reduce_sum) through the C-ABI against the CPU oracle.  Tolerances norm-wise:
fp32 1e-5, bf16/f16 2e-2 (outputs rounded to the storage type)."""
import numpy as np
import pytest

from pyc_b200 import abi, workloads

pytestmark = pytest.mark.gpu
DTYPES = [abi.DTYPE_F32, abi.DTYPE_BF16, abi.DTYPE_F16]
# (rows, cols): warp-per-row, block-per-row (cached), wide rows (re-read path), odd widths (scalar path)
SHAPES = [(64, 96), (37, 1024), (16, 4096), (8, 16384), (5, 40000), (33, 77), (3, 1)]


def _setup(dtype, shape, seed, std=1.0):
    from gpu_util import empty_device, round_to, to_device
    x_s, x_r = round_to(dtype, workloads.normal(shape, seed, std))
    return to_device(x_s), x_r, empty_device(dtype, shape)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_layernorm_softmax_reduce(backend, oracle_lib, dtype, shape):
    from gpu_util import TOL, empty_device, rel_err, round_to, sync_ok, to_device, to_host_f32
    rows, cols = shape
    d_x, x_r, d_o = _setup(dtype, shape, 41 + cols)
    if cols > 1:
        backend.layernorm(dtype, d_x.data_ptr(), None, None, d_o.data_ptr(), rows, cols)
        sync_ok()
        assert rel_err(to_host_f32(dtype, d_o), oracle_lib.layernorm(x_r)) <= TOL[dtype]
        g_s, g_r = round_to(dtype, workloads.uniform((cols,), 5)); b_s, b_r = round_to(dtype, workloads.uniform((cols,), 6))
        d_g, d_b = to_device(g_s), to_device(b_s)
        backend.layernorm(dtype, d_x.data_ptr(), d_g.data_ptr(), d_b.data_ptr(), d_o.data_ptr(), rows, cols)
        sync_ok()
        assert rel_err(to_host_f32(dtype, d_o), oracle_lib.layernorm(x_r, g_r, b_r)) <= TOL[dtype]
    backend.softmax(dtype, d_x.data_ptr(), d_o.data_ptr(), rows, cols)
    sync_ok()
    assert rel_err(to_host_f32(dtype, d_o), oracle_lib.softmax(x_r)) <= TOL[dtype]
    d_s = empty_device(dtype, (rows,))
    backend.reduce_sum(dtype, d_x.data_ptr(), d_s.data_ptr(), rows, cols)
    sync_ok()
    want = oracle_lib.reduce_sum(x_r)
    # fp32 row sums: the GPU adds in a different order, bound the error by the sum of magnitudes
    err = np.abs(to_host_f32(dtype, d_s).astype(np.float64) - want).max()
    assert err <= TOL[dtype] * max(np.abs(x_r).sum(-1).max(), 1e-30)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(128, 256), (33, 77), (1, 8), (2048, 4096)])
def test_add_and_bias_act(backend, oracle_lib, dtype, shape):
    from gpu_util import TOL, rel_err, round_to, sync_ok, to_device, to_host_f32
    rows, cols = shape
    d_x, x_r, d_o = _setup(dtype, shape, 51)
    y_s, y_r = round_to(dtype, workloads.normal(shape, 52)); d_y = to_device(y_s)
    backend.add(dtype, d_x.data_ptr(), d_y.data_ptr(), d_o.data_ptr(), rows * cols)
    sync_ok()
    assert rel_err(to_host_f32(dtype, d_o), oracle_lib.add(x_r, y_r)) <= TOL[dtype]
    b_s, b_r = round_to(dtype, workloads.normal((cols,), 53)); d_b = to_device(b_s)
    for mode, addp, addv in [(abi.ADD_ROW_BIAS, d_b, b_r), (abi.ADD_MATRIX, d_y, y_r), (abi.ADD_SCALAR, d_b, b_r[:1]), (abi.ADD_NONE, None, None)]:
        for act, fn in [(abi.ACT_NONE, lambda v: v), (abi.ACT_RELU, oracle_lib.relu), (abi.ACT_GELU, oracle_lib.gelu)]:
            backend.bias_act(dtype, d_x.data_ptr(), addp.data_ptr() if addp is not None else None, mode, act, d_o.data_ptr(), rows, cols)
            sync_ok()
            want = fn(oracle_lib.add(x_r, addv) if addv is not None else x_r)
            assert rel_err(to_host_f32(dtype, d_o), want) <= TOL[dtype], (mode, act)


def test_relu_is_bit_exact_f32(backend, oracle_lib):
    # pure selection: no rounding involved, so the bar is bit-exact
    from gpu_util import sync_ok
    d_x, x_r, d_o = _setup(abi.DTYPE_F32, (257, 513), 61)
    backend.bias_act(abi.DTYPE_F32, d_x.data_ptr(), None, abi.ADD_NONE, abi.ACT_RELU, d_o.data_ptr(), 257, 513)
    sync_ok()
    assert d_o.cpu().numpy().tobytes() == oracle_lib.relu(x_r).tobytes()
    d_y, y_r, _ = _setup(abi.DTYPE_F32, (257, 513), 62)
    backend.add(abi.DTYPE_F32, d_x.data_ptr(), d_y.data_ptr(), d_o.data_ptr(), 257 * 513)
    sync_ok()
    assert d_o.cpu().numpy().tobytes() == oracle_lib.add(x_r, y_r).tobytes()
