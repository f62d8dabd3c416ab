"""GPU: ops PyC's IR has no kind for -- attention, conv2d, softmax, the fp8 FFN block -- flowing through PyC's unmodified
pyc_compile_model / pyc_run_model.  They are carried by REDUCE_SUM ops whose NAME ("b200.<op>...") is the attribute side
table the backend reads; PyC's front half passes names and declared shapes through untouched.  Each result is checked against
the CPU oracle at the dtype's tolerance, and PyC's decision log must say the GPU ran it."""
import os

import numpy as np
import pytest

import oracle
from pyc_b200 import abi, ir, workloads

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(oracle.REF_FRONT_SO), reason="PyC's front half was not built (no PyC checkout at build time)")]


@pytest.fixture(scope="module")
def front():
    return oracle.RefRuntime(oracle.REF_FRONT_SO, threads=4)


def _run(front, backend, module, inputs, out_shape, out_dtype, expect_kernel):
    model = front.compile(module, backend=abi.BACKEND_CUDA, fusion=0)
    for _ in range(2):
        out, = front.run(model, inputs, [(out_shape, out_dtype)])
    log = front.decision_log(model)
    assert "cuda_fallback=0" in log and "b200_graph_" in log, log
    assert expect_kernel in backend.last_plan(module)
    front.destroy(model)
    return out


def test_attention_causal_through_pyc_run_model(front, backend, oracle_lib):
    BH, S, D = 6, 320, 128
    bits = [workloads.to_bf16_bits(workloads.normal((BH, S, D), 1300 + i)) for i in range(3)]
    q, k, v = (workloads.bf16_bits_to_f32(b) for b in bits)
    b = ir.ModuleBuilder()
    ids = [b.input(n, abi.DTYPE_BF16, [BH, S, D]) for n in "qkv"]
    b.output(b.extended("b200.attention.causal", abi.DTYPE_BF16, [BH, S, D], ids))
    out = _run(front, backend, b.module, [(t, abi.DTYPE_BF16) for t in bits], (BH, S, D), abi.DTYPE_BF16, "b200_attention_bf16_causal")
    want = oracle_lib.attention(q, k, v, D ** -0.5, True)
    assert np.abs(workloads.bf16_bits_to_f32(out) - want).max() / np.abs(want).max() <= 2e-2


def test_conv2d_bias_relu_and_softmax_through_pyc_run_model(front, backend, oracle_lib):
    N, H, W, C, K = 3, 14, 18, 64, 96
    xb = workloads.to_bf16_bits(workloads.uniform((N, H, W, C), 1310)); wb = workloads.to_bf16_bits(workloads.normal((K, 3, 3, C), 1311, (2.0 / (9 * C)) ** 0.5))
    bb = workloads.to_bf16_bits(workloads.normal((K,), 1312, 0.1))
    b = ir.ModuleBuilder()
    ids = [b.input("x", abi.DTYPE_BF16, [N, H, W, C]), b.input("w", abi.DTYPE_BF16, [K, 3, 3, C]), b.input("bias", abi.DTYPE_BF16, [K])]
    b.output(b.extended("b200.conv2d.p1x1.s1x1.relu", abi.DTYPE_BF16, [N, H, W, K], ids))
    out = _run(front, backend, b.module, [(t, abi.DTYPE_BF16) for t in (xb, wb, bb)], (N, H, W, K), abi.DTYPE_BF16, "b200_conv2d_fprop_bf16")
    want = oracle_lib.conv2d(workloads.bf16_bits_to_f32(xb), workloads.bf16_bits_to_f32(wb), workloads.bf16_bits_to_f32(bb), relu=True)
    assert np.abs(workloads.bf16_bits_to_f32(out) - want).max() / np.abs(want).max() <= 2e-2
    # softmax behind a matmul: an extended op consuming an ordinary IR op's result
    M, Kd, Nd = 64, 96, 1000
    x = workloads.normal((M, Kd), 1320); w = workloads.normal((Kd, Nd), 1321, 0.2)
    b = ir.ModuleBuilder()
    mm = b.matmul(b.input("x", abi.DTYPE_F32, [M, Kd]), b.input("w", abi.DTYPE_F32, [Kd, Nd]))
    b.output(b.extended("b200.softmax", abi.DTYPE_F32, [M, Nd], [mm]))
    out = _run(front, backend, b.module, [(x, abi.DTYPE_F32), (w, abi.DTYPE_F32)], (M, Nd), abi.DTYPE_F32, "b200_softmax_f32")
    want = oracle_lib.softmax(oracle_lib.matmul(x, w))
    assert np.abs(out - want).max() / np.abs(want).max() <= 1e-5


def test_fp8_ffn_block_through_pyc_run_model(front, backend, oracle_lib):
    T, H, I = 256, 256, 1024
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(T, H, I)
    b = ir.ModuleBuilder()
    ids = [b.input("x", abi.DTYPE_BF16, [T, H]), b.input("w1", abi.DTYPE_I8, [H, I]), b.input("s1", abi.DTYPE_F32, [I]),
           b.input("w2", abi.DTYPE_I8, [I, H]), b.input("s2", abi.DTYPE_F32, [H])]
    b.output(b.extended("b200.ffn_fp8", abi.DTYPE_BF16, [T, H], ids))
    ins = [(xb, abi.DTYPE_BF16), (w1.view(np.int8), abi.DTYPE_I8), (s1.astype(np.float32), abi.DTYPE_F32), (w2.view(np.int8), abi.DTYPE_I8),
           (s2.astype(np.float32), abi.DTYPE_F32)]
    out = _run(front, backend, b.module, ins, (T, H), abi.DTYPE_BF16, "b200_ffn_fp8_block")
    want = oracle.ffn_reference(oracle_lib, workloads.bf16_bits_to_f32(xb), w1, s1, w2, s2)
    assert np.abs(workloads.bf16_bits_to_f32(out) - want).max() / np.abs(want).max() <= 6e-2


def test_unknown_extended_name_is_not_run_on_the_gpu(backend):
    from test_gpu_dispatch import _host
    b = ir.ModuleBuilder()
    x = b.input("x", abi.DTYPE_F32, [4, 4])
    b.output(b.extended("b200.no_such_op", abi.DTYPE_F32, [4, 4], [x]))
    a = np.zeros((4, 4), np.float32)
    st, trace = backend.dispatch(b.module, [_host(a, 1)], [_host(a.copy(), 1)], require_gpu=False)
    assert st == abi.DISPATCH_ERROR and b"b200_unsupported_module" in trace.reason
