"""CPU: pin the oracle (oracle/pyc_oracle.c) before anything trusts it.

1. Known-answer vectors of PyC's own tests, read from
   tests/compiler_next/test_cpu_execution.c:56-59,135-138 and
   tests/compiler_next/test_cuda_backend.c:84-89,261-262.
2. Bit-exact agreement with outputs of PyC's unmodified CPU executor stored in
   tests/golden/ref_cpu_cases.npz (made by tests/golden/make_golden.py).
3. When oracle/_ref/libpyc_ref_cpu.so is present (built from a PyC checkout),
   live bit-exact comparison on fresh seeds.
4. Definitions of the ops PyC does not implement (unpinned) against numpy.
"""
import importlib.util
import math
import os

import numpy as np
import pytest

import oracle
from pyc_b200 import abi, ir, workloads

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)


def test_kat_matmul_2x3_3x2(oracle_lib):
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([[1, 2], [3, 4], [5, 6]], np.float32)
    assert oracle_lib.matmul(a, b).reshape(-1).tolist() == [22.0, 28.0, 49.0, 64.0]


def test_kat_add_relu(oracle_lib):
    a = np.array([-1, 2, -3, 4], np.float32)
    b = np.array([2, -5, 4, -1], np.float32)
    assert oracle_lib.relu(oracle_lib.add(a, b)).tolist() == [1.0, 0.0, 1.0, 3.0]


def test_kat_row_bias_relu_module(oracle_lib):
    # test_cuda_backend.c:84-89
    lhs = np.array([[1, -2], [3, 4]], np.float32)
    rhs = np.array([[2, 1], [-1, 3]], np.float32)
    bias = np.array([0.5, -1.5], np.float32)
    mod = ir.matmul_bias_act(abi.DTYPE_F32, 2, 2, 2, bias="row", act="relu")
    out, = oracle_lib.run_module(mod, [(lhs, abi.DTYPE_F32), (rhs, abi.DTYPE_F32), (bias, abi.DTYPE_F32)], [((2, 2), abi.DTYPE_F32)])
    assert out.reshape(-1).tolist() == [4.5, 0.0, 2.5, 13.5]
    assert np.array_equal(out, oracle_lib.relu(oracle_lib.add(oracle_lib.matmul(lhs, rhs), bias)))


def test_kat_bf16_passthrough_bytes(oracle_lib):
    bits = np.array([0x3F80, 0x4000, 0x4040, 0x4080], np.uint16)  # test_cuda_backend.c:261-262
    b = ir.ModuleBuilder()
    b.output(b.input("input0", abi.DTYPE_BF16, [4]))
    out, = oracle_lib.run_module(b.module, [(bits, abi.DTYPE_BF16)], [((4,), abi.DTYPE_BF16)])
    assert out.tolist() == bits.tolist()
    assert workloads.bf16_bits_to_f32(bits).tolist() == [1.0, 2.0, 3.0, 4.0]


@pytest.mark.parametrize("idx", range(len(make_golden.CASES)))
def test_golden_bit_exact(oracle_lib, idx):
    name, M, K, N, bias, act = make_golden.CASES[idx]
    gold = np.load(os.path.join(GOLDEN, "ref_cpu_cases.npz"))[name]
    a, b, c = make_golden.case_inputs(idx, M, K, N, bias)
    mod = ir.matmul_bias_act(abi.DTYPE_F32, M, K, N, bias=bias, act=act)
    ins = [(a, abi.DTYPE_F32), (b, abi.DTYPE_F32)] + ([(c, abi.DTYPE_F32)] if bias else [])
    out, = oracle_lib.run_module(mod, ins, [((M, N), abi.DTYPE_F32)])
    assert out.tobytes() == gold.tobytes()
    for threads in (1, 3):  # row splitting never changes a result
        oracle_lib.set_threads(threads)
        assert oracle_lib.matmul(a, b).tobytes() == oracle.Oracle().matmul(a, b).tobytes()
    oracle_lib.set_threads(os.cpu_count() or 1)


@pytest.mark.skipif(not os.path.exists(oracle.REF_CPU_SO), reason="PyC's own CPU runtime was not built (no PyC checkout)")
def test_live_against_pyc_cpu_executor(oracle_lib):
    ref = oracle.ref_cpu(threads=4)
    for seed, (M, K, N) in enumerate([(7, 9, 11), (100, 130, 70), (256, 384, 192)]):
        a = workloads.uniform((M, K), 900 + seed); b = workloads.uniform((K, N), 950 + seed); c = workloads.uniform((M, N), 990 + seed)
        mod = ir.matmul_bias_act(abi.DTYPE_F32, M, K, N, bias="matrix", act="relu")
        model = ref.compile(mod, backend=abi.BACKEND_CPU, fusion=0)
        want, = ref.run(model, [(a, 1), (b, 1), (c, 1)], [((M, N), 1)])
        ref.destroy(model)
        got, = oracle_lib.run_module(mod, [(a, 1), (b, 1), (c, 1)], [((M, N), 1)])
        assert got.tobytes() == want.tobytes()


def test_bf16_rounding(oracle_lib):
    x = workloads.normal((4096,), 77)
    assert np.array_equal(workloads.to_bf16_bits(x), oracle.f32_to_bf16_bits(x))
    L = oracle_lib.lib
    for v in (0.0, 1.0, -1.0, 1.00390625, 3.1415927, 65504.0, 1e-30, -2.5e7):
        assert L.oracle_f32_to_bf16(v) == int(workloads.to_bf16_bits(np.array([v], np.float32))[0])
    # ties to even: 1 + 2^-8 is halfway between 1.0 (0x3F80) and 1.0078125 (0x3F81)
    assert L.oracle_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    assert L.oracle_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82


def test_f16_and_e4m3_round_trip(oracle_lib):
    L = oracle_lib.lib
    for h in list(range(0, 0x7C00, 97)) + [0x0001, 0x03FF, 0x0400, 0x7BFF]:
        assert L.oracle_f32_to_f16(L.oracle_f16_to_f32(h)) == h
    for v in range(256):
        f = L.oracle_e4m3_to_f32(v)
        if math.isnan(f):
            assert v & 0x7F == 0x7F
        else:
            assert L.oracle_f32_to_e4m3(f) == v or (f == 0.0 and v in (0x00, 0x80))
    assert L.oracle_e4m3_to_f32(0x7E) == 448.0 and L.oracle_f32_to_e4m3(1e6) == 0x7E


def test_unpinned_ops_match_numpy(oracle_lib):
    x = workloads.normal((37, 96), 5)
    erf = np.vectorize(math.erf)
    np.testing.assert_allclose(oracle_lib.gelu(x), 0.5 * x * (1 + erf(x / math.sqrt(2))), rtol=1e-6, atol=1e-7)
    mu = x.astype(np.float64).mean(-1, keepdims=True); var = x.astype(np.float64).var(-1, keepdims=True)
    np.testing.assert_allclose(oracle_lib.layernorm(x), (x - mu) / np.sqrt(var + 1e-5), rtol=1e-5, atol=1e-6)
    g = workloads.uniform((96,), 6); bt = workloads.uniform((96,), 7)
    np.testing.assert_allclose(oracle_lib.layernorm(x, g, bt), (x - mu) / np.sqrt(var + 1e-5) * g + bt, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(oracle_lib.reduce_sum(x), x.astype(np.float64).sum(-1), rtol=1e-6)
    e = np.exp(x - x.max(-1, keepdims=True))
    np.testing.assert_allclose(oracle_lib.softmax(x), e / e.sum(-1, keepdims=True), rtol=1e-5, atol=1e-7)


def test_attention_and_conv_definitions(oracle_lib):
    q = workloads.normal((3, 16, 8), 11); k = workloads.normal((3, 16, 8), 12); v = workloads.normal((3, 16, 8), 13)
    scale = 1 / math.sqrt(8)
    for causal in (False, True):
        s = np.einsum("bid,bjd->bij", q, k).astype(np.float64) * scale
        if causal:
            s = np.where(np.tril(np.ones((16, 16), bool)), s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
        np.testing.assert_allclose(oracle_lib.attention(q, k, v, scale, causal), p @ v, rtol=1e-5, atol=1e-6)
    x = workloads.uniform((2, 6, 5, 4), 21); w = workloads.uniform((3, 3, 3, 4), 22); b = workloads.uniform((3,), 23)
    xp = np.pad(x, ((0, 0), (1, 1), (1, 1), (0, 0)))
    want = np.zeros((2, 6, 5, 3), np.float64)
    for r in range(3):
        for s_ in range(3):
            want += np.einsum("nhwc,kc->nhwk", xp[:, r:r + 6, s_:s_ + 5, :], w[:, r, s_, :])
    want = np.maximum(want + b, 0)
    np.testing.assert_allclose(oracle_lib.conv2d(x, w, b, pad=(1, 1), stride=(1, 1), relu=True), want, rtol=1e-5, atol=1e-5)


def test_module_walk_rejects_what_pyc_rejects(oracle_lib):
    b = ir.ModuleBuilder()
    b._add(abi.OP_CONST, "c", abi.DTYPE_F32, [4])
    b.output(0)
    with pytest.raises(RuntimeError):
        oracle_lib.run_module(b.module, [], [((4,), abi.DTYPE_F32)])
    with pytest.raises(ValueError):  # ir.c:80-89: inputs must reference earlier ops
        ir.ModuleBuilder()._add(abi.OP_RELU, "r", abi.DTYPE_F32, [4], (0,))


def test_gelu_and_layernorm_definitions_agree_with_torch_fp64(oracle_lib):
    """The reference has no executor for GELU / LAYERNORM; its only semantic hint is torch.nn.GELU() / nn.LayerNorm(hidden) in its
    benchmark workloads (benchmark/benchmarks/gpu/workloads/standard_workload.py:58-62).  The oracle's definitions (exact-erf
    GELU; last axis, biased variance, eps 1e-5 inside the root, optional affine) are held to torch's fp64 results of those two
    modules.  This is the most the reference allows: conv2d, attention and fp8 stay unpinned."""
    import torch
    from pyc_b200 import workloads
    x = workloads.normal((37, 300), 4242, 3.0)
    g = torch.nn.functional.gelu(torch.from_numpy(x).double()).numpy()
    np.testing.assert_allclose(oracle_lib.gelu(x), g, rtol=2e-6, atol=2e-7)
    gamma, beta = workloads.normal((300,), 4243), workloads.normal((300,), 4244)
    ln = torch.nn.LayerNorm(300, eps=1e-5).double()
    with torch.no_grad():
        ln.weight.copy_(torch.from_numpy(gamma).double()); ln.bias.copy_(torch.from_numpy(beta).double())
        want_affine = ln(torch.from_numpy(x).double()).numpy()
        want_plain = torch.nn.functional.layer_norm(torch.from_numpy(x).double(), (300,), eps=1e-5).numpy()
    np.testing.assert_allclose(oracle_lib.layernorm(x, gamma, beta), want_affine, rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(oracle_lib.layernorm(x), want_plain, rtol=1e-5, atol=2e-6)


def test_attention_conv_softmax_and_e4m3_definitions_agree_with_torch(oracle_lib):
    """The reference holds nothing that pins attention (its kernel is an identity stub), conv2d (fp16-only CUTLASS
    instantiation), softmax (no executor) or fp8 (no dtype).  The oracle's restated definitions are therefore also held to
    an independent implementation: torch on the CPU in fp64 -- scaled_dot_product_attention with and without the causal
    mask, conv2d as cross-correlation on NHWC / KRSC data with symmetric padding and a stride, softmax over the last
    axis -- and torch's own float8_e4m3fn decoding for every one of the 256 codes."""
    import torch
    F = torch.nn.functional
    q = workloads.normal((2, 3, 40, 16), 31); k = workloads.normal((2, 3, 40, 16), 32); v = workloads.normal((2, 3, 40, 16), 33)
    scale = 1 / math.sqrt(16)
    for causal in (False, True):
        want = F.scaled_dot_product_attention(torch.from_numpy(q).double(), torch.from_numpy(k).double(), torch.from_numpy(v).double(),
                                              is_causal=causal, scale=scale).numpy()
        got = oracle_lib.attention(q.reshape(6, 40, 16), k.reshape(6, 40, 16), v.reshape(6, 40, 16), scale, causal).reshape(2, 3, 40, 16)
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    x = workloads.uniform((2, 9, 7, 8), 41); w = workloads.uniform((5, 3, 3, 8), 42); b = workloads.uniform((5,), 43)
    for pad, stride in (((1, 1), (1, 1)), ((0, 0), (1, 1)), ((1, 1), (2, 2)), ((2, 1), (1, 2))):
        want = F.conv2d(torch.from_numpy(x).double().permute(0, 3, 1, 2), torch.from_numpy(w).double().permute(0, 3, 1, 2),
                        torch.from_numpy(b).double(), stride=stride, padding=pad).permute(0, 2, 3, 1).numpy()
        np.testing.assert_allclose(oracle_lib.conv2d(x, w, b, pad=pad, stride=stride, relu=False), want, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(oracle_lib.conv2d(x, w, b, pad=pad, stride=stride, relu=True), np.maximum(want, 0), rtol=1e-5, atol=1e-5)
    s = workloads.normal((11, 257), 51, 4.0)
    np.testing.assert_allclose(oracle_lib.softmax(s), F.softmax(torch.from_numpy(s).double(), dim=-1).numpy(), rtol=1e-5, atol=1e-8)
    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    got = workloads.e4m3_decode(codes)
    finite = np.isfinite(want)                      # 0x7f / 0xff are NaN in e4m3fn; the encoder never produces them
    assert finite.sum() == 254
    np.testing.assert_array_equal(got[finite], want[finite])
    vals = workloads.normal((4096,), 61, 100.0)
    enc = torch.from_numpy(np.clip(vals, -448.0, 448.0)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.testing.assert_array_equal(workloads.e4m3_encode(vals), enc)     # round to nearest even, saturating at +-448


def test_ffn_block_definition_agrees_with_torch(oracle_lib):
    """The FFN block the fp8 kernels are held to (LayerNorm without affine, dequantised e4m3 weights with one scale per output
    channel, exact-erf GELU, fp32 contractions in PyC's summation order) against the same chain in torch fp64."""
    import torch
    import oracle
    F = torch.nn.functional
    tokens, hidden, inner = 24, 64, 256
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(tokens, hidden, inner)
    x = workloads.bf16_bits_to_f32(xb)
    got = oracle.ffn_reference(oracle_lib, x, w1, s1, w2, s2)
    deq = lambda codes, scale: torch.from_numpy(codes).view(torch.float8_e4m3fn).double() * torch.from_numpy(np.asarray(scale)).double()[None, :]
    h = F.gelu(F.layer_norm(torch.from_numpy(x).double(), (hidden,), eps=1e-5) @ deq(w1, s1))
    want = (h @ deq(w2, s2)).numpy()
    assert np.abs(got - want).max() / np.abs(want).max() <= 1e-5
