"""GPU parity: pyc_cuda_dispatch (the seam PyC's pyc_run_model calls) on whole IR
modules, host and device tensors, against the oracle's module walk; graph
capture/replay, arena reuse, env switches and reason strings."""
import os

import numpy as np
import pytest

from pyc_b200 import abi, ir, workloads

pytestmark = pytest.mark.gpu


def _host(arr, dtype):
    from pyc_b200 import backend
    return backend.make_tensor(arr.ctypes.data, arr.nbytes, dtype, arr.shape)


def run_module_both(backend, oracle_lib, module, arrays, dtype, out_shape, device):
    """arrays: fp32 inputs.  Returns (gpu result widened to fp32, oracle result, trace)."""
    from gpu_util import dev_tensor, empty_device, round_to, to_device, to_host_f32
    stor = [round_to(dtype, a) for a in arrays]
    want, = oracle_lib.run_module(module, [(s, dtype) for s, _ in stor], [(out_shape, abi.DTYPE_F32 if dtype == abi.DTYPE_F32 else dtype)])
    if dtype != abi.DTYPE_F32:
        want = workloads.bf16_bits_to_f32(want) if dtype == abi.DTYPE_BF16 else want.view(np.float16).astype(np.float32)
    if device:
        d_in = [to_device(s) for s, _ in stor]; d_out = empty_device(dtype, out_shape)
        st, trace = backend.dispatch(module, [dev_tensor(t, dtype) for t in d_in], [dev_tensor(d_out, dtype)])
        got = to_host_f32(dtype, d_out)
    else:
        h_in = [np.ascontiguousarray(s) for s, _ in stor]
        h_out = np.zeros(out_shape, np.float32 if dtype == abi.DTYPE_F32 else np.uint16)
        st, trace = backend.dispatch(module, [_host(a, dtype) for a in h_in], [_host(h_out, dtype)])
        got = h_out if dtype == abi.DTYPE_F32 else (workloads.bf16_bits_to_f32(h_out) if dtype == abi.DTYPE_BF16 else h_out.view(np.float16).astype(np.float32))
    return got, want, trace


def test_kat_row_bias_relu_host_tensors_and_replay(backend, oracle_lib):
    # PyC's known-answer case, tests/compiler_next/test_cuda_backend.c:84-89, run twice (second = graph replay).
    lhs = np.array([[1, -2], [3, 4]], np.float32); rhs = np.array([[2, 1], [-1, 3]], np.float32); bias = np.array([0.5, -1.5], np.float32)
    mod = ir.matmul_bias_act(abi.DTYPE_F32, 2, 2, 2, bias="row", act="relu")
    out = np.zeros((2, 2), np.float32)
    reasons = []
    for _ in range(2):
        out[:] = 0
        st, trace = backend.dispatch(mod, [_host(lhs, 1), _host(rhs, 1), _host(bias, 1)], [_host(out, 1)])
        assert st == abi.DISPATCH_OK and trace.fallback_to_cpu == 0
        np.testing.assert_allclose(out.reshape(-1), [4.5, 0.0, 2.5, 13.5], atol=1e-5)
        reasons.append(trace.reason.decode())
    assert reasons[0].startswith("b200_graph_capture:b200_gemm_f32_") and reasons[1].startswith("b200_graph_replay:b200_gemm_f32_")
    assert backend.runtime_info().kernels_per_graph == 1  # matmul + bias + relu fused into one kernel


def test_passthrough_is_byte_exact(backend, oracle_lib):
    bits = np.array([0x3F80, 0x4000, 0x4040, 0x4080], np.uint16); got = np.zeros(4, np.uint16)
    b = ir.ModuleBuilder(); b.output(b.input("input0", abi.DTYPE_BF16, [4]))
    st, trace = backend.dispatch(b.module, [_host(bits, abi.DTYPE_BF16)], [_host(got, abi.DTYPE_BF16)])
    assert st == abi.DISPATCH_OK and got.tolist() == bits.tolist()
    x = workloads.normal((1000,), 3); y = np.zeros(1000, np.float32)
    b = ir.ModuleBuilder(); b.output(b.input("x", abi.DTYPE_F32, [1000]))
    backend.dispatch(b.module, [_host(x, 1)], [_host(y, 1)])
    assert x.tobytes() == y.tobytes()


@pytest.mark.parametrize("device", [False, True])
@pytest.mark.parametrize("dtype,tol", [(abi.DTYPE_F32, 1e-5), (abi.DTYPE_BF16, 2e-2)])
@pytest.mark.parametrize("bias,act", [("row", "relu"), ("row", "gelu"), ("matrix", None), ("scalar", "relu"), (None, None)])
def test_matmul_chains(backend, oracle_lib, device, dtype, tol, bias, act):
    from gpu_util import rel_err
    M, K, N = 192, 256, 320
    mod = ir.matmul_bias_act(dtype, M, K, N, bias=bias, act=act)
    arrays = [workloads.normal((M, K), 71, 0.5), workloads.normal((K, N), 72, 0.5)]
    if bias:
        arrays.append(workloads.normal({"row": (N,), "matrix": (M, N), "scalar": (1,)}[bias], 73, 2.0))
    got, want, trace = run_module_both(backend, oracle_lib, mod, arrays, dtype, (M, N), device)
    assert rel_err(got, want) <= tol
    assert trace.reason.decode().startswith("b200_graph_")


def test_large_f32_module_is_planned_on_the_packed_fma_tile_and_replays(backend, oracle_lib):
    # large enough for the wave model to prefer the 128 x 128 fp32 tile; first call captures the graph (with the kernel's
    # shared-memory opt-in inside the capture), second replays it
    from gpu_util import rel_err
    M, K, N = 2048, 384, 2304
    mod = ir.matmul_bias_act(abi.DTYPE_F32, M, K, N, bias="row", act="gelu")
    arrays = [workloads.normal((M, K), 81, 0.5), workloads.normal((K, N), 82, 0.5), workloads.normal((N,), 83, 2.0)]
    for want_reason in ("b200_graph_capture:", "b200_graph_replay:"):
        got, want, trace = run_module_both(backend, oracle_lib, mod, arrays, abi.DTYPE_F32, (M, N), True)
        assert rel_err(got, want) <= 1e-5
        assert trace.reason.decode() == want_reason + "b200_gemm_f32_simt_x2_128x128x32"


@pytest.mark.parametrize("dtype,tol", [(abi.DTYPE_F32, 1e-5), (abi.DTYPE_BF16, 2e-2)])
def test_ffn_like_module_with_arena_reuse(backend, oracle_lib, dtype, tol):
    # layernorm -> matmul -> +bias -> gelu -> matmul -> +bias -> (+ residual) -> reduce_sum as second output
    from gpu_util import dev_tensor, empty_device, rel_err, round_to, to_device, to_host_f32
    T, H, I = 256, 128, 512
    b = ir.ModuleBuilder()
    x = b.input("x", dtype, [T, H]); w1 = b.input("w1", dtype, [H, I]); b1 = b.input("b1", dtype, [I])
    w2 = b.input("w2", dtype, [I, H]); b2 = b.input("b2", dtype, [H])
    h = b.gelu(b.add(b.matmul(b.layernorm(x), w1), b1))
    y = b.add(b.add(b.matmul(h, w2), b2), x)
    b.output(y); b.output(b.reduce_sum(y))
    arrays = [workloads.normal((T, H), 81), workloads.normal((H, I), 82, H ** -0.5), workloads.normal((I,), 83, 0.1),
              workloads.normal((I, H), 84, I ** -0.5), workloads.normal((H,), 85, 0.1)]
    stor = [round_to(dtype, a) for a in arrays]
    odt = dtype
    want_y, want_s = oracle_lib.run_module(b.module, [(s, dtype) for s, _ in stor], [((T, H), odt), ((T,), odt)])
    if dtype == abi.DTYPE_BF16:
        want_y, want_s = workloads.bf16_bits_to_f32(want_y), workloads.bf16_bits_to_f32(want_s)
    d_in = [to_device(s) for s, _ in stor]; d_y = empty_device(dtype, (T, H)); d_s = empty_device(dtype, (T,))
    for _ in range(2):
        st, trace = backend.dispatch(b.module, [dev_tensor(t, dtype) for t in d_in], [dev_tensor(d_y, dtype), dev_tensor(d_s, dtype)])
    assert trace.graph_replayed == 1
    assert rel_err(to_host_f32(dtype, d_y), want_y) <= tol
    assert np.abs(to_host_f32(dtype, d_s) - want_s).max() <= (tol * 4) * np.abs(want_y).sum(-1).max()
    info = backend.runtime_info()
    assert info.kernels_per_graph == 5           # ln, gemm+bias+gelu, gemm+bias, add, reduce_sum
    assert info.plan_peak_bytes < info.plan_total_bytes  # lifetimes let buffers share arena offsets


def test_env_switches_on_a_real_device(backend, oracle_lib):
    lhs = workloads.normal((64, 64), 91); rhs = workloads.normal((64, 64), 92); out = np.zeros((64, 64), np.float32)
    mod = ir.matmul_bias_act(abi.DTYPE_F32, 64, 64, 64, bias=None, act=None)
    ins, outs = [_host(lhs, 1), _host(rhs, 1)], [_host(out, 1)]
    try:
        os.environ["PYC_CUDA_FORCE_ERROR"] = "1"
        st, trace = backend.dispatch(mod, ins, outs, require_gpu=False)
        assert st == abi.DISPATCH_ERROR and trace.reason == b"forced_error"
        os.environ["PYC_CUDA_FORCE_ERROR"] = "0"
        os.environ["PYC_CUDA_ENABLE_GRAPH_REPLAY"] = "0"
        st, trace = backend.dispatch(mod, ins, outs)
        assert trace.reason.decode().startswith("b200_stream:") and trace.graph_replayed == 0
        os.environ["PYC_CUDA_ENABLE_GRAPH_REPLAY"] = "1"
        os.environ["PYC_CUDA_ASSUME_STATIC_RHS"] = "1"
        # fresh buffers and a shape nothing has used yet: the FIRST run must upload the RHS, later runs may skip it
        lhs2 = workloads.normal((80, 96), 93); rhs2 = workloads.normal((96, 72), 94); out2 = np.zeros((80, 72), np.float32)
        mod2 = ir.matmul_bias_act(abi.DTYPE_F32, 80, 96, 72, bias=None, act=None)
        ins2, outs2 = [_host(lhs2, 1), _host(rhs2, 1)], [_host(out2, 1)]
        scale = np.abs(oracle_lib.matmul(lhs2, rhs2)).max()
        for i in range(3):  # LHS changes every run, RHS is static
            lhs2[:] = workloads.normal((80, 96), 100 + i)
            out2[:] = 0
            backend.dispatch(mod2, ins2, outs2)
            np.testing.assert_allclose(out2, oracle_lib.matmul(lhs2, rhs2), rtol=0, atol=1e-5 * scale)
    finally:
        for k in ["PYC_CUDA_FORCE_ERROR", "PYC_CUDA_ENABLE_GRAPH_REPLAY", "PYC_CUDA_ASSUME_STATIC_RHS"]:
            os.environ.pop(k, None)


def test_unsupported_module_uses_callers_executor_and_says_so(backend):
    b = ir.ModuleBuilder()
    b._add(abi.OP_CONST, "c", abi.DTYPE_F32, [4]); b.output(0)
    out = np.zeros(4, np.float32); calls = []

    @abi.CPU_EXECUTOR_FN
    def executor(module, inputs, n_in, outputs, n_out, ctx):
        calls.append(1); return 0

    st, trace = backend.dispatch(b.module, [_host(out, 1)], [_host(out, 1)], cpu_executor=executor, require_gpu=False)
    assert st == abi.DISPATCH_FALLBACK and trace.fallback_to_cpu == 1 and trace.reason == b"cuda_native_unsupported_fallback" and calls


def test_hardware_family_and_autotune_feed_registry(backend):
    assert backend.load().pyc_cuda_current_hardware_family() == 3  # B200 reports PyC's highest family (hopper)
    sym, ms, n = backend.autotune_gemm(abi.DTYPE_BF16, 1024, 1024, 1024, iters=3)
    assert sym.startswith("b200_gemm_bf16_tc_") and ms > 0 and n >= 3


def test_dispatch_autotunes_on_first_sight_when_asked(backend, oracle_lib, monkeypatch):
    # PYC_B200_AUTOTUNE=1: the tile configuration that goes into the graph is the measured winner for this shape
    from gpu_util import rel_err
    monkeypatch.setenv("PYC_B200_AUTOTUNE", "1")
    M, K, N = 768, 1024, 1280
    mod = ir.matmul_bias_act(abi.DTYPE_BF16, M, K, N, bias="row", act="relu")
    arrays = [workloads.normal((M, K), 111, 0.5), workloads.normal((K, N), 112, 0.5), workloads.normal((N,), 113, 2.0)]
    got, want, trace = run_module_both(backend, oracle_lib, mod, arrays, abi.DTYPE_BF16, (M, N), True)
    assert rel_err(got, want) <= 2e-2
    assert "b200_gemm_bf16_tc" in trace.reason.decode()
    sym, ms, n = backend.autotune_gemm(abi.DTYPE_BF16, M, N, K, iters=2)   # same shape again: consistent answer format
    assert sym.startswith("b200_gemm_bf16_") and n >= 4


def test_pinned_host_tensors_take_the_pipelined_path_and_match(backend, oracle_lib):
    # Large pinned host operands: A goes up in row chunks, each chunk's GEMM and download overlap the next upload.
    # Ragged on purpose (2100 rows = four 512-row chunks + 52).  Checked against the serial order of the same
    # call (PYC_B200_PIPELINE_HOST_COPIES=0), against the oracle on rows around every chunk edge, under graph
    # capture, graph replay (with new A contents) and on a plain stream.
    import torch
    M, K, N = 2100, 4096, 4096
    dtype = abi.DTYPE_BF16
    mod = ir.matmul_bias_act(dtype, M, K, N, bias="row", act="gelu")
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).pin_memory()
    a_bits = [workloads.to_bf16_bits(workloads.normal((M, K), 300 + i)) for i in range(2)]
    b_bits = workloads.to_bf16_bits(workloads.normal((K, N), 310) * np.float32(K ** -0.5))
    bias_bits = workloads.to_bf16_bits(workloads.normal((N,), 311))
    A, B, bias = pin(a_bits[0]), pin(b_bits), pin(bias_bits)
    out = torch.zeros((M, N), dtype=torch.int16).pin_memory()
    T = lambda t, shape: backend.make_tensor(t.data_ptr(), t.numel() * 2, dtype, shape)
    ins, outs = [T(A, (M, K)), T(B, (K, N)), T(bias, (N,))], [T(out, (M, N))]
    rows = sorted(set(list(range(0, 8)) + [r for e in (512, 1024, 1536, 2048) for r in range(e - 4, e + 4)] + list(range(M - 8, M))))
    b_f32, bias_f32 = workloads.bf16_bits_to_f32(b_bits), workloads.bf16_bits_to_f32(bias_bits)

    def check(which):
        got = workloads.bf16_bits_to_f32(out.numpy().view(np.uint16)[rows])
        a_f32 = workloads.bf16_bits_to_f32(a_bits[which][rows])
        want = oracle_lib.gelu(oracle_lib.add(oracle_lib.matmul(a_f32, b_f32), bias_f32))
        err = np.abs(got - want).max() / np.abs(want).max()
        assert err < 2e-2, err   # bf16 storage tolerance

    results = {}
    try:
        for mode, env in (("serial", {"PYC_B200_PIPELINE_HOST_COPIES": "0"}), ("pipelined", {}),
                          ("pipelined_stream", {"PYC_CUDA_ENABLE_GRAPH_REPLAY": "0"})):
            os.environ.update(env)
            for run in range(2 if mode == "pipelined" else 1):
                A.numpy()[:] = a_bits[run].view(np.int16)
                out.zero_()
                st, trace = backend.dispatch(mod, ins, outs)
                assert st == abi.DISPATCH_OK and trace.fallback_to_cpu == 0
                check(run)
                results[(mode, run)] = out.numpy().copy()
                if mode == "pipelined":
                    assert trace.graph_replayed == run
                    assert backend.runtime_info().kernels_per_graph == 5   # one GEMM per chunk
                if mode == "serial":
                    assert backend.runtime_info().kernels_per_graph == 1
            for k in env:
                os.environ.pop(k, None)
    finally:
        for k in ("PYC_B200_PIPELINE_HOST_COPIES", "PYC_CUDA_ENABLE_GRAPH_REPLAY"):
            os.environ.pop(k, None)
    # chunking only changes which CTA computes a row, not the arithmetic of the row
    serial = workloads.bf16_bits_to_f32(results[("serial", 0)].view(np.uint16))
    for key in (("pipelined", 0), ("pipelined_stream", 0)):
        piped = workloads.bf16_bits_to_f32(results[key].view(np.uint16))
        assert np.abs(piped - serial).max() <= 2e-2 * np.abs(serial).max()


def test_a_wait_that_runs_out_is_reported_not_hung(backend):
    """A kernel's bounded wait on a barrier nobody arrives at gives up by itself (about 50 us here), the kernel returns, and the
    host sees where: the status word carries (site << 8) | 1.  A dispatch that finds the word set reports
    b200_kernel_wait_timeout as an ERROR (never a CPU fallback), clears it, and the next dispatch is fine again."""
    import torch
    torch.cuda.synchronize()
    assert backend.device_status() == 0
    backend.selftest_wait_timeout(50)
    torch.cuda.synchronize()
    assert backend.device_status() == (0x7f << 8) | 1
    assert backend.device_status() == 0                      # read-and-clear
    lhs = np.array([[1, -2], [3, 4]], np.float32); rhs = np.array([[2, 1], [-1, 3]], np.float32); bias = np.array([0.5, -1.5], np.float32)
    mod = ir.matmul_bias_act(abi.DTYPE_F32, 2, 2, 2, bias="row", act="relu")
    out = np.zeros((2, 2), np.float32)
    arrays = [lhs, rhs, bias]
    _host_tensors = lambda arrs: [_host(a, 1) for a in arrs]
    backend.selftest_wait_timeout(50)
    torch.cuda.synchronize()
    st, trace = backend.dispatch(mod, _host_tensors(arrays), _host_tensors([out]), require_gpu=False)
    assert st == abi.DISPATCH_ERROR and trace.fallback_to_cpu == 0
    assert trace.reason.decode() == "b200_kernel_wait_timeout:0x7f01"
    st, trace = backend.dispatch(mod, _host_tensors(arrays), _host_tensors([out]))
    assert st == abi.DISPATCH_OK
    np.testing.assert_allclose(out.reshape(-1), [4.5, 0.0, 2.5, 13.5], atol=1e-5)
