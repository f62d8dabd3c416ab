"""GPU: the whole drop-in path.  PyC's unmodified front half (pyc_compile_model /
pyc_run_model, compiled from PyC's sources into oracle/_ref/libpyc_ref_front.so)
calls this library's pyc_cuda_dispatch with backend = CUDA; results are checked
against the oracle, and PyC's own decision log must say the GPU ran it.
Also: PyC's own C tests for the seam, run on the GPU box."""
import glob
import os
import subprocess

import numpy as np
import pytest

import oracle
from pyc_b200 import abi, ir, workloads

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(oracle.REF_FRONT_SO), reason="PyC's front half was not built (no PyC checkout at build time)")]


@pytest.fixture(scope="module")
def front():
    return oracle.RefRuntime(oracle.REF_FRONT_SO, threads=4)


@pytest.mark.parametrize("bias,act", [("row", "relu"), (None, None), ("matrix", "relu")])
def test_pyc_run_model_on_cuda_backend_f32(front, oracle_lib, bias, act):
    M, K, N = 512, 512, 512   # benchmark configuration 1 shape
    x, w, b = workloads.gemm_inputs(1, M, K, N, ("uniform", -1.0, 1.0))
    if bias == "matrix":
        b = workloads.uniform((M, N), 77)
    mod = ir.matmul_bias_act(abi.DTYPE_F32, M, K, N, bias=bias, act=act)
    # PyC switches its lossy fusion pass off for the CUDA backend by itself (compiler_api.c:2484-2488); ask for it anyway.
    model = front.compile(mod, backend=abi.BACKEND_CUDA, fusion=1)
    ins = [(x, 1), (w, 1)] + ([(b, 1)] if bias else [])
    for run in range(3):
        out, = front.run(model, ins, [((M, N), 1)])
        log = front.decision_log(model)
        assert "cuda_fallback=0" in log, log
        assert "b200_graph_" in log, log
    want = oracle_lib.matmul(x, w)
    if bias:
        want = oracle_lib.add(want, b)
    if act:
        want = oracle_lib.relu(want)
    assert np.abs(out - want).max() / np.abs(want).max() <= 1e-5
    front.destroy(model)


def test_pyc_run_model_bf16_gelu_chain(front, oracle_lib):
    # A graph PyC's own GPU path rejects (GELU, bf16 with an ADD): here it runs fused on the tensor cores.
    M, K, N = 256, 512, 384
    a, b, bias = workloads.gemm_inputs(2, M, K, N, ("normal", 0.05))
    bits = [workloads.to_bf16_bits(t) for t in (a, b, bias)]
    vals = [workloads.bf16_bits_to_f32(t) for t in bits]
    mod = ir.matmul_bias_act(abi.DTYPE_BF16, M, K, N, bias="row", act="gelu")
    model = front.compile(mod, backend=abi.BACKEND_CUDA, fusion=0)
    out, = front.run(model, [(t, abi.DTYPE_BF16) for t in bits], [((M, N), abi.DTYPE_BF16)])
    log = front.decision_log(model)
    assert "cuda_fallback=0" in log and "b200_gemm_bf16_tc_" in log, log
    want = oracle_lib.gelu(oracle_lib.add(oracle_lib.matmul(vals[0], vals[1]), vals[2]))
    got = workloads.bf16_bits_to_f32(out)
    assert np.abs(got - want).max() / np.abs(want).max() <= 2e-2
    front.destroy(model)


BINARIES = sorted(glob.glob(os.path.join(os.path.dirname(oracle.REF_FRONT_SO), "ctest_*")))


@pytest.mark.parametrize("path", BINARIES, ids=[os.path.basename(p) for p in BINARIES])
def test_pyc_ctest_on_the_gpu(path, tmp_path):
    root_file = os.path.join(os.path.dirname(path), "ref_root.txt")
    if path.endswith("test_pass_golden") and os.path.exists(root_file) and not os.path.isdir(open(root_file).read().strip()):
        pytest.skip("PyC's source tree (golden file) is not on this machine")
    env = dict(os.environ)
    env["PYC_AUTOTUNE_DB_PATH"] = str(tmp_path / "autotune.db")
    r = subprocess.run([path], cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, f"{os.path.basename(path)} exited {r.returncode}\n{r.stdout[-2000:]}\n{r.stderr[-2000:]}"
