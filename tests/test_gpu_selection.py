"""GPU: who chooses the GEMM tile configuration, and that the backend says truthfully what ran.

  * through PyC's unmodified front half (pyc_run_model): PyC's registry scoring makes the choice ("[registry]"), the
    sidecar plan names the kernel and the IR ops it absorbed, and it agrees with the kernel named in PyC's decision log;
  * a symbol promoted in PyC's registry, PYC_CUDA_BF16_GEMM_SYMBOL and PYC_CUDA_ENABLE_PROMOTED_GEMM=0 steer it;
  * autotune results persist in PyC's DB format and steer a fresh process."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import oracle
from pyc_b200 import abi, ir, workloads

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
needs_front = pytest.mark.skipif(not os.path.exists(oracle.REF_FRONT_SO), reason="PyC's front half was not built (no PyC checkout at build time)")


def _bf16_problem(M, K, N, seed=900):
    bits = [workloads.to_bf16_bits(workloads.normal(s, seed + i, 0.05)) for i, s in enumerate(((M, K), (K, N), (N,)))]
    return bits, [workloads.bf16_bits_to_f32(b) for b in bits]


@needs_front
def test_front_half_run_is_chosen_by_pycs_registry_and_the_plan_says_what_ran(backend, oracle_lib):
    front = oracle.RefRuntime(oracle.REF_FRONT_SO, threads=4)
    M, K, N = 2048, 1024, 2048                      # PyC's "large_square" class -> the CTA-pair tile is the registry's pick
    bits, vals = _bf16_problem(M, K, N)
    mod = ir.matmul_bias_act(abi.DTYPE_BF16, M, K, N, bias="row", act="gelu")
    model = front.compile(mod, backend=abi.BACKEND_CUDA, fusion=0)
    for _ in range(2):
        out, = front.run(model, [(t, abi.DTYPE_BF16) for t in bits], [((M, N), abi.DTYPE_BF16)])
    log = front.decision_log(model)
    ran = re.search(r"b200_graph_(?:capture|replay):(b200_gemm_\w+)", log)
    assert ran, log
    plan = backend.last_plan(mod)
    assert plan is not None
    gemm_lines = [l for l in plan.splitlines() if "b200_gemm_" in l]
    assert len(gemm_lines) == 1
    m = re.match(r"step \d+: (b200_gemm_\w+) \[(\w+)\] <- matmul#2 \+ add#4 \+ gelu#5", gemm_lines[0])
    assert m, plan
    assert m.group(1) == ran.group(1) == "b200_gemm_bf16_tc2_256x256x64_s6"     # the plan, PyC's log and the registry's pick agree
    assert m.group(2) == "registry"
    assert "copy_h2d <- input#0" in plan and "copy_d2h <- output#6" in plan
    want = oracle_lib.gelu(oracle_lib.add(oracle_lib.matmul(vals[0], vals[1]), vals[2]))
    assert np.abs(workloads.bf16_bits_to_f32(out) - want).max() / np.abs(want).max() <= 2e-2
    # a promotion made through PyC's registry changes the kernel of the next run (new graph), and is reported as such
    L = front.lib
    L.pyc_kernel_promote_symbol.argtypes = [__import__("ctypes").c_char_p, __import__("ctypes").c_int, __import__("ctypes").c_char_p]
    try:
        assert L.pyc_kernel_promote_symbol(b"matmul", 1, b"b200_gemm_bf16_tc_128x256x64_s4") == 0
        out2, = front.run(model, [(t, abi.DTYPE_BF16) for t in bits], [((M, N), abi.DTYPE_BF16)])
        assert "b200_graph_capture:b200_gemm_bf16_tc_128x256x64_s4" in front.decision_log(model)
        assert "b200_gemm_bf16_tc_128x256x64_s4 [promoted]" in backend.last_plan(mod)
        assert np.abs(workloads.bf16_bits_to_f32(out2) - want).max() / np.abs(want).max() <= 2e-2
        os.environ["PYC_CUDA_ENABLE_PROMOTED_GEMM"] = "0"          # PyC's switch, off: the promotion is ignored again
        front.run(model, [(t, abi.DTYPE_BF16) for t in bits], [((M, N), abi.DTYPE_BF16)])
        assert "b200_gemm_bf16_tc2_256x256x64_s6 [registry]" in backend.last_plan(mod)
    finally:
        os.environ.pop("PYC_CUDA_ENABLE_PROMOTED_GEMM", None)
        L.pyc_kernel_promote_symbol(b"matmul", 1, b"")
    front.destroy(model)


def test_env_symbol_and_model_choice_without_pycs_registry(backend, oracle_lib, monkeypatch):
    # stand-alone (PyC's registry may or may not be in the process): PYC_CUDA_BF16_GEMM_SYMBOL wins over registry and model
    from test_gpu_dispatch import run_module_both
    from gpu_util import rel_err
    M, K, N = 640, 512, 768
    mod = ir.matmul_bias_act(abi.DTYPE_BF16, M, K, N, bias="row", act="relu")
    arrays = [workloads.normal((M, K), 121, 0.5), workloads.normal((K, N), 122, 0.5), workloads.normal((N,), 123, 2.0)]
    monkeypatch.setenv("PYC_CUDA_BF16_GEMM_SYMBOL", "b200_gemm_bf16_tc_128x128x64_s6")
    got, want, trace = run_module_both(backend, oracle_lib, mod, arrays, abi.DTYPE_BF16, (M, N), True)
    assert rel_err(got, want) <= 2e-2
    assert trace.reason.decode().endswith(":b200_gemm_bf16_tc_128x128x64_s6")
    assert "b200_gemm_bf16_tc_128x128x64_s6 [env]" in backend.last_plan(mod)
    monkeypatch.setenv("PYC_CUDA_BF16_GEMM_SYMBOL", "cutlass_gemm_tensorcore_bf16")    # PyC's default name: no constraint
    monkeypatch.setenv("PYC_B200_REGISTRY_SELECT", "0")
    got, want, trace = run_module_both(backend, oracle_lib, mod, arrays, abi.DTYPE_BF16, (M, N), True)
    assert rel_err(got, want) <= 2e-2
    assert "[model]" in backend.last_plan(mod)


def test_autotune_persists_in_pycs_db_format_and_steers_a_fresh_process(backend, tmp_path, monkeypatch):
    db = tmp_path / "autotune.db"
    monkeypatch.setenv("PYC_AUTOTUNE_DB_PATH", str(db))
    M, N, K = 1024, 768, 512
    sym, ms, n = backend.autotune_gemm(abi.DTYPE_BF16, M, N, K, iters=5)
    assert n >= 4 and ms > 0
    lines = db.read_text().splitlines()
    per_symbol = [l for l in lines if l.startswith("matmul|1|")]
    per_shape = [l for l in lines if l.startswith(f"matmul@bf16:{M}x{N}x{K}|1|")]
    assert len(per_symbol) == n and len(per_shape) == n
    assert all(re.fullmatch(r"[^|]+\|1\|b200_gemm_bf16_\w+\|\d+\.\d{6}", l) for l in per_symbol + per_shape)
    best = min(per_shape, key=lambda l: float(l.rsplit("|", 1)[1]))
    assert best.split("|")[2] == sym
    assert os.path.exists(str(db) + ".lock")
    # Make a DIFFERENT symbol the fastest on file, then let a fresh process (which tunes nothing) run that shape.
    other = "b200_gemm_bf16_tc_128x64x64_s8" if not sym.endswith("tc_128x64x64_s8") else "b200_gemm_bf16_tc_128x128x64_s6"
    with open(db, "a") as f:
        f.write(f"matmul@bf16:{M}x{N}x{K}|1|{other}|0.000100\n")
    code = f"""
import numpy as np, torch, sys
sys.path.insert(0, {ROOT!r})
from pyc_b200 import abi, backend, ir
backend.load()
M, N, K = {M}, {N}, {K}
mod = ir.matmul_bias_act(abi.DTYPE_BF16, M, K, N, bias=None, act=None)
a = torch.zeros((M, K), dtype=torch.int16, device="cuda"); b = torch.zeros((K, N), dtype=torch.int16, device="cuda"); o = torch.zeros((M, N), dtype=torch.int16, device="cuda")
T = lambda t: backend.make_tensor(t.data_ptr(), t.numel() * 2, abi.DTYPE_BF16, tuple(t.shape))
st, trace = backend.dispatch(mod, [T(a), T(b)], [T(o)])
print("REASON", trace.reason.decode()); print(backend.last_plan(mod))
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=dict(os.environ))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert f"REASON b200_graph_capture:{other}" in r.stdout, r.stdout
    assert f"{other} [autotune]" in r.stdout, r.stdout
