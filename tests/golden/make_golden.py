"""Regenerate tests/golden/ref_cpu_cases.npz from PyC's own CPU executor.

Needs a PyC checkout (PYC_REFERENCE_DIR, default: a `reference` directory next to this repository) and `make -C oracle ref`.  Each
case is a small IR module run through pyc_compile_model / pyc_run_model of the
UNMODIFIED PyC sources with backend CPU, fusion off, fp32 tensors and the bias
materialised to [M,N] (PyC's CPU ADD has no broadcast,
src/compiler/compiler_api.c:1974-2014).  Inputs are regenerated from seeds by
the tests; only PyC's outputs are stored.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from pyc_b200 import abi, ir, workloads  # noqa: E402

# (name, M, K, N, bias, act)
CASES = [
    ("mm_8x3x5", 8, 3, 5, None, None),
    ("mm_64x48x40", 64, 48, 40, None, None),
    ("mm_add_relu_33x65x17", 33, 65, 17, "matrix", "relu"),
    ("mm_add_96x128x72", 96, 128, 72, "matrix", None),
    ("mm_relu_128x256x64", 128, 256, 64, None, "relu"),
    ("mm_add_relu_256x512x128", 256, 512, 128, "matrix", "relu"),
]


def case_inputs(idx, M, K, N, bias):
    a = workloads.uniform((M, K), workloads.tensor_seed(100 + idx, 0))
    b = workloads.uniform((K, N), workloads.tensor_seed(100 + idx, 1))
    c = workloads.uniform((M, N), workloads.tensor_seed(100 + idx, 2)) if bias else None
    return a, b, c


def main():
    oracle.build()
    ref = oracle.ref_cpu(threads=4)
    out = {}
    for idx, (name, M, K, N, bias, act) in enumerate(CASES):
        a, b, c = case_inputs(idx, M, K, N, bias)
        mod = ir.matmul_bias_act(abi.DTYPE_F32, M, K, N, bias=bias, act=act)
        model = ref.compile(mod, backend=abi.BACKEND_CPU, fusion=0)
        ins = [(a, abi.DTYPE_F32), (b, abi.DTYPE_F32)] + ([(c, abi.DTYPE_F32)] if bias else [])
        res, = ref.run(model, ins, [((M, N), abi.DTYPE_F32)])
        ref.destroy(model)
        out[name] = res
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cpu_cases.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
