"""Build libpyc_b200.so in-tree with nvcc for sm_100a.

    python -m pyc_b200.build            # compile (only files that changed)
    python -m pyc_b200.build --verbose  # also print ptxas resource usage
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libpyc_b200.so")
COMM_SRC = os.path.join(HERE, "csrc_comm", "comm_nccl.cpp")
COMM_LIB = os.path.join(HERE, "libpyc_b200_comm_nccl.so")   # NCCL backend for PyC's collective interface (loaded by path)

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
          f"-I{INCLUDE}", f"-I{CSRC}", "-DPYC_B200_BUILD"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _stale(src, obj):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)] + [src]
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(name, verbose):
    src = os.path.join(CSRC, name)
    obj = os.path.join(OBJ, os.path.splitext(name)[0] + ".o")
    if not _stale(src, obj):
        return obj, ""
    cmd = [NVCC, *ARCH, *COMMON, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        results = list(ex.map(lambda n: _compile(n, verbose), sources()))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-cudart", "static", "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    deps = [COMM_SRC] + [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    if not os.path.exists(COMM_LIB) or any(os.path.getmtime(d) > os.path.getmtime(COMM_LIB) for d in deps):
        cmd = [NVCC, "-O2", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden", f"-I{INCLUDE}", "-shared", "-o", COMM_LIB, COMM_SRC,
               "-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"comm backend build failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv))
