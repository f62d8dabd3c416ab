"""TEST INFRASTRUCTURE ONLY -- Python access to the CPU checkers.

`Oracle` wraps oracle/_build/libpyc_oracle.so (pyc_oracle.c, the restatement).
`RefCpu` wraps oracle/_ref/libpyc_ref_cpu.so, PyC's own compiler-next runtime
compiled CPU-only from PyC's sources by oracle/Makefile (`make ref`), driven the
way PyC's tests drive it: backend CPU, fusion off, fp32 tensors
(tests/compiler_next/test_cpu_execution.c:86-93).

Only tests/, the smoke check and the benchmark's CPU-baseline legs import this
package.  The product (pyc_b200/) never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from pyc_b200 import abi

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "libpyc_oracle.so")
REF_CPU_SO = os.path.join(_HERE, "_ref", "libpyc_ref_cpu.so")
REF_FRONT_SO = os.path.join(_HERE, "_ref", "libpyc_ref_front.so")

F32, BF16, F16 = 0, 1, 2


def build(ref_root=None):
    """Compile the restatement and, if a PyC checkout is present, PyC's own CPU runtime."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    ref_root = ref_root or os.environ.get("PYC_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if os.path.isdir(os.path.join(ref_root, "src", "compiler")):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"], check=True)


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (numpy, vectorised)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (u + (0x7FFF + ((u >> 16) & 1))) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class Oracle:
    def __init__(self, threads=None):
        if not os.path.exists(ORACLE_SO):
            build()
        L = self.lib = C.CDLL(ORACLE_SO)
        fp, sz, i = C.POINTER(C.c_float), C.c_size_t, C.c_int
        L.oracle_matmul_f32.argtypes = [fp, fp, fp, sz, sz, sz]
        L.oracle_add.argtypes = [fp, fp, fp, sz]
        L.oracle_add_row_bias.argtypes = [fp, fp, fp, sz, sz]
        L.oracle_add_scalar.argtypes = [fp, C.c_float, fp, sz]
        L.oracle_relu.argtypes = [fp, fp, sz]
        L.oracle_gelu.argtypes = [fp, fp, sz]
        L.oracle_layernorm.argtypes = [fp, fp, fp, fp, sz, sz, C.c_float]
        L.oracle_reduce_sum.argtypes = [fp, fp, sz, sz]
        L.oracle_softmax.argtypes = [fp, fp, sz, sz]
        L.oracle_attention.argtypes = [fp, fp, fp, fp, i, i, i, C.c_float, i]
        L.oracle_conv2d_nhwc.argtypes = [fp, fp, fp, fp] + [i] * 12
        L.oracle_run_module.argtypes = [C.POINTER(abi.IrModule), C.POINTER(abi.Tensor), sz, C.POINTER(abi.Tensor), sz]
        L.oracle_run_module.restype = i
        L.oracle_f32_to_bf16.argtypes = [C.c_float]; L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_bf16_to_f32.argtypes = [C.c_uint16]; L.oracle_bf16_to_f32.restype = C.c_float
        L.oracle_f32_to_f16.argtypes = [C.c_float]; L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]; L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_e4m3_to_f32.argtypes = [C.c_uint8]; L.oracle_e4m3_to_f32.restype = C.c_float
        L.oracle_f32_to_e4m3.argtypes = [C.c_float]; L.oracle_f32_to_e4m3.restype = C.c_uint8
        L.oracle_set_threads.argtypes = [i]
        self.set_threads(threads or os.cpu_count() or 1)

    def set_threads(self, n):
        self.threads = int(n)
        self.lib.oracle_set_threads(int(n))

    @staticmethod
    def _c(x):
        return np.ascontiguousarray(x, dtype=np.float32)

    def matmul(self, a, b):
        a, b = self._c(a), self._c(b)
        out = np.empty((a.shape[0], b.shape[1]), np.float32)
        self.lib.oracle_matmul_f32(_fp(a), _fp(b), _fp(out), a.shape[0], a.shape[1], b.shape[1])
        return out

    def add(self, a, b):
        a, b = self._c(a), self._c(b)
        out = np.empty_like(a)
        if b.size == a.size:
            self.lib.oracle_add(_fp(a), _fp(b), _fp(out), a.size)
        elif b.size == 1:
            self.lib.oracle_add_scalar(_fp(a), float(b.reshape(-1)[0]), _fp(out), a.size)
        else:
            assert b.size == a.shape[-1]
            self.lib.oracle_add_row_bias(_fp(a), _fp(b), _fp(out), a.size // a.shape[-1], a.shape[-1])
        return out

    def relu(self, a):
        a = self._c(a); out = np.empty_like(a); self.lib.oracle_relu(_fp(a), _fp(out), a.size); return out

    def gelu(self, a):
        a = self._c(a); out = np.empty_like(a); self.lib.oracle_gelu(_fp(a), _fp(out), a.size); return out

    def layernorm(self, x, gamma=None, beta=None, eps=1e-5):
        x = self._c(x); out = np.empty_like(x)
        g = self._c(gamma) if gamma is not None else None
        b = self._c(beta) if beta is not None else None
        self.lib.oracle_layernorm(_fp(x), _fp(g) if g is not None else None, _fp(b) if b is not None else None,
                                  _fp(out), x.size // x.shape[-1], x.shape[-1], eps)
        return out

    def reduce_sum(self, x):
        x = self._c(x); out = np.empty(x.shape[:-1] or (1,), np.float32)
        self.lib.oracle_reduce_sum(_fp(x), _fp(out), x.size // x.shape[-1], x.shape[-1]); return out

    def softmax(self, x):
        x = self._c(x); out = np.empty_like(x)
        self.lib.oracle_softmax(_fp(x), _fp(out), x.size // x.shape[-1], x.shape[-1]); return out

    def attention(self, q, k, v, scale, causal):
        q, k, v = self._c(q), self._c(k), self._c(v)
        bh, s, d = q.shape[:-2], q.shape[-2], q.shape[-1]
        out = np.empty_like(q)
        self.lib.oracle_attention(_fp(q), _fp(k), _fp(v), _fp(out), int(np.prod(bh)) if bh else 1, s, d, scale, int(causal))
        return out

    def conv2d(self, x, w, bias=None, pad=(1, 1), stride=(1, 1), relu=False):
        x, w = self._c(x), self._c(w)
        n, h, wd, c = x.shape; k, r, s, c2 = w.shape
        assert c == c2
        p = (h - r + 2 * pad[0]) // stride[0] + 1; q = (wd - s + 2 * pad[1]) // stride[1] + 1
        out = np.empty((n, p, q, k), np.float32)
        b = self._c(bias) if bias is not None else None
        self.lib.oracle_conv2d_nhwc(_fp(x), _fp(w), _fp(b) if b is not None else None, _fp(out),
                                    n, h, wd, c, k, r, s, pad[0], pad[1], stride[0], stride[1], int(relu))
        return out

    def run_module(self, module, inputs, out_specs):
        """inputs: list of (numpy array, pyc dtype); arrays hold storage bits (float32, or uint16 for bf16/f16).
        out_specs: list of (shape, pyc dtype).  Returns numpy arrays of storage bits."""
        ins = (abi.Tensor * len(inputs))()
        keep = []
        for t, (arr, dt) in zip(ins, inputs):
            arr = np.ascontiguousarray(arr); keep.append(arr)
            t.data = arr.ctypes.data; t.size_bytes = arr.nbytes; t.dtype = dt; t.shape = abi.Shape.of(arr.shape)
        outs = (abi.Tensor * len(out_specs))()
        res = []
        for t, (shape, dt) in zip(outs, out_specs):
            arr = np.zeros(shape, np.float32 if dt == abi.DTYPE_F32 else np.uint16); res.append(arr)
            t.data = arr.ctypes.data; t.size_bytes = arr.nbytes; t.dtype = dt; t.shape = abi.Shape.of(shape)
        rc = self.lib.oracle_run_module(C.byref(module), ins, len(inputs), outs, len(out_specs))
        if rc != 0:
            raise RuntimeError("oracle_run_module rejected the module")
        return res


class _Rails(C.Structure):
    _fields_ = [("enable_auto_switch", C.c_int), ("enable_hard_rollback", C.c_int), ("dwell_steps", C.c_size_t),
                ("cooldown_steps", C.c_size_t), ("consecutive_breach_windows", C.c_size_t),
                ("latency_regression_threshold", C.c_double), ("throughput_regression_threshold", C.c_double),
                ("pressure_score_threshold", C.c_double), ("pressure_events_threshold", C.c_size_t),
                ("rematerialized_tensors_threshold", C.c_size_t)]


class _DistOptions(C.Structure):
    _fields_ = [("enabled", C.c_int), ("backend", C.c_int), ("strategy", C.c_int), ("world_size", C.c_int),
                ("rank", C.c_int), ("local_rank", C.c_int), ("backend_path", C.c_char_p), ("config_json", C.c_char_p)]


class CompileOptions(C.Structure):
    """pyc_compile_options, include/pyc/compiler_api.h:64-80 (208 bytes)."""
    _fields_ = [("enable_fusion", C.c_int), ("enable_memory_reuse", C.c_int), ("enable_autotune", C.c_int),
                ("enable_speculative_plans", C.c_int), ("enable_phantom_graph", C.c_int),
                ("max_speculative_plans", C.c_size_t), ("phantom_horizon_steps", C.c_size_t),
                ("objective_mode", C.c_int), ("memory_budget_bytes", C.c_size_t),
                ("target_utilization_floor", C.c_double), ("deterministic_strict", C.c_int),
                ("compile_budget_ms", C.c_double), ("cache_mode", C.c_int), ("autotune_db_path", C.c_char_p),
                ("rails", _Rails), ("distributed", _DistOptions)]


class _ModelDesc(C.Structure):
    _fields_ = [("module", C.POINTER(abi.IrModule)), ("backend", C.c_int)]


assert C.sizeof(CompileOptions) == 208

RUN_STATS_BYTES = 1368  # sizeof(pyc_run_stats), include/pyc/compiler_api.h:90-159


class RefRuntime:
    """PyC's compile/run API from one of the libraries oracle/Makefile builds."""

    def __init__(self, so_path, threads=None):
        if not os.path.exists(so_path):
            raise FileNotFoundError(f"{so_path}: run `make -C oracle ref` where the PyC sources are available")
        if threads:
            os.environ["PYC_NUM_THREADS"] = str(min(32, int(threads)))  # executor caps at 32, compiler_api.c:1790-1812
        self.threads = int(os.environ.get("PYC_NUM_THREADS", "1"))
        L = self.lib = C.CDLL(so_path, mode=C.RTLD_GLOBAL)
        L.pyc_compile_model.argtypes = [C.POINTER(_ModelDesc), C.POINTER(CompileOptions), C.POINTER(C.c_void_p)]
        L.pyc_compile_model.restype = C.c_int
        L.pyc_run_model.argtypes = [C.c_void_p, C.POINTER(abi.Tensor), C.c_size_t, C.POINTER(abi.Tensor), C.c_size_t, C.c_void_p]
        L.pyc_run_model.restype = C.c_int
        L.pyc_destroy_model.argtypes = [C.c_void_p]
        L.pyc_runtime_rails_default.argtypes = [C.POINTER(_Rails)]
        L.pyc_model_last_decision_log.argtypes = [C.c_void_p]
        L.pyc_model_last_decision_log.restype = C.c_char_p

    def compile(self, module, backend=abi.BACKEND_CPU, fusion=0):
        opts = CompileOptions()
        opts.enable_fusion = fusion
        opts.enable_memory_reuse = 1
        opts.objective_mode = 0
        opts.target_utilization_floor = 0.70
        opts.deterministic_strict = 1
        self.lib.pyc_runtime_rails_default(C.byref(opts.rails))
        desc = _ModelDesc(C.pointer(module), backend)
        model = C.c_void_p()
        st = self.lib.pyc_compile_model(C.byref(desc), C.byref(opts), C.byref(model))
        if st != 0 or not model:
            raise RuntimeError(f"pyc_compile_model status {st}")
        return model

    def run(self, model, inputs, out_specs):
        """inputs: list of (numpy array | raw pointer tuple, dtype); see Oracle.run_module."""
        ins = (abi.Tensor * len(inputs))(); keep = []
        for t, (arr, dt) in zip(ins, inputs):
            arr = np.ascontiguousarray(arr); keep.append(arr)
            t.data = arr.ctypes.data; t.size_bytes = arr.nbytes; t.dtype = dt; t.shape = abi.Shape.of(arr.shape)
        outs = (abi.Tensor * len(out_specs))(); res = []
        for t, (shape, dt) in zip(outs, out_specs):
            arr = np.zeros(shape, np.float32 if dt == abi.DTYPE_F32 else np.uint16); res.append(arr)
            t.data = arr.ctypes.data; t.size_bytes = arr.nbytes; t.dtype = dt; t.shape = abi.Shape.of(shape)
        stats = (C.c_uint8 * RUN_STATS_BYTES)()
        st = self.lib.pyc_run_model(model, ins, len(inputs), outs, len(out_specs), stats)
        if st != 0:
            raise RuntimeError(f"pyc_run_model status {st}: {self.decision_log(model)}")
        return res

    def decision_log(self, model):
        s = self.lib.pyc_model_last_decision_log(model)
        return s.decode() if s else ""

    def destroy(self, model):
        self.lib.pyc_destroy_model(model)


def ref_cpu(threads=None):
    return RefRuntime(REF_CPU_SO, threads)


def ffn_reference(orc, x, w1_codes, s1, w2_codes, s2, b1=None, b2=None, eps=1e-5):
    """CPU definition of the FFN block (UNPINNED: PyC has neither fp8 nor an FFN op): fp32 throughout on the given
    bf16-rounded x and the DEQUANTISED fp8 weights; the contractions are the oracle's matmul (PyC's summation order)."""
    from pyc_b200 import workloads
    w1 = workloads.e4m3_decode(w1_codes) * np.asarray(s1, np.float32)[None, :]
    w2 = workloads.e4m3_decode(w2_codes) * np.asarray(s2, np.float32)[None, :]
    h = orc.matmul(orc.layernorm(x, eps=eps), w1)
    if b1 is not None:
        h = orc.add(h, b1)
    y = orc.matmul(orc.gelu(h), w2)
    return orc.add(y, b2) if b2 is not None else y
