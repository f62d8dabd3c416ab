"""CPU: the places where this backend hands decisions to PyC's own front half, checked against PyC's own code
(libpyc_ref_front.so = PyC's compiler_api.c / kernel_registry.c / runtime_allocator.c / comm_backend_loader.c compiled from
PyC's sources and linked against this library).  Skipped where that library was not built (no PyC checkout at build time).

  * PyC's registry scoring (pyc_kernel_coselect_with_context, kernel_registry.c:374-454) picks, from the descriptors this
    backend registers under "matmul.<dtype>", the tile configuration meant for each of PyC's workload families, and a
    measured time moves the choice between equal-priority tiles;
  * the arena plan of the dispatch layer equals what PyC's planner (pyc_alloc_plan_build_with_mode,
    runtime_allocator.c:123-187) computes from the same requests: same offsets, same peak;
  * the autotune DB (PyC's line format, compiler_api.c:2145-2305) is read back: per-symbol lines reach PyC's registry,
    per-shape lines become winners;
  * this package's NCCL collective backend loads through PyC's loader (comm_backend_loader.c) and refuses bad arguments
    with PyC's status codes."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle
from pyc_b200 import abi, backend, ir

pytestmark = pytest.mark.skipif(not os.path.exists(oracle.REF_FRONT_SO), reason="PyC's front half was not built (no PyC checkout at build time)")

HOPPER, CUDA = 3, 1
SMALL, SQUARE, LARGE_SQUARE, TALL, WIDE = 1, 2, 3, 4, 5


class CoselectContext(C.Structure):
    _fields_ = [("pressure_score", C.c_double), ("pressure_events", C.c_size_t), ("rematerialized_tensors", C.c_size_t),
                ("reused_allocations", C.c_size_t), ("total_requested_bytes", C.c_size_t), ("peak_bytes", C.c_size_t),
                ("memory_budget_bytes", C.c_size_t), ("workload_family", C.c_int), ("hardware_family", C.c_int)]


class AllocRequest(C.Structure):
    _fields_ = [("tensor_id", C.c_int), ("size_bytes", C.c_size_t), ("alignment", C.c_size_t), ("start_step", C.c_int), ("end_step", C.c_int)]


MAX_REQ = 2048


class AllocPlan(C.Structure):
    _fields_ = [("requests", AllocRequest * MAX_REQ), ("request_count", C.c_size_t), ("offsets", C.c_size_t * MAX_REQ),
                ("peak_bytes", C.c_size_t), ("reused_allocations", C.c_size_t), ("allocation_events", C.c_size_t),
                ("overlap_pairs_observed", C.c_size_t), ("largest_allocation_bytes", C.c_size_t), ("rematerialized_tensors", C.c_size_t),
                ("rematerialized_bytes", C.c_size_t), ("pressure_events", C.c_size_t), ("pressure_score", C.c_double)]


@pytest.fixture(scope="module")
def front():
    backend.load()
    L = C.CDLL(oracle.REF_FRONT_SO, mode=C.RTLD_GLOBAL)
    L.pyc_kernel_coselect_with_context.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(CoselectContext), C.POINTER(abi.KernelDesc), C.c_void_p]
    L.pyc_kernel_benchmark_update_symbol.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_double]
    L.pyc_alloc_plan_build_with_mode.argtypes = [C.POINTER(AllocPlan), C.c_int, C.c_size_t]
    L.pyc_load_comm_backend.argtypes = [C.c_char_p, C.c_char_p]; L.pyc_load_comm_backend.restype = C.c_void_p
    L.pyc_unload_comm_backend.argtypes = [C.c_void_p]; L.pyc_unload_comm_backend.restype = None
    backend.load().pyc_cutlass_registry_init()
    return L


def _select(front, key, family):
    ctx = CoselectContext(workload_family=family, hardware_family=HOPPER)
    out = abi.KernelDesc()
    assert front.pyc_kernel_coselect_with_context(key.encode(), CUDA, 0, C.byref(ctx), C.byref(out), None) == 0
    return out.symbol.decode()


def test_pyc_scoring_picks_the_tile_meant_for_each_workload_family(front):
    assert _select(front, "matmul.bf16", LARGE_SQUARE) == "b200_gemm_bf16_tc2_256x256x64_s6"
    assert _select(front, "matmul.bf16", SQUARE) == "b200_gemm_bf16_tc_128x256x64_s4"
    assert _select(front, "matmul.bf16", TALL) == "b200_gemm_bf16_tc_128x128x64_s6"
    assert _select(front, "matmul.bf16", SMALL) == "b200_gemm_bf16_tc_128x64x64_s8"
    assert _select(front, "matmul.f16", LARGE_SQUARE) == "b200_gemm_f16_tc2_256x256x64_s6"
    assert _select(front, "matmul.f32", SMALL) == "b200_gemm_f32_simt_async_32x64x32"
    assert _select(front, "matmul.f32", LARGE_SQUARE) == "b200_gemm_f32_simt_x2_128x128x32"
    # Tensor-core tiles share one priority, so once every candidate has been timed (PyC scores -100 per measured ms and
    # nothing for an untimed kernel) the measured times decide, here between the two CTA-pair variants.
    times = {"tc2_256x256x64_s6": 0.80, "tc2_256x256x64_s7": 0.75, "tc_128x256x64_s4": 0.82, "tc_128x128x64_s6": 0.95, "tc_128x64x64_s8": 1.30,
             "simt_128x128x16": 30.0, "simt_64x64x16": 35.0, "simt_32x64x16": 50.0}
    for suffix, ms in times.items():
        assert front.pyc_kernel_benchmark_update_symbol(b"matmul.bf16", CUDA, f"b200_gemm_bf16_{suffix}".encode(), ms) == 0
    assert _select(front, "matmul.bf16", LARGE_SQUARE) == "b200_gemm_bf16_tc2_256x256x64_s7"


def _ffn_like_module():
    # two blocks of layernorm -> matmul -> add(bias) -> gelu -> matmul -> add(residual): intermediates with different lifetimes
    b = ir.ModuleBuilder()
    x = b.input("x", abi.DTYPE_F32, [64, 128]); w1 = b.input("w1", abi.DTYPE_F32, [128, 512]); b1 = b.input("b1", abi.DTYPE_F32, [512])
    w2 = b.input("w2", abi.DTYPE_F32, [512, 128])
    h = b.gelu(b.add(b.matmul(b.layernorm(x), w1), b1))
    y1 = b.add(b.matmul(h, w2), x)
    h2 = b.gelu(b.add(b.matmul(b.layernorm(y1), w1), b1))      # a second block on the same weights
    b.output(b.add(b.matmul(h2, w2), y1))
    return b.module, [(64, 128), (128, 512), (512,), (512, 128)], (64, 128)


@pytest.mark.parametrize("on_device", [0, 1])
def test_arena_plan_equals_pycs_planner_on_the_same_requests(front, on_device):
    module, in_shapes, out_shape = _ffn_like_module()
    arrays = [np.zeros(s, np.float32) for s in in_shapes]; out = np.zeros(out_shape, np.float32)
    ins = (abi.Tensor * len(arrays))(*[backend.make_tensor(a.ctypes.data, a.nbytes, abi.DTYPE_F32, a.shape) for a in arrays])
    outs = (abi.Tensor * 1)(backend.make_tensor(out.ctypes.data, out.nbytes, abi.DTYPE_F32, out.shape))
    reqs = (AllocRequest * 64)(); offs = (C.c_size_t * 64)(); n = C.c_size_t(); peak = C.c_size_t()
    L = backend.load()
    L.pyc_b200_plan_arena.argtypes = [C.POINTER(abi.IrModule), C.POINTER(abi.Tensor), C.c_size_t, C.POINTER(abi.Tensor), C.c_size_t, C.c_int,
                                      C.POINTER(AllocRequest), C.POINTER(C.c_size_t), C.c_size_t, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    assert L.pyc_b200_plan_arena(C.byref(module), ins, len(arrays), outs, 1, on_device, reqs, offs, 64, C.byref(n), C.byref(peak)) == 0, backend.last_error()
    assert n.value >= (5 if on_device else 9)
    plan = AllocPlan()
    for i in range(n.value):
        plan.requests[i] = reqs[i]
    plan.request_count = n.value
    assert front.pyc_alloc_plan_build_with_mode(C.byref(plan), 0, 0) == 0
    assert [plan.offsets[i] for i in range(n.value)] == [offs[i] for i in range(n.value)]
    assert plan.peak_bytes == peak.value
    total = sum(reqs[i].size_bytes for i in range(n.value))
    assert peak.value < total and plan.reused_allocations >= 1          # lifetimes really are reused


def test_autotune_db_in_pycs_format_is_read_back(front, tmp_path):
    db = tmp_path / "autotune.db"
    db.write_text("matmul|1|b200_gemm_bf16_tc_128x256x64_s4|0.412000\n"
                  "matmul@bf16:4096x4096x4096|1|b200_gemm_bf16_tc_128x256x64_s4|0.101000\n"
                  "matmul@bf16:4096x4096x4096|1|b200_gemm_bf16_tc2_256x256x64_s6|0.099000\n"
                  "matmul@f32:512x512x512|1|b200_gemm_f32_simt_async_32x64x32|0.014000\n"
                  "matmul@bf16:64x64x64|1|no_such_symbol|0.001\n"          # unknown symbol: ignored
                  "matmul@bf16:8x8x8|0|b200_gemm_bf16_tc_128x64x64_s8|0.001\n"   # CPU backend line: ignored
                  "garbage line\n")
    assert backend.autotune_db_load(str(db)) == 2
    assert backend.autotune_db_load(str(tmp_path / "missing.db")) == 0
    # the per-symbol line went into PyC's registry: the timed 128x256 tile now beats the untimed... (time is a penalty), so check the read-back value
    class Bench(C.Structure):
        _fields_ = [("selected", C.c_int), ("considered", C.c_int), ("best_time_ms", C.c_double)]
    b = Bench()
    front.pyc_kernel_benchmark_read.argtypes = [C.c_char_p, C.c_int, C.POINTER(Bench)]
    front.pyc_kernel_benchmark_read.restype = None
    front.pyc_kernel_benchmark_read(b"matmul", CUDA, C.byref(b))
    assert b.considered >= 1 and 0.0 < b.best_time_ms <= 0.412


def test_nccl_collective_backend_loads_through_pycs_loader(front):
    from pyc_b200 import ffn
    path = ffn.CollectiveBackend.DEFAULT
    assert os.path.exists(path)
    vt = front.pyc_load_comm_backend(path.encode(), b"{}")
    assert vt, "PyC's loader rejected libpyc_b200_comm_nccl.so"
    words = (C.c_void_p * 8).from_address(vt)
    assert all(words[i] for i in range(1, 8))                       # all seven entry points present
    all_reduce = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p)(words[1])
    buf = (C.c_char * 64)()
    INVALID = 3
    assert all_reduce(words[0], None, buf, buf, 8, abi.DTYPE_BF16, 0, None) == INVALID          # no communicator
    assert all_reduce(words[0], 0x10, buf, buf, 0, abi.DTYPE_BF16, 0, None) == INVALID          # nothing to reduce
    assert all_reduce(words[0], 0x10, buf, buf, 8, abi.DTYPE_UNKNOWN, 0, None) == INVALID       # dtype without an NCCL type
    assert all_reduce(words[0], 0x10, None, buf, 8, abi.DTYPE_BF16, 0, None) == INVALID         # NULL buffer
    assert all_reduce(words[0], 0x10, buf, buf, 8, abi.DTYPE_BF16, 9, None) == INVALID          # unknown reduce op
    front.pyc_unload_comm_backend(vt)
