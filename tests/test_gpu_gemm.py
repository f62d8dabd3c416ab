"""GPU parity: the GEMM kernels (tcgen05 bf16/f16, fp32 SIMT) through the C-ABI
against the CPU oracle on the same seeded, storage-rounded inputs.

Tolerances (norm-wise, vs the fp32 CPU result): fp32 1e-5, bf16/f16 2e-2.
"""
import numpy as np
import pytest

from pyc_b200 import abi, workloads

pytestmark = pytest.mark.gpu

TC = ["tc_128x256x64_s4", "tc_128x128x64_s6", "tc_128x64x64_s8", "tc2_256x256x64_s7", "tc2_256x256x64_s6"]
SIMT = ["simt_128x128x16", "simt_64x64x16", "simt_32x64x16"]
NAME = {abi.DTYPE_F32: "f32", abi.DTYPE_BF16: "bf16", abi.DTYPE_F16: "f16"}


def run_case(backend, oracle_lib, dtype, M, K, N, cfg=None, add_mode=abi.ADD_NONE, act=abi.ACT_NONE, alpha=1.0,
             b_col_major=False, seed=0, scale=1.0):
    from gpu_util import TOL, empty_device, rel_err, round_to, sync_ok, to_device, to_host_f32
    a = workloads.normal((M, K), 1000 + seed, scale); b = workloads.normal((K, N), 2000 + seed, scale)
    a_s, a_r = round_to(dtype, a); b_s, b_r = round_to(dtype, b)
    add_shape = {abi.ADD_NONE: None, abi.ADD_MATRIX: (M, N), abi.ADD_ROW_BIAS: (N,), abi.ADD_SCALAR: (1,)}[add_mode]
    want = alpha * oracle_lib.matmul(a_r, b_r)
    d_add = None
    if add_shape:
        c_s, c_r = round_to(dtype, workloads.normal(add_shape, 3000 + seed, scale * np.sqrt(K)))
        d_add = to_device(c_s)
        want = oracle_lib.add(want, c_r)
    if act == abi.ACT_RELU:
        want = oracle_lib.relu(want)
    elif act == abi.ACT_GELU:
        want = oracle_lib.gelu(want)
    d_a = to_device(a_s); d_b = to_device(np.ascontiguousarray(b_s.T) if b_col_major else b_s)
    d_out = empty_device(dtype, (M, N))
    symbol = f"b200_gemm_{NAME[dtype]}_{cfg}" if cfg else None
    backend.gemm(dtype, M, N, K, d_a.data_ptr(), d_b.data_ptr(), d_out.data_ptr(),
                 add=d_add.data_ptr() if d_add is not None else None, add_mode=add_mode, act=act, alpha=alpha,
                 b_col_major=b_col_major, symbol=symbol)
    sync_ok()
    err = rel_err(to_host_f32(dtype, d_out), want)
    assert err <= TOL[dtype], f"{symbol} {M}x{K}x{N}: rel err {err:.3e} > {TOL[dtype]}"
    return err


@pytest.mark.parametrize("cfg", TC)
@pytest.mark.parametrize("shape", [(128, 64, 64), (256, 512, 256), (384, 1024, 512)])
def test_tc_bf16_plain(backend, oracle_lib, cfg, shape):
    run_case(backend, oracle_lib, abi.DTYPE_BF16, *shape, cfg=cfg)


@pytest.mark.parametrize("cfg", TC)
def test_tc_bf16_ragged_edges(backend, oracle_lib, cfg):
    # M, N not multiples of the tile, K not a multiple of 64 (TMA zero fill), N % 8 == 0 only.
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 200, 264, 328, cfg=cfg, add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_RELU, seed=1)
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 1, 8, 8, cfg=cfg, seed=2)
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 129, 72, 264, cfg=cfg, add_mode=abi.ADD_MATRIX, seed=3)


@pytest.mark.parametrize("add_mode,act", [(abi.ADD_ROW_BIAS, abi.ACT_GELU), (abi.ADD_ROW_BIAS, abi.ACT_RELU),
                                          (abi.ADD_MATRIX, abi.ACT_NONE), (abi.ADD_SCALAR, abi.ACT_RELU), (abi.ADD_NONE, abi.ACT_GELU)])
def test_tc_bf16_epilogues(backend, oracle_lib, add_mode, act):
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 256, 256, 512, cfg=TC[0], add_mode=add_mode, act=act, seed=4, scale=0.5)


def test_tc_many_tiles_persistent_loop(backend, oracle_lib):
    # more tiles than SMs: every CTA walks several tiles, both TMEM accumulators and every ring phase get reused
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 2048, 320, 2304, cfg=TC[1], add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_GELU, seed=5, scale=0.25)
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 1536, 192, 4096, cfg=TC[0], seed=6, scale=0.25)


def test_tc_f16_and_col_major_b(backend, oracle_lib):
    run_case(backend, oracle_lib, abi.DTYPE_F16, 256, 256, 256, cfg=TC[0], seed=7, scale=0.25)
    run_case(backend, oracle_lib, abi.DTYPE_F16, 256, 320, 384, cfg=TC[1], b_col_major=True, add_mode=abi.ADD_ROW_BIAS, seed=8, scale=0.25)
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 200, 136, 72, cfg=TC[2], b_col_major=True, seed=9)


def test_alpha_and_heuristic_choice(backend, oracle_lib):
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 256, 128, 256, alpha=0.5, seed=10)
    run_case(backend, oracle_lib, abi.DTYPE_BF16, 100, 36, 52, seed=11)   # N % 8 != 0: the any-shape SIMT path
    run_case(backend, oracle_lib, abi.DTYPE_F32, 512, 512, 512, add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_RELU, seed=12)


@pytest.mark.parametrize("cfg", SIMT)
def test_simt_f32(backend, oracle_lib, cfg):
    run_case(backend, oracle_lib, abi.DTYPE_F32, 33, 65, 17, cfg=cfg, add_mode=abi.ADD_MATRIX, act=abi.ACT_RELU, seed=13)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 256, 512, 192, cfg=cfg, add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_GELU, seed=14)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 130, 70, 100, cfg=cfg, b_col_major=True, seed=15)


def test_simt_latency_tile_f32(backend, oracle_lib):
    cfg = "simt_async_32x64x32"
    run_case(backend, oracle_lib, abi.DTYPE_F32, 512, 512, 512, cfg=cfg, add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_RELU, seed=21)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 100, 64, 72, cfg=cfg, add_mode=abi.ADD_MATRIX, act=abi.ACT_GELU, seed=22)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 33, 68, 20, cfg=cfg, add_mode=abi.ADD_SCALAR, seed=23)      # ragged tiles, K not a multiple of 32
    run_case(backend, oracle_lib, abi.DTYPE_F32, 1, 4, 4, cfg=cfg, seed=24)
    with pytest.raises(backend.BackendError):   # N % 4 != 0 is not this tile's business
        run_case(backend, oracle_lib, abi.DTYPE_F32, 16, 16, 18, cfg=cfg, seed=25)


def test_simt_packed_fma_tile_f32(backend, oracle_lib):
    cfg = "simt_x2_128x128x32"
    run_case(backend, oracle_lib, abi.DTYPE_F32, 512, 512, 512, cfg=cfg, add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_RELU, seed=31)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 130, 100, 72, cfg=cfg, add_mode=abi.ADD_MATRIX, act=abi.ACT_GELU, seed=32)   # ragged in M, N and K
    run_case(backend, oracle_lib, abi.DTYPE_F32, 33, 20, 68, cfg=cfg, add_mode=abi.ADD_SCALAR, alpha=0.5, seed=33)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 1, 4, 4, cfg=cfg, seed=34)
    run_case(backend, oracle_lib, abi.DTYPE_F32, 1024, 516, 1280, cfg=cfg, seed=35)     # several tiles per CTA slot, K % 8 != 0
    with pytest.raises(backend.BackendError):   # N % 4 != 0 is not this tile's business
        run_case(backend, oracle_lib, abi.DTYPE_F32, 16, 16, 18, cfg=cfg, seed=36)


def test_simt_packed_fma_is_bit_identical_to_the_scalar_fma_kernel(backend):
    # fma.rn.f32x2 is two independent IEEE FMAs and both kernels accumulate in ascending k with one accumulator per output.
    from gpu_util import empty_device, sync_ok, to_device
    M, K, N = 300, 516, 260
    a = workloads.normal((M, K), 41, 1.0); b = workloads.normal((K, N), 42, 1.0); bias = workloads.normal((N,), 43, 1.0)
    d_a, d_b, d_c = to_device(a), to_device(b), to_device(bias)
    outs = []
    for cfg in ("simt_x2_128x128x32", "simt_64x64x16"):
        d_o = empty_device(abi.DTYPE_F32, (M, N))
        backend.gemm(abi.DTYPE_F32, M, N, K, d_a.data_ptr(), d_b.data_ptr(), d_o.data_ptr(), add=d_c.data_ptr(),
                     add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_RELU, symbol=f"b200_gemm_f32_{cfg}")
        sync_ok()
        outs.append(d_o.cpu().numpy())
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))


def test_config1_f32_512_matches_golden_definition(backend, oracle_lib):
    # benchmark configuration 1: X[512,512] W[512,512] b[512] ~ U(-1,1), matmul -> add -> relu.
    from gpu_util import empty_device, rel_err, sync_ok, to_device
    x, w, b = workloads.gemm_inputs(1, 512, 512, 512, ("uniform", -1.0, 1.0))
    want = oracle_lib.relu(oracle_lib.add(oracle_lib.matmul(x, w), b))
    d_x, d_w, d_b = to_device(x), to_device(w), to_device(b); d_o = empty_device(abi.DTYPE_F32, (512, 512))
    backend.gemm(abi.DTYPE_F32, 512, 512, 512, d_x.data_ptr(), d_w.data_ptr(), d_o.data_ptr(), add=d_b.data_ptr(),
                 add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_RELU)
    sync_ok()
    assert rel_err(d_o.cpu().numpy(), want) <= 1e-5


def test_legacy_symbols_and_beta(backend, oracle_lib):
    from gpu_util import empty_device, rel_err, round_to, sync_ok, to_device, to_host_f32
    M, K, N = 256, 192, 320
    a = workloads.normal((M, K), 31); b = workloads.normal((K, N), 32); c0 = workloads.normal((M, N), 33, 4.0)
    for sym, dtype, colmajor in [("cutlass_gemm_tensorcore_bf16", abi.DTYPE_BF16, False), ("cutlass_gemm_tensorcore_f16", abi.DTYPE_F16, True),
                                 ("cutlass_gemm_simt_f32", abi.DTYPE_F32, False), ("ada_gemm_k64_warp32_async_f32", abi.DTYPE_F32, False)]:
        a_s, a_r = round_to(dtype, a); b_s, b_r = round_to(dtype, b); c_s, c_r = round_to(dtype, c0)
        d_a = to_device(a_s); d_b = to_device(np.ascontiguousarray(b_s.T) if colmajor else b_s); d_c = to_device(c_s)
        backend.gemm_by_symbol(sym, M, N, K, d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), alpha=1.5, beta=0.5)
        sync_ok()
        want = 1.5 * oracle_lib.matmul(a_r, b_r) + 0.5 * c_r
        from gpu_util import TOL
        assert rel_err(to_host_f32(dtype, d_c), want) <= TOL[dtype], sym


def test_full_size_8192_spot_rows_and_linearity(backend, oracle_lib):
    # benchmark configuration 2 at full size: sampled rows against the oracle, plus a size-independent property
    # (GEMM is linear in alpha; bias+GELU epilogue applied to the same accumulators).
    import torch
    from gpu_util import rel_err, sync_ok, to_device, to_host_f32
    n = 8192
    a, b, bias = workloads.gemm_inputs(2, n, n, n, ("normal", 0.02))
    a_bits, b_bits, bias_bits = workloads.to_bf16_bits(a), workloads.to_bf16_bits(b), workloads.to_bf16_bits(bias)
    del a, b
    d_a, d_b, d_bias = to_device(a_bits), to_device(b_bits), to_device(bias_bits)
    d_o = torch.zeros((n, n), dtype=torch.int16, device="cuda"); d_o2 = torch.zeros_like(d_o)
    backend.gemm(abi.DTYPE_BF16, n, n, n, d_a.data_ptr(), d_b.data_ptr(), d_o.data_ptr(), add=d_bias.data_ptr(),
                 add_mode=abi.ADD_ROW_BIAS, act=abi.ACT_GELU)
    backend.gemm(abi.DTYPE_BF16, n, n, n, d_a.data_ptr(), d_b.data_ptr(), d_o2.data_ptr())
    sync_ok()
    rows = [0, 1, 127, 128, 4095, 4097, 8191]
    b_f = workloads.bf16_bits_to_f32(b_bits)
    a_rows = workloads.bf16_bits_to_f32(a_bits[rows])
    plain = oracle_lib.matmul(a_rows, b_f)
    want = oracle_lib.gelu(oracle_lib.add(plain, workloads.bf16_bits_to_f32(bias_bits)))
    got = to_host_f32(abi.DTYPE_BF16, d_o[rows]); got2 = to_host_f32(abi.DTYPE_BF16, d_o2[rows])
    assert rel_err(got2, plain) <= 2e-2
    assert rel_err(got, want) <= 2e-2
    # checksum of checksums: column sums of the plain product == (column sums of A) @ B
    colsum = d_o2.view(torch.bfloat16).float().sum(0).double().cpu().numpy()
    want_colsum = workloads.bf16_bits_to_f32(a_bits).astype(np.float64).sum(0) @ b_f.astype(np.float64)
    assert rel_err(colsum, want_colsum) <= 2e-2
