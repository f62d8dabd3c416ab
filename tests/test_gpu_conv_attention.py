"""GPU parity: conv2d (implicit GEMM on tcgen05 + direct kernel) and fused attention
(tcgen05 + row-per-warp kernel) through the C-ABI against the CPU oracle.
Tolerance norm-wise vs the fp32 CPU result on the storage-rounded inputs: bf16/f16 2e-2, fp32 1e-5
(attention fp32: 1e-4, its oracle sums in double while the kernel keeps fp32 statistics)."""
import math

import numpy as np
import pytest

from pyc_b200 import abi, workloads

pytestmark = pytest.mark.gpu


def conv_case(backend, oracle_lib, dtype, N, H, W, C, K, R=3, S=3, pad=(1, 1), stride=(1, 1), bias=True, relu=True, seed=0, symbol=None):
    from gpu_util import TOL, empty_device, rel_err, round_to, sync_ok, to_device, to_host_f32
    x_s, x_r = round_to(dtype, workloads.uniform((N, H, W, C), 4000 + seed))
    w_s, w_r = round_to(dtype, workloads.normal((K, R, S, C), 4100 + seed, math.sqrt(2.0 / (R * S * C))))
    b_s, b_r = round_to(dtype, workloads.normal((K,), 4200 + seed, 0.1))
    P = (H - R + 2 * pad[0]) // stride[0] + 1; Q = (W - S + 2 * pad[1]) // stride[1] + 1
    d_x, d_w, d_b = to_device(x_s), to_device(w_s), to_device(b_s)
    d_o = empty_device(dtype, (N, P, Q, K))
    if symbol:
        rc = backend.load().pyc_cutlass_conv2d_dispatch(symbol.encode(), N, H, W, C, K, R, S, pad[0], pad[1], stride[0], stride[1],
                                                        d_x.data_ptr(), d_w.data_ptr(), d_o.data_ptr(), None)
        assert rc == 0, backend.last_error()
        bias = relu = False
    else:
        backend.conv2d(dtype, N, H, W, C, K, R, S, pad, stride, d_x.data_ptr(), d_w.data_ptr(), d_b.data_ptr() if bias else None, relu, d_o.data_ptr())
    sync_ok()
    want = oracle_lib.conv2d(x_r, w_r, b_r if bias else None, pad=pad, stride=stride, relu=relu)
    err = rel_err(to_host_f32(dtype, d_o), want)
    assert err <= TOL[dtype], f"conv {N}x{H}x{W}x{C}->{K} {R}x{S}: rel err {err:.3e}"


@pytest.mark.parametrize("shape", [(4, 56, 56, 64, 64), (8, 14, 14, 256, 256), (3, 17, 23, 32, 40), (2, 8, 8, 128, 128), (5, 7, 9, 72, 136)])
def test_conv_tc_bf16_bias_relu(backend, oracle_lib, shape):
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, *shape, seed=shape[1])


def test_conv_tc_filter_shapes_and_f16(backend, oracle_lib):
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 12, 12, 64, 64, R=1, S=1, pad=(0, 0), seed=1)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 16, 20, 64, 96, R=5, S=5, pad=(2, 2), seed=2)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 16, 20, 64, 64, R=3, S=5, pad=(0, 1), bias=False, relu=False, seed=3)
    conv_case(backend, oracle_lib, abi.DTYPE_F16, 4, 14, 14, 128, 64, seed=4)


def test_conv_64_filters_two_ctas_per_sm(backend, oracle_lib):
    # K <= 64 runs two co-resident CTAs per SM: ragged P/Q, 1 x 1 and 3 x 2 filters, fewer than 64 filters, no padding, f16,
    # and more bricks than CTA slots
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 3, 19, 21, 64, 64, seed=31)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 56, 56, 64, 64, seed=32)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 17, 9, 64, 40, R=3, S=2, pad=(1, 0), seed=33)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 12, 12, 64, 64, R=1, S=1, pad=(0, 0), bias=False, relu=False, seed=34)
    conv_case(backend, oracle_lib, abi.DTYPE_F16, 2, 30, 8, 64, 64, R=3, S=3, pad=(0, 0), seed=35)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 150, 8, 16, 64, 64, seed=36)                  # more bricks than SMs: CTAs loop


def test_conv_direct_paths_and_legacy_symbols(backend, oracle_lib):
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 15, 15, 64, 32, stride=(2, 2), seed=5)      # stride 2
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 9, 9, 12, 20, seed=6)                        # C % 8 != 0
    conv_case(backend, oracle_lib, abi.DTYPE_F32, 2, 10, 11, 16, 24, seed=7)                       # fp32
    conv_case(backend, oracle_lib, abi.DTYPE_F16, 2, 14, 14, 64, 64, symbol="cutlass_conv2d_fprop_f16", seed=8)
    conv_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 14, 14, 64, 64, symbol="b200_conv2d_fprop_bf16", seed=9)
    assert backend.load().pyc_cutlass_conv2d_dispatch(b"nope", 1, 4, 4, 8, 8, 3, 3, 1, 1, 1, 1, None, None, None, None) == -1


def test_conv_full_size_configs_sampled_images(backend, oracle_lib):
    # benchmark configuration 4 at full size; the oracle checks the first, a middle and the last image (images are independent).
    from gpu_util import empty_device, rel_err, round_to, sync_ok, to_device, to_host_f32
    for (N, H, C, K) in [(64, 56, 64, 64), (256, 14, 256, 256)]:
        x_s, x_r = round_to(abi.DTYPE_BF16, workloads.uniform((N, H, H, C), workloads.tensor_seed(4, 0)))
        w_s, w_r = round_to(abi.DTYPE_BF16, workloads.normal((K, 3, 3, C), workloads.tensor_seed(4, 1), math.sqrt(2.0 / (9 * C))))
        b_s, b_r = round_to(abi.DTYPE_BF16, workloads.normal((K,), workloads.tensor_seed(4, 2), 0.1))
        d_x, d_w, d_b = to_device(x_s), to_device(w_s), to_device(b_s); d_o = empty_device(abi.DTYPE_BF16, (N, H, H, K))
        backend.conv2d(abi.DTYPE_BF16, N, H, H, C, K, 3, 3, (1, 1), (1, 1), d_x.data_ptr(), d_w.data_ptr(), d_b.data_ptr(), True, d_o.data_ptr())
        sync_ok()
        pick = [0, N // 2, N - 1]
        want = oracle_lib.conv2d(x_r[pick], w_r, b_r, relu=True)
        assert rel_err(to_host_f32(abi.DTYPE_BF16, d_o[pick]), want) <= 2e-2


def attn_case(backend, oracle_lib, dtype, bh, seq, d, causal, seed=0, symbol=None, tol=None):
    from gpu_util import TOL, empty_device, rel_err, round_to, sync_ok, to_device, to_host_f32
    q_s, q_r = round_to(dtype, workloads.normal((bh, seq, d), 5000 + seed))
    k_s, k_r = round_to(dtype, workloads.normal((bh, seq, d), 5100 + seed))
    v_s, v_r = round_to(dtype, workloads.normal((bh, seq, d), 5200 + seed))
    d_q, d_k, d_v = to_device(q_s), to_device(k_s), to_device(v_s); d_o = empty_device(dtype, (bh, seq, d))
    scale = 1.0 / math.sqrt(d)
    if symbol:
        assert bh == 1
        rc = backend.load().pyc_cutlass_attention_dispatch(symbol.encode(), seq, d, d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_o.data_ptr(), scale, None)
        assert rc == 0, backend.last_error()
    else:
        backend.attention(dtype, bh, seq, d, d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_o.data_ptr(), scale, causal)
    sync_ok()
    want = oracle_lib.attention(q_r, k_r, v_r, scale, causal)
    err = rel_err(to_host_f32(dtype, d_o), want)
    assert err <= (tol or TOL[dtype]), f"attention bh={bh} seq={seq} d={d} causal={causal}: rel err {err:.3e}"


@pytest.fixture(params=["1", "2", "3", "4"], ids=["kernel1_smemP", "kernel2_tmemP", "kernel3_persistent", "kernel4_two_tiles"])
def attn_kernel(request, monkeypatch):
    # all tensor-core kernels are held to the same bar; the env switch picks one
    monkeypatch.setenv("PYC_B200_ATTENTION_KERNEL", request.param)
    return request.param


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("seq", [128, 256, 200, 1, 640, 129, 64, 65])
def test_attention_tc_bf16_d128(backend, oracle_lib, attn_kernel, seq, causal):
    attn_case(backend, oracle_lib, abi.DTYPE_BF16, 3, seq, 128, causal, seed=seq)


def test_attention_tc_d64_f16_and_symbols(backend, oracle_lib, attn_kernel):
    attn_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 384, 64, True, seed=1)
    attn_case(backend, oracle_lib, abi.DTYPE_F16, 2, 300, 128, False, seed=2)
    attn_case(backend, oracle_lib, abi.DTYPE_BF16, 1, 256, 128, True, seed=3, symbol="b200_attention_bf16_causal")
    attn_case(backend, oracle_lib, abi.DTYPE_F16, 1, 256, 128, False, seed=4, symbol="cutlass_attention_f16")
    assert backend.load().pyc_cutlass_attention_dispatch(b"nope", 8, 8, None, None, None, None, 1.0, None) == -1


def test_attention_persistent_ctas_walk_several_query_blocks(backend, oracle_lib):
    # more work units than the 2 x 148 resident CTAs of the default (persistent) kernel, so CTAs go round their loop more
    # than once: barriers, TMEM and the K/V ring carry over from one query block to the next
    attn_case(backend, oracle_lib, abi.DTYPE_BF16, 75, 512, 128, False, seed=21)    # 300 single-block units
    attn_case(backend, oracle_lib, abi.DTYPE_BF16, 160, 384, 64, True, seed=22)     # 320 units: pairs (2, 0) and the lone middle block
    attn_case(backend, oracle_lib, abi.DTYPE_F16, 70, 520, 128, True, seed=23)      # ragged: 5 query blocks, last one 8 rows


def test_attention_row_warp_paths(backend, oracle_lib):
    attn_case(backend, oracle_lib, abi.DTYPE_F32, 2, 77, 40, True, seed=5, tol=1e-4)
    attn_case(backend, oracle_lib, abi.DTYPE_BF16, 2, 50, 96, False, seed=6)
    attn_case(backend, oracle_lib, abi.DTYPE_F32, 1, 33, 200, False, seed=7, tol=1e-4)


def test_attention_config3_shape_sampled_heads(backend, oracle_lib):
    # benchmark configuration 3: 8 x 32 heads, seq 2048, d 128, causal.  All 256 heads run; the oracle checks three of them
    # (heads are independent), and every row of every head must be a convex combination of V rows (|out| <= max|V|).
    import torch
    from gpu_util import rel_err, sync_ok, to_device, to_host_f32
    bh, seq, d = 256, 2048, 128
    shape = (bh, seq, d)
    q_b = workloads.to_bf16_bits(workloads.normal(shape, workloads.tensor_seed(3, 0)))
    k_b = workloads.to_bf16_bits(workloads.normal(shape, workloads.tensor_seed(3, 1)))
    v_b = workloads.to_bf16_bits(workloads.normal(shape, workloads.tensor_seed(3, 2)))
    d_q, d_k, d_v = to_device(q_b), to_device(k_b), to_device(v_b); d_o = torch.zeros(shape, dtype=torch.int16, device="cuda")
    scale = 1.0 / math.sqrt(d)
    backend.attention(abi.DTYPE_BF16, bh, seq, d, d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), d_o.data_ptr(), scale, True)
    sync_ok()
    pick = [0, 101, 255]
    f = workloads.bf16_bits_to_f32
    want = oracle_lib.attention(f(q_b[pick]), f(k_b[pick]), f(v_b[pick]), scale, True)
    assert rel_err(to_host_f32(abi.DTYPE_BF16, d_o[pick]), want) <= 2e-2
    out = d_o.view(torch.bfloat16).float()
    vmax = d_v.view(torch.bfloat16).float().abs().amax()
    assert torch.isfinite(out).all() and out.abs().amax() <= vmax * 1.01
    # first query row of a causal head attends to key 0 only: out[0] == V[0] exactly
    assert torch.equal(d_o[:, 0, :], d_v[:, 0, :])
