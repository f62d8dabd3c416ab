"""GPU parity: fp8 (e4m3) GEMM, per-token quantisers and the FFN block through the C-ABI against the CPU oracle.
fp8 GEMM on exactly representable operands: 1e-5-level (only the summation order differs); quantisers: every value
within half an e4m3 step of the oracle value; FFN block: 6e-2 norm-wise vs the fp32 CPU result (the fp8 tolerance)."""
import numpy as np
import pytest

import oracle
from pyc_b200 import abi, workloads

pytestmark = pytest.mark.gpu


def _dev_u8(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.uint8)).cuda()


def _dev_f32(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


@pytest.fixture(params=["0", "1"], ids=["single_cta", "cta_pair"])
def fp8_kernel(request, monkeypatch):
    # both fp8 tensor-core kernels are held to the same bar on every shape; without the switch the library picks by size
    monkeypatch.setenv("PYC_B200_FP8_PAIR", request.param)
    return request.param


@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 512, 384), (200, 272, 336), (1024, 1024, 2048), (2250, 400, 2320)])
@pytest.mark.parametrize("colmajor", [False, True])
def test_fp8_gemm_with_scales(backend, oracle_lib, fp8_kernel, shape, colmajor):
    import torch
    from gpu_util import rel_err, sync_ok
    M, K, N = shape
    a_c = workloads.e4m3_encode(workloads.normal((M, K), 61, 2.0)); b_c = workloads.e4m3_encode(workloads.normal((K, N), 62, 2.0))
    rs = np.abs(workloads.normal((M,), 63)) + 0.5; cs = np.abs(workloads.normal((N,), 64)) + 0.5
    bias_b = workloads.to_bf16_bits(workloads.normal((N,), 65, 8.0))
    want = oracle_lib.matmul(workloads.e4m3_decode(a_c), workloads.e4m3_decode(b_c)) * rs[:, None] * cs[None, :] + workloads.bf16_bits_to_f32(bias_b)
    want = oracle_lib.relu(want)
    d_a = _dev_u8(a_c); d_b = _dev_u8(b_c.T if colmajor else b_c); d_rs, d_cs = _dev_f32(rs), _dev_f32(cs)
    d_bias = torch.from_numpy(bias_b.view(np.int16)).cuda(); d_o = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    backend.gemm_fp8(M, N, K, d_a.data_ptr(), d_b.data_ptr(), d_o.data_ptr(), d_rs.data_ptr(), d_cs.data_ptr(), d_bias.data_ptr(), abi.ACT_RELU, colmajor)
    sync_ok()
    got = workloads.bf16_bits_to_f32(d_o.cpu().numpy().view(np.uint16))
    assert rel_err(got, want) <= 2e-2 / 4   # output is bf16-rounded; the products themselves are exact in fp32


# rows >= 64 and 1024 / 2048 / 4096 columns take the one-warp-per-row kernels (row counts that do not fill the last CTA)
@pytest.mark.parametrize("shape", [(64, 256), (37, 4096), (16, 16384), (5, 1024), (100, 4096), (67, 2048), (201, 1024)])
def test_row_quantisers(backend, oracle_lib, shape):
    import torch
    from gpu_util import sync_ok
    rows, cols = shape
    xb = workloads.to_bf16_bits(workloads.normal(shape, 71, 3.0)); x = workloads.bf16_bits_to_f32(xb)
    d_x = torch.from_numpy(xb.view(np.int16)).cuda()
    d_q = torch.zeros(shape, dtype=torch.uint8, device="cuda"); d_s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    for ln in (False, True):
        if ln:
            backend.layernorm_quantize(d_x.data_ptr(), None, None, d_q.data_ptr(), d_s.data_ptr(), rows, cols)
            ref = oracle_lib.layernorm(x)
        else:
            backend.quantize_rows(d_x.data_ptr(), d_q.data_ptr(), d_s.data_ptr(), rows, cols)
            ref = x
        sync_ok()
        scale = d_s.cpu().numpy(); q = workloads.e4m3_decode(d_q.cpu().numpy())
        np.testing.assert_allclose(scale, np.abs(ref).max(-1) / 448.0, rtol=1e-5)
        # dequantised value within half an e4m3 step (relative 2^-4 of the value's binade, absolute 2^-10 near zero) of the reference
        err = np.abs(q * scale[:, None] - ref)
        bound = np.maximum(np.abs(ref) * 2.0 ** -4, scale[:, None] * 2.0 ** -10) * 1.01 + 1e-6
        assert (err <= bound).all()
        assert np.abs(q).max() <= 448.0


@pytest.mark.parametrize("dims", [(256, 256, 1024), (512, 1024, 4096)])
def test_ffn_block_vs_oracle(backend, oracle_lib, dims):
    import torch
    from gpu_util import rel_err, sync_ok
    from pyc_b200 import ffn
    T, H, I = dims
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(T, H, I)
    want = oracle.ffn_reference(oracle_lib, workloads.bf16_bits_to_f32(xb), w1, s1, w2, s2)
    blk = ffn.FfnBlock(T, H, I, w1, s1, w2, s2, torch)
    d_x = torch.from_numpy(xb.view(np.int16)).cuda()
    for _ in range(2):
        out = blk.run(d_x)
    sync_ok()
    err = rel_err(out.float().cpu().numpy(), want)
    assert err <= 6e-2, f"ffn {dims}: rel err {err:.3e}"
    # emulated 2-way tensor parallelism on one GPU: two shards run one after the other, partial sums added
    parts = []
    for r in range(2):
        w1r, s1r, w2r = ffn.shard_weights(w1, s1, w2, r, 2)
        parts.append(ffn.FfnBlock(T, H, I // 2, w1r, s1r, w2r, s2, torch).run(d_x).float().clone())
    sync_ok()
    assert rel_err((parts[0] + parts[1]).cpu().numpy(), want) <= 6e-2


def test_ffn_workspace_is_checked(backend):
    import torch
    x = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(backend.BackendError, match="workspace"):
        backend.ffn_block(256, 256, 1024, x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 1024)
    assert backend.ffn_workspace_bytes(8192, 4096, 16384) > 8192 * 16384 * 3


@pytest.mark.parametrize("world", [2, 4])
def test_ffn_peer_exchange_emulated_on_one_gpu(backend, oracle_lib, world):
    # The tensor-parallel block without a library collective, all ranks played in turn by this process on one GPU (the
    # kernels never wait on one another, so that is legitimate): every rank's second GEMM scatters its partial rows into the
    # owners' receive buffers, then every rank reduces what it received and stores its rows into every rank's output.
    # Bit-exact against the fp32 sum of the per-rank partials of the ordinary block, and within the fp8 tolerance of the oracle.
    import torch
    from pyc_b200 import ffn
    from gpu_util import rel_err, sync_ok
    T, H, I = 512, 1024, 4096
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(T, H, I)
    X = torch.from_numpy(xb.view(np.int16)).cuda()
    rows = T // world
    recv = [torch.zeros((world, rows, H), dtype=torch.int16, device="cuda") for _ in range(world)]
    outs = [torch.zeros((T, H), dtype=torch.int16, device="cuda") for _ in range(world)]
    partial_sum = torch.zeros((T, H), dtype=torch.float32, device="cuda")
    keep = []
    for r in range(world):
        w1r, s1r, w2r = ffn.shard_weights(w1, s1, w2, r, world)
        d = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (w1r, s1r.astype(np.float32), w2r, s2.astype(np.float32))]
        keep.append(d)
        ws_bytes = backend.ffn_workspace_bytes(T, H, I // world)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        backend.ffn_block_scatter(T, H, I // world, X.data_ptr(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                                  ws.data_ptr(), ws_bytes, [t.data_ptr() for t in recv], r)
        part = torch.zeros((T, H), dtype=torch.int16, device="cuda")
        backend.ffn_block(T, H, I // world, X.data_ptr(), d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(),
                          part.data_ptr(), ws.data_ptr(), ws_bytes)
        partial_sum += part.view(torch.bfloat16).float()      # same order as the reduction kernel: rank 0, 1, ...
        # the scatter put exactly this rank's partial rows into slot r of each owner
        for o in range(world):
            assert torch.equal(recv[o][r], part[o * rows:(o + 1) * rows])
    for r in range(world):
        backend.tp_reduce_broadcast(recv[r].data_ptr(), [t.data_ptr() for t in outs], r, rows, H)
    sync_ok()
    want_bits = partial_sum.to(torch.bfloat16).view(torch.int16)
    for o in outs:
        assert torch.equal(o, want_bits)
    ref = oracle.ffn_reference(oracle_lib, workloads.bf16_bits_to_f32(xb), w1, s1, w2, s2)
    got = workloads.bf16_bits_to_f32(outs[0].cpu().numpy().view(np.uint16))
    assert rel_err(got, ref) <= 6e-2
