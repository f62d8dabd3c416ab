"""GPU (one device is enough): pyc_b200_ffn_block_tp calls the collective through PyC's pyc_collective_comm vtable
(include/pyc/collective_comm.h:30-42) exactly once per block, with the bf16 dtype, the sum op, the partial-sum buffer in
place and the caller's stream; and the full-size benchmark configuration 5 (tokens 8192, hidden 4096, inner 16384) is
checked against the CPU oracle on sampled token rows at the fp8 tolerance (6e-2)."""
import ctypes as C

import numpy as np
import pytest

import oracle
from pyc_b200 import abi, workloads

pytestmark = pytest.mark.gpu

ALL_REDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p)


class _Vtable(C.Structure):
    _fields_ = [("backend_ctx", C.c_void_p), ("all_reduce", ALL_REDUCE_FN)] + [(n, C.c_void_p) for n in
                ("all_gather", "reduce_scatter", "broadcast", "send", "recv", "barrier")]


def test_tp_entry_calls_the_vtable_once_with_bf16_sum(backend, oracle_lib):
    import torch
    from gpu_util import rel_err, sync_ok
    T, H, I = 256, 256, 1024
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(T, H, I)
    calls = []

    @ALL_REDUCE_FN
    def fake_all_reduce(ctx, comm, send, recv, count, dtype, op, stream):
        calls.append((ctx, comm, send, recv, count, dtype, op, stream))
        return 0

    vt = _Vtable(backend_ctx=0x1234, all_reduce=fake_all_reduce)
    dev = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (w1[:, :I // 2], s1[:I // 2].astype(np.float32), w2[:I // 2], s2.astype(np.float32))]
    X = torch.from_numpy(xb.view(np.int16)).cuda()
    out = torch.zeros((T, H), dtype=torch.int16, device="cuda")
    ws_bytes = backend.ffn_workspace_bytes(T, H, I // 2)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    backend.ffn_block_tp(T, H, I // 2, X.data_ptr(), dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), out.data_ptr(),
                         ws.data_ptr(), ws_bytes, C.addressof(vt), 0xBEEF, 2, 0, stream=stream.cuda_stream)
    sync_ok()
    assert len(calls) == 1
    ctx, comm, send, recv, count, dtype, op, st = calls[0]
    assert (ctx, comm, send, recv, count) == (0x1234, 0xBEEF, out.data_ptr(), out.data_ptr(), T * H)
    assert dtype == abi.DTYPE_BF16 and op == 0 and st == stream.cuda_stream      # PYC_DTYPE_BF16, PYC_REDUCE_SUM
    # what was handed to the collective is this rank's partial sum of the block
    half = oracle.ffn_reference(oracle_lib, workloads.bf16_bits_to_f32(xb), w1[:, :I // 2], s1[:I // 2], w2[:I // 2], s2)
    assert rel_err(workloads.bf16_bits_to_f32(out.cpu().numpy().view(np.uint16)), half) <= 6e-2
    # a failing collective is an error of the call, with the status in the message
    calls.clear()

    @ALL_REDUCE_FN
    def failing(ctx, comm, send, recv, count, dtype, op, stream):
        return 2

    vt2 = _Vtable(backend_ctx=0, all_reduce=failing)
    with pytest.raises(backend.BackendError, match="pyc_comm_status 2"):
        backend.ffn_block_tp(T, H, I // 2, X.data_ptr(), dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), out.data_ptr(),
                             ws.data_ptr(), ws_bytes, C.addressof(vt2), 0xBEEF, 2, 0)
    with pytest.raises(backend.BackendError, match="needs a collective vtable"):
        backend.ffn_block_tp(T, H, I // 2, X.data_ptr(), dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), out.data_ptr(),
                             ws.data_ptr(), ws_bytes, None, None, 2, 0)
    torch.cuda.synchronize()


def test_config5_full_size_against_the_oracle_on_sampled_rows(backend, oracle_lib):
    """tokens 8192, hidden 4096 -> 16384 -> 4096: the whole block on the GPU, 72 token rows (first, last, 128/256-row tile
    edges, random) recomputed by the oracle; also the LayerNorm-quantise of those rows and the 16384-wide re-quantise."""
    import torch
    from gpu_util import rel_err, sync_ok
    from pyc_b200 import ffn
    T, H, I = 8192, 4096, 16384
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(T, H, I)
    rng = np.random.default_rng(55)
    rows = sorted(set([0, 1, 127, 128, 255, 256, 4095, 4096, T - 129, T - 128, T - 1] + rng.integers(0, T, 61).tolist()))
    x_rows = workloads.bf16_bits_to_f32(xb[rows])
    blk = ffn.FfnBlock(T, H, I, w1, s1, w2, s2, torch)
    X = torch.from_numpy(xb.view(np.int16)).cuda()
    for _ in range(2):
        out = blk.run(X)
    sync_ok()
    want = oracle.ffn_reference(oracle_lib, x_rows, w1, s1, w2, s2)
    got = out[rows].float().cpu().numpy()
    err = rel_err(got, want)
    assert err <= 6e-2, f"config 5 full size: rel err {err:.3e}"
    assert np.isfinite(out.float().sum().item())
    # the two quantisers at their config-5 widths, same rows, against the oracle's LayerNorm / the GPU's own GELU output
    d_q = torch.zeros((T, H), dtype=torch.uint8, device="cuda"); d_s = torch.zeros(T, dtype=torch.float32, device="cuda")
    backend.layernorm_quantize(X.data_ptr(), None, None, d_q.data_ptr(), d_s.data_ptr(), T, H)
    sync_ok()
    ln = oracle_lib.layernorm(x_rows)
    scale = d_s[rows].cpu().numpy(); q = workloads.e4m3_decode(d_q[rows].cpu().numpy())
    np.testing.assert_allclose(scale, np.abs(ln).max(-1) / 448.0, rtol=2e-5)
    bound = np.maximum(np.abs(ln) * 2.0 ** -4, scale[:, None] * 2.0 ** -10) * 1.01 + 1e-6
    assert (np.abs(q * scale[:, None] - ln) <= bound).all()
    hb = workloads.to_bf16_bits(workloads.normal((len(rows), I), 77, 1.5)); h = workloads.bf16_bits_to_f32(hb)
    d_h = torch.from_numpy(hb.view(np.int16)).cuda()
    d_q2 = torch.zeros((len(rows), I), dtype=torch.uint8, device="cuda"); d_s2 = torch.zeros(len(rows), dtype=torch.float32, device="cuda")
    backend.quantize_rows(d_h.data_ptr(), d_q2.data_ptr(), d_s2.data_ptr(), len(rows), I)
    backend.layernorm_quantize(d_h.data_ptr(), None, None, d_q.data_ptr(), d_s.data_ptr(), len(rows), I)   # the widest LayerNorm form
    sync_ok()
    sc2 = d_s2.cpu().numpy(); q2 = workloads.e4m3_decode(d_q2.cpu().numpy())
    np.testing.assert_allclose(sc2, np.abs(h).max(-1) / 448.0, rtol=1e-5)
    assert (np.abs(q2 * sc2[:, None] - h) <= np.maximum(np.abs(h) * 2.0 ** -4, sc2[:, None] * 2.0 ** -10) * 1.01 + 1e-6).all()
    ln_w = oracle_lib.layernorm(h)
    sc3 = d_s[:len(rows)].cpu().numpy(); q3 = workloads.e4m3_decode(d_q.view(-1)[:len(rows) * I].view(len(rows), I).cpu().numpy())
    np.testing.assert_allclose(sc3, np.abs(ln_w).max(-1) / 448.0, rtol=2e-5)
    assert (np.abs(q3 * sc3[:, None] - ln_w) <= np.maximum(np.abs(ln_w) * 2.0 ** -4, sc3[:, None] * 2.0 ** -10) * 1.01 + 1e-6).all()
    blk.close()
