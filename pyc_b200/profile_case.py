"""Run one kernel of the library a few times on seeded inputs, for profilers.

    python -m pyc_b200.profile_case gemm --dtype bf16 --m 8192 --n 8192 --k 2048 --epilogue bias_gelu --iters 3
    python -m pyc_b200.profile_case layernorm --dtype bf16 --rows 16384 --cols 8192 --iters 3

Prints the mean device time per launch (CUDA events).  Under a profiler use few
iterations and a shape that keeps a few hundred MB on the device.
"""
import argparse

import numpy as np
import torch

from . import abi, backend, workloads

DT = {"bf16": abi.DTYPE_BF16, "f16": abi.DTYPE_F16, "f32": abi.DTYPE_F32}


def _dev(dtype, shape, seed, std):
    x = workloads.normal(shape, seed, std)
    if dtype == abi.DTYPE_F32:
        return torch.from_numpy(x).cuda()
    if dtype == abi.DTYPE_BF16:
        return torch.from_numpy(workloads.to_bf16_bits(x).view(np.int16)).cuda()
    return torch.from_numpy(x.astype(np.float16).view(np.int16)).cuda()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "add", "bias_gelu", "layernorm", "softmax", "reduce_sum", "attention", "conv2d", "ffn", "gemm_fp8", "latency"])
    ap.add_argument("--dtype", default="bf16", choices=list(DT))
    ap.add_argument("--m", type=int, default=8192); ap.add_argument("--n", type=int, default=8192); ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=16384); ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--batch-heads", type=int, default=32); ap.add_argument("--seq", type=int, default=2048); ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--causal", type=int, default=1)
    ap.add_argument("--conv", default="64,56,56,64,64", help="N,H,W,C,K (3x3, pad 1, stride 1)")
    ap.add_argument("--epilogue", default="bias_gelu", choices=["none", "bias_relu", "bias_gelu"])
    ap.add_argument("--tokens", type=int, default=8192); ap.add_argument("--hidden", type=int, default=4096); ap.add_argument("--inner", type=int, default=16384)
    ap.add_argument("--chunks", type=int, default=None, help="ffn: row slices whose all-reduce overlaps the next slice (default: 4 when tensor parallel)")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer"], help="ffn under torchrun: NCCL all-reduce or stores into peer memory")
    ap.add_argument("--symbol", default=None)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    a = ap.parse_args()
    dt = DT[a.dtype]
    import os
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend.load()
    es = abi.DTYPE_SIZE[dt]
    if a.op == "gemm":
        A, B, bias = _dev(dt, (a.m, a.k), 1, 0.02), _dev(dt, (a.k, a.n), 2, 0.02), _dev(dt, (a.n,), 3, 0.02)
        D = torch.zeros((a.m, a.n), dtype=A.dtype, device="cuda")
        mode = abi.ADD_NONE if a.epilogue == "none" else abi.ADD_ROW_BIAS
        act = {"none": abi.ACT_NONE, "bias_relu": abi.ACT_RELU, "bias_gelu": abi.ACT_GELU}[a.epilogue]
        run = lambda: backend.gemm(dt, a.m, a.n, a.k, A.data_ptr(), B.data_ptr(), D.data_ptr(), add=bias.data_ptr(), add_mode=mode, act=act, symbol=a.symbol)
        work = ("TFLOP/s", 2.0 * a.m * a.n * a.k / 1e12)
    elif a.op in ("add", "bias_gelu", "layernorm", "softmax", "reduce_sum"):
        X = _dev(dt, (a.rows, a.cols), 4, 1.0); Y = _dev(dt, (a.rows, a.cols), 5, 1.0); bias = _dev(dt, (a.cols,), 6, 1.0)
        O = torch.zeros_like(X); n = a.rows * a.cols
        run = {"add": lambda: backend.add(dt, X.data_ptr(), Y.data_ptr(), O.data_ptr(), n),
               "bias_gelu": lambda: backend.bias_act(dt, X.data_ptr(), bias.data_ptr(), abi.ADD_ROW_BIAS, abi.ACT_GELU, O.data_ptr(), a.rows, a.cols),
               "layernorm": lambda: backend.layernorm(dt, X.data_ptr(), None, None, O.data_ptr(), a.rows, a.cols),
               "softmax": lambda: backend.softmax(dt, X.data_ptr(), O.data_ptr(), a.rows, a.cols),
               "reduce_sum": lambda: backend.reduce_sum(dt, X.data_ptr(), O.data_ptr(), a.rows, a.cols)}[a.op]
        nbytes = {"add": 3, "reduce_sum": 1}.get(a.op, 2) * n * es
        work = ("GB/s", nbytes / 1e9)
    elif a.op == "latency":
        # benchmark configuration 1: the 512^3 fp32 matmul -> add(bias) -> relu module through pyc_cuda_dispatch, device tensors;
        # wall-clock per call (graph replay + stream sync), p50 / p95 over --iters calls
        import time
        from . import ir
        x, w, b = workloads.gemm_inputs(1, a.m, a.k, a.n, ("uniform", -1.0, 1.0))
        dev = [torch.from_numpy(t).cuda() for t in (x, w, b)]
        out = torch.zeros((a.m, a.n), dtype=torch.float32, device="cuda")
        host = [torch.from_numpy(t).pin_memory() for t in (x, w, b)]; hout = torch.zeros((a.m, a.n), dtype=torch.float32).pin_memory()
        module = ir.matmul_bias_act(abi.DTYPE_F32, a.m, a.k, a.n, bias="row", act="relu")
        def tens(ts, o):
            return ([backend.make_tensor(t.data_ptr(), t.numel() * 4, abi.DTYPE_F32, tuple(t.shape)) for t in ts],
                    [backend.make_tensor(o.data_ptr(), o.numel() * 4, abi.DTYPE_F32, (a.m, a.n))])
        for label, (ins, outs) in (("device tensors", tens(dev, out)), ("pinned host tensors", tens(host, hout))):
            for _ in range(20):
                backend.dispatch(module, ins, outs)
            ts = []
            for _ in range(a.iters):
                t0 = time.perf_counter(); st, trace = backend.dispatch(module, ins, outs); ts.append((time.perf_counter() - t0) * 1e6)
            ts.sort()
            print(f"latency f32 {a.m}x{a.k}x{a.n} {label}: p50 {ts[len(ts) // 2]:.1f} us  p95 {ts[int(len(ts) * 0.95)]:.1f} us  min {ts[0]:.1f} us  ({trace.reason.decode()})")
        return
    elif a.op == "gemm_fp8":
        A = torch.randint(0, 120, (a.m, a.k), dtype=torch.uint8, device="cuda"); B = torch.randint(0, 120, (a.k, a.n), dtype=torch.uint8, device="cuda")
        rs = torch.ones(a.m, device="cuda"); cs = torch.ones(a.n, device="cuda"); D = torch.zeros((a.m, a.n), dtype=torch.int16, device="cuda")
        run = lambda: backend.gemm_fp8(a.m, a.n, a.k, A.data_ptr(), B.data_ptr(), D.data_ptr(), rs.data_ptr(), cs.data_ptr(), None, abi.ACT_GELU)
        work = ("TFLOP/s", 2.0 * a.m * a.n * a.k / 1e12)
    elif a.op == "ffn":
        # benchmark configuration 5; with WORLD_SIZE > 1 (torchrun) the inner dimension is sharded and one all-reduce ends the block
        from . import ffn
        xb, w1, s1, w2, s2 = workloads.ffn_inputs(a.tokens, a.hidden, a.inner)
        w1r, s1r, w2r = ffn.shard_weights(w1, s1, w2, rank, world)
        blk = ffn.FfnBlock(a.tokens, a.hidden, a.inner // world, w1r, s1r, w2r, s2, torch, chunks=a.chunks, exchange=a.exchange)
        X = torch.from_numpy(xb.view(np.int16)).cuda()
        run = lambda: blk.run(X)
        work = ("TFLOP/s (whole block, all ranks)", 4.0 * a.tokens * a.hidden * a.inner / 1e12)
        if world > 1 and a.exchange == "peer":
            # same inputs through the NCCL variant: the two exchanges must agree to bf16 rounding of the sum
            ref = ffn.FfnBlock(a.tokens, a.hidden, a.inner // world, w1r, s1r, w2r, s2, torch).run(X).float()
            got = blk.run(X).float()
            torch.cuda.synchronize()
            err = float((got - ref).abs().max() / ref.abs().max())
            print(f"rank {rank}: peer exchange vs NCCL all-reduce: max |diff| / max |ref| = {err:.3e}", flush=True)
            assert err < 2e-2, err
    elif a.op == "attention":
        shape = (a.batch_heads, a.seq, a.d)
        Q, K_, V = _dev(dt, shape, 7, 1.0), _dev(dt, shape, 8, 1.0), _dev(dt, shape, 9, 1.0); O = torch.zeros_like(Q)
        run = lambda: backend.attention(dt, a.batch_heads, a.seq, a.d, Q.data_ptr(), K_.data_ptr(), V.data_ptr(), O.data_ptr(), a.d ** -0.5, a.causal)
        pairs = a.seq * (a.seq + 1) / 2 if a.causal else a.seq * a.seq
        work = ("TFLOP/s", 4.0 * a.batch_heads * a.d * pairs / 1e12)
    else:
        N, H, W, C, K = [int(v) for v in a.conv.split(",")]
        X = _dev(dt, (N, H, W, C), 10, 1.0); Wt = _dev(dt, (K, 3, 3, C), 11, (2.0 / (9 * C)) ** 0.5); b = _dev(dt, (K,), 12, 0.1)
        O = torch.zeros((N, H, W, K), dtype=X.dtype, device="cuda")
        run = lambda: backend.conv2d(dt, N, H, W, C, K, 3, 3, (1, 1), (1, 1), X.data_ptr(), Wt.data_ptr(), b.data_ptr(), True, O.data_ptr())
        work = ("TFLOP/s", 2.0 * N * H * W * C * K * 9 / 1e12)
    for _ in range(a.warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    assert backend.device_status() == 0
    ms = e0.elapsed_time(e1) / a.iters
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t[0])
        torch.distributed.barrier()
        if a.op == "ffn" and getattr(blk, "peer", None) is not None:
            blk.peer.close()
        torch.distributed.destroy_process_group()
        if rank != 0:
            return
    print(f"{a.op} {a.dtype} x{world}: {ms:.4f} ms/launch, {work[1] / (ms * 1e-3):.1f} {work[0]}")


if __name__ == "__main__":
    main()
