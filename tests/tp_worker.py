"""Worker for the multi-GPU tensor-parallel FFN test: one process per GPU (torchrun), benchmark configuration 5's block
with the inner dimension sharded over the ranks.  All four exchanges run -- the all-reduce through PyC's collective vtable
(NCCL backend), the peer-store exchange, the in-switch (multimem) all-reduce and the GEMM with that reduction fused into its
epilogue -- and EACH result is compared with the CPU oracle's unsharded block on sampled
token rows (fp8 tolerance 6e-2, norm-wise).  Prints one line per rank and exchange that the test parses.

    python -m torch.distributed.run --nproc-per-node 2 ... tests/tp_worker.py --tokens 1024 --hidden 1024 --inner 4096
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402  (checker)
from pyc_b200 import backend, ffn, workloads  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024); ap.add_argument("--hidden", type=int, default=1024); ap.add_argument("--inner", type=int, default=4096)
    ap.add_argument("--rows", type=int, default=48, help="token rows compared with the oracle")
    ap.add_argument("--exchanges", default="nccl,peer,multimem,fused")
    a = ap.parse_args()
    world, rank, local = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    backend.load()
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(a.tokens, a.hidden, a.inner)
    rng = np.random.default_rng(5)
    per = a.tokens // world
    rows = sorted(set([0, a.tokens - 1] + [r * per + d for r in range(world) for d in (0, per - 1)] +
                      rng.integers(0, a.tokens, a.rows).tolist()))
    want = oracle.ffn_reference(oracle.Oracle(), workloads.bf16_bits_to_f32(xb[rows]), w1, s1, w2, s2)
    w1r, s1r, w2r = ffn.shard_weights(w1, s1, w2, rank, world)
    X = torch.from_numpy(xb.view(np.int16)).cuda()
    comm = ffn.CollectiveBackend(torch)
    ok = True
    full = {}
    for exchange in a.exchanges.split(","):
        try:
            blk, why = ffn.FfnBlock(a.tokens, a.hidden, a.inner // world, w1r, s1r, w2r, s2, torch, exchange=exchange, comm=comm), ""
        except Exception as exc:                  # a machine without NVLink multicast has no in-switch exchanges
            if exchange not in ("multimem", "fused"):
                raise
            blk, why = None, f"{type(exc).__name__}: {exc}"
        have = torch.tensor([1 if blk is not None else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(have, op=dist.ReduceOp.MIN)
        if int(have[0]) == 0:                     # every rank skips it together
            if blk is not None:
                blk.close()
            print(f"tp_worker rank {rank}/{world} exchange {exchange}: unavailable ({why[:120]})", flush=True)
            continue
        for _ in range(3):                     # repeated calls: the in-switch exchange advances its epoch counters each time
            out = blk.run(X)
        torch.cuda.synchronize()
        status = backend.device_status()
        if exchange in ("multimem", "fused") and status == 0:   # ...and a captured graph replays with the counters it finds
            replay = blk.capture(X)
            for _ in range(2):
                out = replay()
            torch.cuda.synchronize()
            status = backend.device_status()
        if status != 0:                        # no assert here: every rank leaves through the orderly shutdown below
            print(f"tp_worker rank {rank}/{world} exchange {exchange}: device status {status:#x}", flush=True)
            ok = False
        full[exchange] = out.clone()
        if exchange == "fused" and "multimem" in full:
            # the same partial sums reduced by the same switch operation: the two results must agree in every element
            same = bool(torch.equal(full["fused"].view(torch.int16), full["multimem"].view(torch.int16)))
            print(f"tp_worker rank {rank}/{world} fused == multimem in every element: {same}", flush=True)
            ok = ok and same
        got = out[rows].float().cpu().numpy()
        err = float(np.abs(got - want).max() / np.abs(want).max())
        print(f"tp_worker rank {rank}/{world} exchange {exchange}: max_rel_err_vs_oracle {err:.4e} rows {len(rows)}", flush=True)
        ok = ok and err <= 6e-2
        dist.barrier()
        blk.close()
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
