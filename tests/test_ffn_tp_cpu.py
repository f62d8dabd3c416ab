"""CPU: the host-side logic of the tensor-parallel FFN block (weight sharding + one sum all-reduce) with two gloo
ranks.  The compute on each rank is the CPU oracle's definition of the block, so this checks the partitioning
algebra the GPU path relies on: sum over ranks of the partial blocks == the unsharded block."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from pyc_b200 import ffn, workloads

T, H, I = 48, 64, 256


def _problem():
    xb, w1, s1, w2, s2 = workloads.ffn_inputs(T, H, I)
    return workloads.bf16_bits_to_f32(xb), w1, s1, w2, s2


def _rank_main(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = oracle.Oracle(threads=1)
        x, w1, s1, w2, s2 = _problem()
        w1r, s1r, w2r = ffn.shard_weights(w1, s1, w2, rank, world)
        assert w1r.shape == (H, I // world) and w2r.shape == (I // world, H) and w1r.flags["C_CONTIGUOUS"]
        partial = torch.from_numpy(oracle.ffn_reference(orc, x, w1r, s1r, w2r, s2))
        dist.all_reduce(partial)  # the one collective of the block
        full = oracle.ffn_reference(orc, x, w1, s1, w2, s2)
        err = float(np.abs(partial.numpy() - full).max() / np.abs(full).max())
        if rank == 0:
            results.put(err)
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_ffn_matches_unsharded():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert results.get(timeout=10) <= 1e-5   # fp32 partial sums, only the summation order differs


def test_shard_bounds_and_errors():
    assert ffn.shard_bounds(16384, 3, 8) == (6144, 8192)
    with pytest.raises(ValueError):
        ffn.shard_bounds(100, 0, 8)
    codes = workloads.e4m3_encode(np.array([0.0, 448.0, -448.0, 1e9, 0.0156, 17.0], np.float32))
    assert workloads.e4m3_decode(codes).tolist() == [0.0, 448.0, -448.0, 448.0, 0.015625, 16.0]
