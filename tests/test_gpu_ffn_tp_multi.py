"""GPU, two processes on two GPUs: the tensor-parallel FFN block with the exchange done by stores into peer memory
(CUDA IPC mapped receive buffers, two stream barriers) against the same block with an NCCL all-reduce.  Skipped on a
machine with one GPU; the kernels themselves are covered there by the one-GPU emulation in test_gpu_ffn_fp8.py."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus():
    import torch
    return torch.cuda.device_count()


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_peer_exchange_matches_nccl_on_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", "-m", "pyc_b200.profile_case", "ffn", "--tokens", "1024", "--hidden", "1024", "--inner", "4096",
           "--iters", "3", "--warmup", "1", "--exchange", "peer"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    agree = [l for l in r.stdout.splitlines() if "peer exchange vs NCCL all-reduce" in l]
    assert len(agree) == 2, r.stdout[-2000:]          # both ranks compared and passed their own assertion
    assert any(l.startswith("ffn bf16 x2") for l in r.stdout.splitlines())
