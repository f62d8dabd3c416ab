"""Host side of the tensor-parallel FFN block (benchmark configuration 5).

    y = gelu(layernorm(x) @ W1) @ W2      x [T,H] bf16, W1 [H,I], W2 [I,H] fp8 e4m3 + per-output-channel fp32 scales

Partitioning (Megatron style): rank r of g holds the column slice W1[:, r*I/g:(r+1)*I/g] with its scales and the row
slice W2[r*I/g:(r+1)*I/g, :]; the LayerNorm input is replicated; GELU is local; every rank produces a partial [T,H]
and ONE all-reduce (sum, bf16, NCCL over NVLink) per block finishes it.  The compute is pyc_b200_ffn_block (C-ABI);
torch.distributed is only the plumbing for the collective.  PyC itself implements no parallel strategy: its options
struct carries world_size/rank (include/pyc/compiler_api.h:53-62) but pyc_run_model never calls a collective.
"""
import numpy as np

from . import backend


def shard_bounds(inner, rank, world):
    if inner % world:
        raise ValueError(f"inner dimension {inner} is not divisible by {world} ranks")
    per = inner // world
    return rank * per, (rank + 1) * per


def shard_weights(w1, s1, w2, rank, world, b1=None):
    """Contiguous per-rank slices of (W1 [H,I], s1 [I], W2 [I,H]) and optionally b1 [I]."""
    lo, hi = shard_bounds(w1.shape[1], rank, world)
    out = (np.ascontiguousarray(w1[:, lo:hi]), np.ascontiguousarray(s1[lo:hi]), np.ascontiguousarray(w2[lo:hi, :]))
    return out + ((np.ascontiguousarray(b1[lo:hi]),) if b1 is not None else ())


class FfnBlock:
    """Device-resident shard of one FFN block plus its workspace; call run() once per step.

    With more than one rank the tokens can be processed in `chunks` row slices: the all-reduce of slice i runs on a
    second stream while slice i+1 is still in its GEMMs.  Measured on 2/4/8 B200s this loses to the unsliced block
    (four times the launches, smaller GEMMs, one NCCL call per slice: 0.79 vs 0.64 ms at 2 ranks), so the default is 1."""

    def __init__(self, tokens, hidden, inner_local, w1, s1, w2, s2, torch, group=None, chunks=None):
        self.torch, self.group = torch, group
        self.tokens, self.hidden, self.inner = tokens, hidden, inner_local
        dev = "cuda"
        self.w1 = torch.from_numpy(np.ascontiguousarray(w1)).to(dev)
        self.s1 = torch.from_numpy(np.ascontiguousarray(s1, dtype=np.float32)).to(dev)
        self.w2 = torch.from_numpy(np.ascontiguousarray(w2)).to(dev)
        self.s2 = torch.from_numpy(np.ascontiguousarray(s2, dtype=np.float32)).to(dev)
        dist = torch.distributed
        self.parallel = group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1)
        if chunks is None:
            chunks = 1
        if tokens % chunks:
            raise ValueError(f"{tokens} tokens do not split into {chunks} equal chunks")
        self.chunks, self.rows = chunks, tokens // chunks
        self.ws_bytes = backend.ffn_workspace_bytes(self.rows, hidden, inner_local)
        # one workspace per chunk in flight: chunk i+1 may start while chunk i's output is still being reduced,
        # but its scratch is free as soon as its last GEMM has been issued on the same stream
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.out = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=dev)
        self.comm_stream = torch.cuda.Stream() if self.parallel and chunks > 1 else None

    def run(self, x_dev, stream=None):
        """x_dev: [T,H] bf16 (or int16 bit pattern) device tensor.  Returns the (all-reduced) bf16 output tensor."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        s = stream if stream is not None else cur.cuda_stream
        row_bytes = self.hidden * 2
        for c in range(self.chunks):
            off = c * self.rows
            backend.ffn_block(self.rows, self.hidden, self.inner, x_dev.data_ptr() + off * row_bytes, self.w1.data_ptr(), self.s1.data_ptr(),
                              self.w2.data_ptr(), self.s2.data_ptr(), self.out.data_ptr() + off * row_bytes, self.ws.data_ptr(), self.ws_bytes, stream=s)
            if not self.parallel:
                continue
            part = self.out[off:off + self.rows]
            if self.comm_stream is None:
                torch.distributed.all_reduce(part, group=self.group)
            else:
                ev = torch.cuda.Event()
                ev.record(cur)
                self.comm_stream.wait_event(ev)
                with torch.cuda.stream(self.comm_stream):
                    torch.distributed.all_reduce(part, group=self.group)
        if self.comm_stream is not None:
            cur.wait_stream(self.comm_stream)
        return self.out
