"""Host side of the tensor-parallel FFN block (benchmark configuration 5).

    y = gelu(layernorm(x) @ W1) @ W2      x [T,H] bf16, W1 [H,I], W2 [I,H] fp8 e4m3 + per-output-channel fp32 scales

Partitioning (Megatron style): rank r of g holds the column slice W1[:, r*I/g:(r+1)*I/g] with its scales and the row
slice W2[r*I/g:(r+1)*I/g, :]; the LayerNorm input is replicated; GELU is local; every rank produces a partial [T,H]
and ONE all-reduce (sum, bf16) per block finishes it.  Two ways to do that all-reduce:

  * exchange="nccl": pyc_b200_ffn_block, then torch.distributed.all_reduce (NCCL over NVLink);
  * exchange="peer": no library collective.  The second GEMM's epilogue stores each row of the partial sum straight into
    the receive buffer of the rank that owns the row (reduce-scatter by plain stores into peer memory, overlapped with the
    GEMM tile by tile), a reduction kernel adds the received slices and stores the owned rows into every rank's output
    (the all-gather, again plain peer stores).  Ranks are ordered by two stream barriers (a one-element NCCL all-reduce
    each); no kernel waits on another GPU.  Buffers are made visible to the other processes with CUDA IPC.

The compute is the C-ABI library; torch.distributed is the plumbing (handle exchange, barriers, the NCCL variant).  PyC itself implements no parallel strategy: its options
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

    def __init__(self, tokens, hidden, inner_local, w1, s1, w2, s2, torch, group=None, chunks=None, exchange="nccl"):
        self.torch, self.group = torch, group
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
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
        self.peer = None
        if exchange == "peer" and self.parallel:
            if chunks != 1:
                raise ValueError("exchange='peer' works on the whole block (chunks=1)")
            self.peer = PeerExchange(tokens, hidden, torch, group)

    def run(self, x_dev, stream=None):
        """x_dev: [T,H] bf16 (or int16 bit pattern) device tensor.  Returns the (all-reduced) bf16 output tensor."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        s = stream if stream is not None else cur.cuda_stream
        row_bytes = self.hidden * 2
        if self.peer is not None:
            px = self.peer
            backend.ffn_block_scatter(self.tokens, self.hidden, self.inner, x_dev.data_ptr(), self.w1.data_ptr(), self.s1.data_ptr(),
                                      self.w2.data_ptr(), self.s2.data_ptr(), self.ws.data_ptr(), self.ws_bytes, px.recv_ptrs, px.rank, stream=s)
            px.barrier()            # every rank's slices have landed (kernel completion makes peer stores visible)
            backend.tp_reduce_broadcast(px.recv_ptrs[px.rank], px.out_ptrs, px.rank, px.rows, self.hidden, stream=s)
            px.barrier()            # every rank has written its rows into this rank's output
            return px.out
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


class _DeviceView:
    """A raw device allocation seen as a CUDA array (zero-copy torch.as_tensor)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3, "strides": None}


class PeerExchange:
    """Receive buffer [world][T/world][H] and output [T][H] (bf16) of this rank, mapped into every other rank's process."""

    def __init__(self, tokens, hidden, torch, group=None):
        dist = torch.distributed
        self.torch, self.group = torch, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if tokens % self.world:
            raise ValueError(f"{tokens} tokens do not split over {self.world} ranks")
        self.rows = tokens // self.world
        nbytes = tokens * hidden * 2
        self._own = [backend.symm_alloc(nbytes), backend.symm_alloc(nbytes)]     # (ptr, handle): receive buffer, output
        handles = [None] * self.world
        dist.all_gather_object(handles, (self._own[0][1], self._own[1][1]), group=group)
        self._opened = []
        self.recv_ptrs, self.out_ptrs = [], []
        for r, (h_recv, h_out) in enumerate(handles):
            if r == self.rank:
                self.recv_ptrs.append(self._own[0][0]); self.out_ptrs.append(self._own[1][0])
            else:
                p_recv, p_out = backend.symm_open(h_recv), backend.symm_open(h_out)
                self._opened += [p_recv, p_out]
                self.recv_ptrs.append(p_recv); self.out_ptrs.append(p_out)
        self.out = torch.as_tensor(_DeviceView(self._own[1][0], (tokens, hidden), "<i2"), device="cuda").view(torch.bfloat16)
        self._token = torch.zeros(1, dtype=torch.float32, device="cuda")
        dist.barrier(group=group)

    def barrier(self):
        # stream-ordered: completes on this rank's stream only after every rank's stream has reached its own call
        self.torch.distributed.all_reduce(self._token, op=self.torch.distributed.ReduceOp.MAX, group=self.group)

    def close(self):
        self.torch.cuda.synchronize()
        self.torch.distributed.barrier(group=self.group)
        for p in self._opened:
            backend.symm_close(p)
        self._opened = []
        self.torch.distributed.barrier(group=self.group)
        for ptr, _ in self._own:
            backend.symm_free(ptr)
        self._own = []
