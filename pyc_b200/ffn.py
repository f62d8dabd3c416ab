"""Host side of the tensor-parallel FFN block (benchmark configuration 5).

    y = gelu(layernorm(x) @ W1) @ W2      x [T,H] bf16, W1 [H,I], W2 [I,H] fp8 e4m3 + per-output-channel fp32 scales

Partitioning (Megatron style): rank r of g holds the column slice W1[:, r*I/g:(r+1)*I/g] with its scales and the row
slice W2[r*I/g:(r+1)*I/g, :]; the LayerNorm input is replicated; GELU is local; every rank produces a partial [T,H]
and ONE all-reduce (sum, bf16) per block finishes it.  Two ways to do that all-reduce:

  * exchange="nccl": pyc_b200_ffn_block_tp -- the block, then one all_reduce through PyC's collective vtable
    (include/pyc/collective_comm.h:30-42), served by libpyc_b200_comm_nccl.so (NCCL over NVLink, bf16 mapped);
  * exchange="peer": no library collective.  The second GEMM's epilogue stores each row of the partial sum straight into
    the receive buffer of the rank that owns the row (reduce-scatter by plain stores into peer memory, overlapped with the
    GEMM tile by tile), a reduction kernel adds the received slices and stores the owned rows into every rank's output
    (the all-gather, again plain peer stores).  Ranks are ordered by two stream barriers (the vtable's barrier, on the
    same stream as the kernels); no kernel waits on another GPU.  Buffers are made visible to the other processes with CUDA IPC.

The compute and the collective calls are the C-ABI library; torch.distributed only carries the bootstrap (NCCL unique
id, IPC handles) between the processes.  PyC itself implements no parallel strategy: its options
struct carries world_size/rank (include/pyc/compiler_api.h:53-62) but pyc_run_model never calls a collective.
"""
import ctypes as C
import os

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


class CollectiveBackend:
    """A loaded collective backend (pyc_comm_backend_create of a shared library that implements PyC's
    pyc_collective_comm, include/pyc/collective_comm.h:93-101) plus one communicator for the ranks of `group`.

    The default library is this package's NCCL backend; the communicator is bootstrapped here (rank 0 draws the NCCL
    unique id, torch.distributed carries it to the others) because PyC expects its launcher to bring one."""

    DEFAULT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libpyc_b200_comm_nccl.so")

    def __init__(self, torch, group=None, path=None, config_json="{}"):
        dist = torch.distributed
        self.torch, self.group = torch, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        path = path or self.DEFAULT
        if not os.path.exists(path):
            raise backend.BackendError(f"{path} is missing: run `python -m pyc_b200.build`")
        L = self.lib = C.CDLL(path)
        L.pyc_comm_backend_create.argtypes = [C.c_char_p]; L.pyc_comm_backend_create.restype = C.c_void_p
        L.pyc_comm_backend_destroy.argtypes = [C.c_void_p]; L.pyc_comm_backend_destroy.restype = None
        L.pyc_b200_nccl_unique_id.argtypes = [C.c_void_p, C.c_char_p]
        L.pyc_b200_nccl_comm_init_rank.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        L.pyc_b200_nccl_comm_destroy.argtypes = [C.c_void_p, C.c_void_p]
        L.pyc_b200_nccl_last_error.argtypes = [C.c_void_p]; L.pyc_b200_nccl_last_error.restype = C.c_char_p
        self.vtable = L.pyc_comm_backend_create(config_json.encode())
        if not self.vtable:
            raise backend.BackendError("pyc_comm_backend_create returned NULL")
        ident = C.create_string_buffer(128)
        if self.rank == 0 and L.pyc_b200_nccl_unique_id(self.vtable, ident) != 0:
            raise backend.BackendError(f"NCCL unique id: {self.error()}")
        box = [ident.raw]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        handle = C.c_void_p()
        if L.pyc_b200_nccl_comm_init_rank(self.vtable, box[0], self.world, self.rank, C.byref(handle)) != 0:
            raise backend.BackendError(f"ncclCommInitRank: {self.error()}")
        self.handle = handle.value
        # the seven entry points of the vtable, for the calls this module makes itself (the barriers of the peer exchange)
        fn = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p)
        words = (C.c_void_p * 8).from_address(self.vtable)
        self._ctx, self._barrier = words[0], fn(words[7])

    def error(self):
        return (self.lib.pyc_b200_nccl_last_error(self.vtable) or b"").decode()

    def barrier(self, stream):
        st = self._barrier(self._ctx, self.handle, stream)
        if st != 0:
            raise backend.BackendError(f"collective barrier failed with pyc_comm_status {st}: {self.error()}")

    def close(self):
        if self.vtable:
            self.torch.cuda.synchronize()
            if self.handle:
                self.lib.pyc_b200_nccl_comm_destroy(self.vtable, self.handle)
            self.lib.pyc_comm_backend_destroy(self.vtable)
            self.vtable = self.handle = None


class FfnBlock:
    """Device-resident shard of one FFN block plus its workspace; call run() once per step."""

    def __init__(self, tokens, hidden, inner_local, w1, s1, w2, s2, torch, group=None, exchange="nccl", comm=None, single=False):
        self.torch, self.group = torch, group
        if exchange not in ("nccl", "peer", "multimem", "fused"):
            raise ValueError("exchange must be 'nccl', 'peer', 'multimem' or 'fused'")
        self.tokens, self.hidden, self.inner = tokens, hidden, inner_local
        dev = "cuda"
        self.w1 = torch.from_numpy(np.ascontiguousarray(w1)).to(dev)
        self.s1 = torch.from_numpy(np.ascontiguousarray(s1, dtype=np.float32)).to(dev)
        self.w2 = torch.from_numpy(np.ascontiguousarray(w2)).to(dev)
        self.s2 = torch.from_numpy(np.ascontiguousarray(s2, dtype=np.float32)).to(dev)
        dist = torch.distributed
        # single=True: the whole block on this GPU even when a process group exists (no collective, no communicator)
        self.parallel = not single and (group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1))
        self.world = dist.get_world_size(group) if self.parallel else 1
        self.rank = dist.get_rank(group) if self.parallel else 0
        self.ws_bytes = backend.ffn_workspace_bytes(tokens, hidden, inner_local)
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.out = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=dev)
        self.comm, self._own_comm, self.peer, self.switch = comm, False, None, None
        self.fused = exchange == "fused" and self.parallel
        if exchange in ("multimem", "fused") and self.parallel:
            self.switch = MultimemExchange(tokens, hidden, torch, group, fused=self.fused)      # needs no communicator
        elif self.parallel and self.comm is None:
            self.comm, self._own_comm = CollectiveBackend(torch, group), True
        if exchange == "peer" and self.parallel:
            self.peer = PeerExchange(tokens, hidden, torch, self.comm, group)

    def run(self, x_dev, stream=None):
        """x_dev: [T,H] bf16 (or int16 bit pattern) device tensor.  Every kernel, the all-reduce and the barriers are
        enqueued on `stream` (default: torch's current stream).  Returns the (all-reduced) bf16 output tensor."""
        s = stream if stream is not None else self.torch.cuda.current_stream().cuda_stream
        if self.peer is not None:
            px = self.peer
            backend.ffn_block_scatter(self.tokens, self.hidden, self.inner, x_dev.data_ptr(), self.w1.data_ptr(), self.s1.data_ptr(),
                                      self.w2.data_ptr(), self.s2.data_ptr(), self.ws.data_ptr(), self.ws_bytes, px.recv_ptrs, px.rank, stream=s)
            self.comm.barrier(s)    # every rank's slices have landed (kernel completion makes peer stores visible)
            backend.tp_reduce_broadcast(px.recv_ptrs[px.rank], px.out_ptrs, px.rank, px.rows, self.hidden, stream=s)
            self.comm.barrier(s)    # every rank has written its rows into this rank's output
            return px.out
        if self.switch is not None and self.fused:
            sw = self.switch
            backend.ffn_block_switch_reduce(self.tokens, self.hidden, self.inner, x_dev.data_ptr(), self.w1.data_ptr(), self.s1.data_ptr(),
                                            self.w2.data_ptr(), self.s2.data_ptr(), sw.out.data_ptr(), self.ws.data_ptr(), self.ws_bytes,
                                            sw.multicast_ptr, sw.unit_flag_ptrs, sw.fin_ptrs, sw.fused_epochs.data_ptr(), sw.rank, stream=s)
            return sw.out
        if self.switch is not None:
            sw = self.switch
            backend.ffn_block(self.tokens, self.hidden, self.inner, x_dev.data_ptr(), self.w1.data_ptr(), self.s1.data_ptr(),
                              self.w2.data_ptr(), self.s2.data_ptr(), sw.out.data_ptr(), self.ws.data_ptr(), self.ws_bytes, stream=s)
            backend.tp_allreduce_multimem(sw.multicast_ptr, sw.flag_ptrs, sw.epochs.data_ptr(), sw.rank, self.tokens, self.hidden, stream=s)
            return sw.out
        backend.ffn_block_tp(self.tokens, self.hidden, self.inner, x_dev.data_ptr(), self.w1.data_ptr(), self.s1.data_ptr(),
                             self.w2.data_ptr(), self.s2.data_ptr(), self.out.data_ptr(), self.ws.data_ptr(), self.ws_bytes,
                             self.comm.vtable if self.comm else None, self.comm.handle if self.comm else None, self.world, self.rank, stream=s)
        return self.out

    def capture(self, x_dev):
        """Record one run() on `x_dev` (its address is baked in) as a CUDA graph -- the four kernels, the collective or the
        peer exchange with its barriers -- and return a callable that replays it on torch's current stream and returns the
        output tensor.  Removes the launch gaps between the block's kernels (~25 us of a 0.9 ms block on one GPU, more of
        the shorter per-rank blocks).  Every rank must capture and replay in step, as with any collective."""
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):                       # first-use set-up (kernel attributes, NCCL channels) outside the capture
                self.run(x_dev, stream=side.cuda_stream)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = self.run(x_dev, stream=torch.cuda.current_stream().cuda_stream)
        self._graph, self._graph_x = graph, x_dev    # keep both alive

        def replay():
            graph.replay()
            return out
        return replay

    def close(self):
        self._graph = None
        if self.peer is not None:
            self.peer.close(); self.peer = None
        if self.switch is not None:
            self.switch.close(); self.switch = None
        if self._own_comm and self.comm is not None:
            self.comm.close(); self.comm = None


class _DeviceView:
    """A raw device allocation seen as a CUDA array (zero-copy torch.as_tensor)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3, "strides": None}


class MultimemExchange:
    """The [T][H] bf16 output of every rank bound to one NVLink multicast object, plus the flag words of the in-switch
    all-reduce kernel.  torch.distributed._symmetric_memory allocates, exchanges the handles and binds the multicast
    object; the data path is this package's kernel (multimem.ld_reduce / multimem.st on the multicast address)."""

    def __init__(self, tokens, hidden, torch, group=None, fused=False):
        import torch.distributed._symmetric_memory as symm_mem
        dist = torch.distributed
        self.torch, self.group = torch, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > backend.TP_MAX_RANKS:
            raise ValueError(f"{self.world} ranks: at most {backend.TP_MAX_RANKS}")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.out = symm_mem.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        handle = symm_mem.rendezvous(self.out, self.group)
        self.multicast_ptr = int(getattr(handle, "multicast_ptr", 0) or 0)
        if not self.multicast_ptr:
            raise backend.BackendError("no NVLink multicast address for the symmetric buffer (NVSwitch multicast is not available here)")
        self.flags = symm_mem.empty(backend.TP_MULTIMEM_BLOCKS * backend.TP_MAX_RANKS, dtype=torch.int32, device=dev)
        self.flags.zero_()
        flag_handle = symm_mem.rendezvous(self.flags, self.group)
        self.flag_ptrs = [int(p) for p in flag_handle.buffer_ptrs]
        self.epochs = torch.zeros(backend.TP_MULTIMEM_BLOCKS, dtype=torch.int32, device=dev)
        self._handles = [handle, flag_handle]
        if fused:      # per-piece flags and end-of-kernel flags of the GEMM with the reduction in its epilogue
            if tokens % 256 or hidden % 256:
                raise ValueError("the fused exchange needs tokens and hidden to be multiples of 256")
            units = (tokens // 256) * (hidden // 256) * 2      # one per CTA and tile of the pair kernel
            self.unit_flags = symm_mem.empty(units * backend.TP_MAX_RANKS, dtype=torch.int32, device=dev)
            self.unit_flags.zero_()
            h1 = symm_mem.rendezvous(self.unit_flags, self.group)
            self.fin = symm_mem.empty(backend.TP_FUSED_EPOCH_SLOTS * backend.TP_MAX_RANKS, dtype=torch.int32, device=dev)
            self.fin.zero_()
            h2 = symm_mem.rendezvous(self.fin, self.group)
            self.unit_flag_ptrs, self.fin_ptrs = [int(p) for p in h1.buffer_ptrs], [int(p) for p in h2.buffer_ptrs]
            self.fused_epochs = torch.zeros(backend.TP_FUSED_EPOCH_SLOTS, dtype=torch.int32, device=dev)
            self._handles += [h1, h2]
        torch.cuda.synchronize()
        dist.barrier(group=group)      # every rank's flag words are zero before anyone signals

    def close(self):
        # leave together and idle: no rank frees memory bound to the multicast object while another may still touch it
        self.torch.cuda.synchronize()
        self.torch.distributed.barrier(group=self.group)
        self._handles = None
        self.out = self.flags = self.epochs = None
        self.unit_flags = self.fin = self.fused_epochs = None


class PeerExchange:
    """Receive buffer [world][T/world][H] and output [T][H] (bf16) of this rank, mapped into every other rank's process."""

    def __init__(self, tokens, hidden, torch, comm, group=None):
        dist = torch.distributed
        self.torch, self.group, self.comm = torch, group, comm
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
        dist.barrier(group=group)

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
