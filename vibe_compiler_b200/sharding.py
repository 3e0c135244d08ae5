"""Host-side partitioning for multi-GPU runs of the hot path (one process per GPU).

Independent units (FA: batch x head; FD with many sequences: batch x kv-head; GEMM: row blocks) are
dealt out in contiguous blocks with no data-path collective. The long-context decode shards the KV
sequence instead: every rank computes the un-finalized (acc, m, l) state of its contiguous KV range,
the states are all-gathered and left-folded in ascending shard order - the fold order of the
reference's spatial flash-decoding materialisation
(lib/Wafer/Transforms/Linalg/SpatialRegionMaterialization.cpp:2420-2433).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def unit_range(units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous block [begin, end) of `units` independent work items owned by `rank`.
    The first `units % world_size` ranks own one extra unit."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank must lie in [0, world_size)")
    base, extra = divmod(units, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def sequence_range(kv_len: int, world_size: int, rank: int, granule: int = 64) -> Tuple[int, int]:
    """Contiguous KV interval of `rank`, boundaries rounded to `granule` keys (the decode kernel's
    per-CTA granule) so every shard but the last is a whole number of tiles."""
    per = -(-kv_len // world_size)
    per = -(-per // granule) * granule
    begin = min(rank * per, kv_len)
    return begin, min(begin + per, kv_len)


def sharded_decode(state_fn: Callable[[int, int], torch.Tensor], merge_fn: Callable[[torch.Tensor], torch.Tensor],
                   kv_len: int, group=None, gathered: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sequence-sharded flash-decoding step.

    state_fn(begin, end) -> this rank's [batch, q_heads, D + 2] float32 state for keys [begin, end)
                            (B200TargetModelBackend.attention_fd_partial on the GPU);
    merge_fn(states)     -> finalized output from [world, batch, q_heads, D + 2] states in shard order
                            (B200TargetModelBackend.attention_fd_merge).
    gathered             -> optional preallocated [world, batch, q_heads, D + 2] buffer, so that a decode loop
                            allocates nothing per step.
    The only exchange is one all-gather of the states (D + 2 floats per query head and rank).
    """
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    begin, end = sequence_range(kv_len, world, rank)
    state = state_fn(begin, end).contiguous()
    if world == 1:
        return merge_fn(state.unsqueeze(0))
    if gathered is None:
        gathered = torch.empty((world,) + tuple(state.shape), dtype=state.dtype, device=state.device)
    # rank r's state lands in gathered[r]: ascending KV order (the flat view keeps chunk shapes equal to the input's)
    dist.all_gather_into_tensor(gathered.view((world * state.shape[0],) + tuple(state.shape[1:])), state, group=group)
    return merge_fn(gathered)


class GraphedDecodeStep:
    """One sequence-sharded decode step (local state, all-gather, merge) captured once into a CUDA graph and replayed:
    a decode step is four small launches plus one collective, so at small per-rank KV lengths the launch path, not the
    HBM stream, sets its time. The callables must use preallocated tensors only (captured addresses are replayed); the
    library's own split-KV scratch is grow-only, so a later decode call with a larger batch x heads x splits reallocates it
    and invalidates this graph: build the step after the largest shape has run once.
    With more than one rank the graph holds an NCCL all-gather: release the step object (and synchronise) before the
    process group is destroyed - a process that tore the group down while the graph was alive did not exit.

        step = GraphedDecodeStep(state_fn, merge_fn, kv_len, gathered, group)
        step()          # replays; outputs are in the tensors merge_fn writes
    """

    def __init__(self, state_fn, merge_fn, kv_len: int, gathered: torch.Tensor, group=None, warmup: int = 2):
        self._graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):                      # first calls size the library's scratch buffers and NCCL's
                sharded_decode(state_fn, merge_fn, kv_len, group, gathered)
            side.synchronize()
            with torch.cuda.graph(self._graph, stream=side):
                sharded_decode(state_fn, merge_fn, kv_len, group, gathered)
        torch.cuda.current_stream().wait_stream(side)

    def __call__(self):
        self._graph.replay()


class PeerExchange:
    """Exchange buffers for the sequence-sharded decode whose state exchange runs inside the kernel
    (B200TargetModelBackend.attention_fd_exchange): one buffer per rank that every rank's GPU can address, plus this
    rank's epoch words. With one rank the buffer is ordinary device memory; with several it is torch symmetric memory
    (peer-mapped over NVLink), and the constructor is a collective call of the group.

        exchange = PeerExchange(backend, batch, q_heads, group)
        backend.attention_fd_exchange(q, k_shard, v_shard, scale, rank=exchange.rank, peer_pointers=exchange.pointers,
                                      epoch=exchange.epoch, out=out)

    The step involves no collective library call, so it may be captured into a CUDA graph. Release the object only after
    every rank has finished its last step (synchronise, then barrier)."""

    def __init__(self, backend, batch: int, q_heads: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        device = device or torch.device("cuda", backend.device)
        nbytes = backend.fd_exchange_bytes(batch, q_heads, self.world)
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        if self.world == 1:
            self.buffer = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            self.pointers = [self.buffer.data_ptr()]
            self._handle = None
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            self.buffer.zero_()
            self._handle = symm_mem.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
            self.pointers = [int(pointer) for pointer in self._handle.buffer_ptrs]
            torch.cuda.synchronize(device)
            dist.barrier(group)          # every rank's buffer is zeroed before anyone's first step


class SwitchSum:
    """Sums over the ranks done by the NVSwitch (B200TargetModelBackend.switch_sum): symmetric buffers bound to an NVLink
    multicast object, this rank's signal words and epoch. The constructor and `allocate` are collective calls of the
    group; `available` is False where the GPUs offer no multicast (then use a library all-reduce instead).

        sums = SwitchSum(backend, group)
        workspace = sums.allocate(nbytes)        # uint8 tensor; the same offsets mean the same data on every rank
        ...                                      # kernels write this rank's partial sums into a region of workspace
        sums(region)                             # in place, on the current stream: every rank now holds the sums

    One object serialises its sums (they share the signal words): give sums that may overlap in time objects of their own.
    Release the object only after every rank has finished its last sum (synchronise, then barrier)."""

    def __init__(self, backend, group=None, device: Optional[torch.device] = None, blocks: int = 0):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.backend, self.blocks = backend, blocks
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = device or torch.device("cuda", backend.device)
        self._buffers = []        # (tensor, handle, multicast pointer)
        self.epoch = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._signals = symm_mem.empty(backend.switch_sum_signal_bytes(self.world), dtype=torch.uint8, device=self.device)
        self._signals.zero_()
        self._signal_handle = symm_mem.rendezvous(self._signals, self.group)
        self.signal_pointers = [int(pointer) for pointer in self._signal_handle.buffer_ptrs]
        self.available = self.world > 1 and int(getattr(self._signal_handle, "multicast_ptr", 0) or 0) != 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)              # every rank's signal words are zero before anyone's first sum

    def allocate(self, nbytes: int) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm_mem
        buffer = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=self.device)
        handle = symm_mem.rendezvous(buffer, self.group)
        multicast = int(handle.multicast_ptr or 0)
        if multicast == 0:
            raise RuntimeError("this allocation has no NVLink multicast mapping")
        self._buffers.append((buffer, handle, multicast))
        return buffer

    def multicast_of(self, region: torch.Tensor) -> int:
        """The multicast address of a tensor that lies inside a buffer made by allocate()."""
        begin = region.data_ptr()
        for buffer, _handle, multicast in self._buffers:
            offset = begin - buffer.data_ptr()
            if 0 <= offset and offset + region.numel() * region.element_size() <= buffer.numel():
                return multicast + offset
        raise ValueError("the region does not lie in a buffer made by allocate()")

    def __call__(self, region: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """region <- sum over the ranks of region (+ residual, this rank's copy of a tensor that is the same on every rank);
        with `out` (inside a buffer made by allocate(), same extent) the result goes there and region keeps the partial sums."""
        if not region.is_contiguous() or (residual is not None and not residual.is_contiguous()) or (out is not None and not out.is_contiguous()):
            raise ValueError("the tensors must be contiguous")
        self.backend.switch_sum(self.multicast_of(region), region.numel(), region.dtype, rank=self.rank,
                                signal_pointers=self.signal_pointers, epoch=self.epoch, blocks=self.blocks,
                                multicast_out=self.multicast_of(out) if out is not None else 0, residual=residual)
        return region if out is None else out

