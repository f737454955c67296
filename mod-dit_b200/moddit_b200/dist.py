"""Ulysses-style re-sharding around the head-parallel hot path: sequence shards in, head shards inside.

Every stage of the path is independent per attention head, so P ranks each take H/P heads.  A caller
that holds sequence shards (1, H, N/P, D) exchanges them for head shards (1, H/P, N, D) with one
all-to-all per tensor before the path and one for the output after it.  The reference only has dead
hooks for this exchange (MoD/models/cogvideox/attention_processor.py:138-155, 220-229).

The functions take any initialised `torch.distributed` process group (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def shard_bounds(total: int, world: int, rank: int):
    """[begin, end) of `rank`'s equal share; `total` must divide evenly."""
    if total % world:
        raise ValueError(f"{total} does not divide evenly over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


def pool_partition(seq_len: int, block_size: int, world: int, rank: int):
    """Which pooled blocks a sequence shard produces: (first block, end block, halo rows, tail rows).

    A block belongs to the rank that holds its last row.  `halo rows` is how many rows of the rank's first
    block lie in the previous rank's shard; `tail rows` is how many of its own last rows belong to a block
    that the next rank finishes (they are that rank's halo)."""
    if seq_len % world:
        raise ValueError(f"{seq_len} rows do not divide evenly over {world} ranks")
    ns = seq_len // world
    if ns < block_size:
        raise ValueError("a sequence shard must hold at least one block")
    nb = (seq_len + block_size - 1) // block_size
    first = (rank * ns) // block_size
    end = nb if rank == world - 1 else ((rank + 1) * ns) // block_size
    halo = rank * ns - first * block_size
    tail = 0 if rank == world - 1 else (rank + 1) * ns - end * block_size
    return first, end, halo, tail


def _exchange(world: int, rank: int, send_view, recv_view, local_copy, group):
    """One grouped exchange: `send_view(peer)` / `recv_view(peer)` give lists of contiguous tensors."""
    ops = []
    for peer in range(world):
        if peer == rank:
            continue
        gpeer = dist.get_global_rank(group, peer) if group is not None else peer
        for t in recv_view(peer):
            ops.append(dist.P2POp(dist.irecv, t, gpeer, group=group))
        for t in send_view(peer):
            ops.append(dist.P2POp(dist.isend, t, gpeer, group=group))
    reqs = dist.batch_isend_irecv(ops) if ops else []
    local_copy()
    for r in reqs:
        r.wait()


# Measured on 8 B200s (89 MB per tensor per GPU): one all_to_all_single plus a repacking copy takes 0.29 ms,
# the grouped per-piece send/recv 0.60 ms; on 2 GPUs (355 MB) it is 0.97 ms against 0.79 ms.
_PIECEWISE_MAX_WORLD = 2


def _seq_to_head_a2a(x: torch.Tensor, world: int, group) -> torch.Tensor:
    _, H, ns, D = x.shape
    hp = H // world
    send = x.reshape(world, hp, ns, D)                         # chunk p = heads of rank p (a view)
    recv = torch.empty_like(send)                              # chunk r = my heads, sequence shard of rank r
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3).reshape(1, hp, world * ns, D).contiguous()


def _head_to_seq_a2a(x: torch.Tensor, world: int, group) -> torch.Tensor:
    _, hp, N, D = x.shape
    ns = N // world
    send = x.reshape(hp, world, ns, D).permute(1, 0, 2, 3).contiguous()   # chunk p = sequence shard of rank p
    recv = torch.empty_like(send)                                        # chunk r = heads of rank r
    dist.all_to_all_single(recv, send, group=group)
    return recv.reshape(1, world * hp, ns, D)


def seq_to_head(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """(1, H, N/P, D) sequence shard -> (1, H/P, N, D) head shard (heads [rank*H/P, (rank+1)*H/P)).

    Up to 2 ranks every (head, sequence shard) piece, contiguous on both sides, travels straight into its
    final place in one grouped send/recv; with more ranks one all-to-all plus a repacking copy is faster.
    """
    world = dist.get_world_size(group)
    if world == 1:
        return x
    rank = dist.get_rank(group)
    if x.shape[1] % world:
        raise ValueError(f"{x.shape[1]} heads do not divide over {world} ranks")
    if world > _PIECEWISE_MAX_WORLD:
        return _seq_to_head_a2a(x.contiguous(), world, group)
    _, H, ns, D = x.shape
    if H % world:
        raise ValueError(f"{H} heads do not divide over {world} ranks")
    if not x.is_contiguous():
        x = x.contiguous()
    hp = H // world
    out = torch.empty(1, hp, world * ns, D, device=x.device, dtype=x.dtype)
    _exchange(
        world, rank,
        send_view=lambda peer: [x[0, peer * hp + h] for h in range(hp)],                   # hp pieces of (ns, D)
        recv_view=lambda peer: [out[0, h, peer * ns:(peer + 1) * ns] for h in range(hp)],  # hp pieces of (ns, D)
        local_copy=lambda: out[0, :, rank * ns:(rank + 1) * ns].copy_(x[0, rank * hp:(rank + 1) * hp]),
        group=group)
    return out


def head_to_seq(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """(1, H/P, N, D) head shard -> (1, H, N/P, D) sequence shard."""
    world = dist.get_world_size(group)
    if world == 1:
        return x
    rank = dist.get_rank(group)
    _, hp, N, D = x.shape
    if N % world:
        raise ValueError(f"sequence length {N} does not divide over {world} ranks")
    if world > _PIECEWISE_MAX_WORLD:
        return _head_to_seq_a2a(x.contiguous(), world, group)
    if not x.is_contiguous():
        x = x.contiguous()
    ns = N // world
    out = torch.empty(1, world * hp, ns, D, device=x.device, dtype=x.dtype)
    _exchange(
        world, rank,
        send_view=lambda peer: [x[0, h, peer * ns:(peer + 1) * ns] for h in range(hp)],
        recv_view=lambda peer: [out[0, peer * hp + h] for h in range(hp)],
        local_copy=lambda: out[0, rank * hp:(rank + 1) * hp].copy_(x[0, :, rank * ns:(rank + 1) * ns]),
        group=group)
    return out


def group_pieces(world: int, rank: int, heads_per_rank: int, groups: int, row_bytes: int, head_bytes: int,
                 x_ptrs, peer_bases):
    """The strided copies of a sequence->head exchange delivered in `groups` runs of the local heads.

    x_ptrs[t]: address of this rank's (H, N/P, D) shard of tensor t; peer_bases[t][p]: address of rank p's
    (H/P, N, D) buffer for tensor t; row_bytes = one (head, sequence shard) piece, head_bytes = one head in an
    owner's buffer.  Returns a list with one (src addresses, dst addresses, rows) triple per run: every piece is
    `rows` rows of row_bytes, source pitch row_bytes, destination pitch head_bytes.  Peers are visited starting
    with the rank itself, so that the ranks do not all write to the same owner at once."""
    groups = max(1, min(int(groups), heads_per_rank))
    hpg = (heads_per_rank + groups - 1) // groups
    out = []
    for g in range(groups):
        h0, h1 = g * hpg, min(heads_per_rank, (g + 1) * hpg)
        if h0 >= h1:
            break
        src, dst = [], []
        for step in range(world):
            peer = (rank + step) % world
            for t, x in enumerate(x_ptrs):
                src.append(x + (peer * heads_per_rank + h0) * row_bytes)
                dst.append(peer_bases[t][peer] + h0 * head_bytes + rank * row_bytes)
        out.append((src, dst, h1 - h0))
    return out


class PeerResharder:
    """Sequence<->head re-shard through peer-mapped (symmetric) buffers on one NVLink/NVSwitch node.

    Every rank owns a head-shard staging buffer per input tensor and a sequence-shard staging buffer for
    the output.  A re-shard is a set of strided row copies issued by this library's own copy kernel: each
    rank stores its pieces straight into their final position in the owner's buffer (P2P stores), so there
    is no repacking pass and no intermediate buffer; a device-side barrier of the symmetric-memory handle
    separates writers from readers.  Buffers are reused every call: the barrier at the start of a call
    guarantees that all ranks have finished reading the previous contents.
    """

    COPY_STREAMS = 4      # side streams the copy-engine pieces of one exchange are spread over
    NARROW_CTAS = 48      # CTAs of one exchange in 'narrow' mode

    def __init__(self, heads: int, seq_len: int, head_dim: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, n_inputs: int = 3, timeout_ms: int = 20000,
                 bulk_copy: str = "dma"):
        import torch.distributed._symmetric_memory as symm_mem
        from . import ops
        self._ops = ops
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if heads % self.world or seq_len % self.world:
            raise ValueError("heads and sequence length must divide over the ranks")
        self.H, self.N, self.D = heads, seq_len, head_dim
        self.hp, self.ns = heads // self.world, seq_len // self.world
        self.dtype, self.device = dtype, device
        self.esize = torch.empty((), dtype=dtype).element_size()
        self.timeout_ms = timeout_ms
        if bulk_copy not in ("dma", "kernel", "narrow"):
            raise ValueError("bulk_copy must be 'dma' (copy engines), 'kernel' (this library's copy kernel on the "
                             "whole GPU) or 'narrow' (the copy kernel on NARROW_CTAS CTAs)")
        self.bulk_copy = bulk_copy
        self._copy_streams = None
        self.inputs, self.in_handles = [], []
        for _ in range(n_inputs):
            t = symm_mem.empty((1, self.hp, self.N, self.D), dtype=dtype, device=device)
            self.inputs.append(t)
            self.in_handles.append(symm_mem.rendezvous(t, self.group))
        self.output = symm_mem.empty((1, self.H, self.ns, self.D), dtype=dtype, device=device)
        self.out_handle = symm_mem.rendezvous(self.output, self.group)

    # `quiesced=True` on the calls below skips the barrier that opens them ("every rank has finished with the
    # previous contents").  It is for a caller whose previous use of these buffers was followed, on every rank and
    # on the stream this call is ordered behind, by one of this class's closing barriers - e.g. the step before
    # ended with `finish_output` or `head_to_seq`: a rank passes that barrier only when all ranks have reached it,
    # i.e. have finished every kernel that read the buffers.

    def seq_to_head(self, x: torch.Tensor, slot: int, channel: int = 0, quiesced: bool = False) -> torch.Tensor:
        """Push this rank's (1, H, N/P, D) shard into slot `slot` of every owner; returns the local head shard
        (1, H/P, N, D), valid on the current stream once the call returns."""
        return self.seq_to_head_many([x], [slot], channel, quiesced)[0]

    def seq_to_head_many(self, xs, slots, channel: int = 0, quiesced: bool = False):
        """Several tensors between one pair of barriers (slot i receives xs[i])."""
        for x in xs:
            if tuple(x.shape) != (1, self.H, self.ns, self.D) or x.dtype != self.dtype or not x.is_contiguous():
                raise ValueError("inputs must be contiguous (1, H, N/P, D) tensors of the configured dtype")
        sync = self.in_handles[slots[0]]
        if not quiesced:
            sync.barrier(channel=channel, timeout_ms=self.timeout_ms)  # readers of the previous contents are done
        row = self.ns * self.D * self.esize                            # bytes of one (head, sequence shard) piece
        src, dst = [], []
        for step in range(self.world):
            peer = (self.rank + step) % self.world                     # start with the local piece, spread the rest
            for x, slot in zip(xs, slots):
                src.append(x.data_ptr() + peer * self.hp * row)
                dst.append(int(self.in_handles[slot].buffer_ptrs[peer]) + self.rank * row)
        self._bulk(src, dst, row, self.N * self.D * self.esize, row, self.hp)
        sync.barrier(channel=channel, timeout_ms=self.timeout_ms)     # every rank's stores have landed
        return [self.inputs[slot] for slot in slots]

    def seq_to_head_groups(self, xs, slots, groups: int, channel: int = 0, quiesced: bool = False):
        """`seq_to_head_many` delivered group of heads by group of heads: the local heads are cut into `groups` runs of
        ceil(H/P / groups) heads; run g of every tensor is sent to every owner, then a barrier, then event g is
        recorded on the current stream - a consumer that works head by head starts on run 0 while the later runs
        are still on the links.  Returns (tensors, events)."""
        for x in xs:
            if tuple(x.shape) != (1, self.H, self.ns, self.D) or x.dtype != self.dtype or not x.is_contiguous():
                raise ValueError("inputs must be contiguous (1, H, N/P, D) tensors of the configured dtype")
        sync = self.in_handles[slots[0]]
        cur = torch.cuda.current_stream(self.device)
        if not quiesced:
            sync.barrier(channel=channel, timeout_ms=self.timeout_ms)  # readers of the previous contents are done
        row = self.ns * self.D * self.esize                            # bytes of one (head, sequence shard) piece
        head = self.N * self.D * self.esize                            # bytes of one head in an owner's buffer
        bases = [[int(p) for p in self.in_handles[slot].buffer_ptrs] for slot in slots]
        events = []
        for src, dst, rows in group_pieces(self.world, self.rank, self.hp, groups, row, head,
                                           [x.data_ptr() for x in xs], bases):
            self._bulk(src, dst, row, head, row, rows)
            sync.barrier(channel=channel, timeout_ms=self.timeout_ms)  # every rank's rows of this run have landed
            ev = torch.cuda.Event()
            ev.record(cur)
            events.append(ev)
        return [self.inputs[slot] for slot in slots], events

    def head_to_seq(self, x: torch.Tensor, channel: int = 0) -> torch.Tensor:
        """Push this rank's (1, H/P, N, D) head shard back; returns the local (1, H, N/P, D) sequence shard."""
        if tuple(x.shape) != (1, self.hp, self.N, self.D) or x.dtype != self.dtype or not x.is_contiguous():
            raise ValueError("input must be a contiguous (1, H/P, N, D) tensor of the configured dtype")
        hdl = self.out_handle
        hdl.barrier(channel=channel, timeout_ms=self.timeout_ms)
        row = self.ns * self.D * self.esize
        src, dst = [], []
        for step in range(self.world):
            peer = (self.rank + step) % self.world
            src.append(x.data_ptr() + peer * row)
            dst.append(int(hdl.buffer_ptrs[peer]) + self.rank * self.hp * row)
        self._bulk(src, dst, self.N * self.D * self.esize, row, row, self.hp)
        hdl.barrier(channel=channel, timeout_ms=self.timeout_ms)
        return self.output

    def _bulk(self, src, dst, src_pitch: int, dst_pitch: int, width: int, rows: int) -> None:
        """The (peer, tensor) pieces of one exchange: asynchronous 2-D copies on the copy engines (the SMs stay
        with the kernels of the step, a peer gets the whole link), or this library's copy kernel, one launch
        per 24 pieces."""
        if self.bulk_copy == "dma":
            # The pieces go to different peers over different links: issued on one stream they would run one after
            # another (each a short 2-D copy that cannot fill a link by itself), so they are spread over a few side
            # streams that fork from the current stream and join it again - several copy engines and links at once.
            cur = torch.cuda.current_stream(self.device)
            if self._copy_streams is None:
                self._copy_streams = [torch.cuda.Stream(device=self.device) for _ in range(self.COPY_STREAMS)]
            lanes = self._copy_streams[:max(1, min(len(self._copy_streams), len(src)))]
            fork = torch.cuda.Event()
            fork.record(cur)
            for st in lanes:
                st.wait_event(fork)
            for i, (s_, d_) in enumerate(zip(src, dst)):
                with torch.cuda.stream(lanes[i % len(lanes)]):
                    self._ops.copy_rows_dma(s_, d_, src_pitch, dst_pitch, width, rows, self.device)
            for st in lanes:
                done = torch.cuda.Event()
                done.record(st)
                cur.wait_event(done)
            return
        for i in range(0, len(src), 24):
            if self.bulk_copy == "narrow":
                self._ops.copy_rows_narrow(src[i:i + 24], dst[i:i + 24], src_pitch, dst_pitch, width, rows, self.device,
                                           max_ctas=self.NARROW_CTAS)
            else:
                self._ops.copy_rows_multi(src[i:i + 24], dst[i:i + 24], src_pitch, dst_pitch, width, rows, self.device)

    # ---- block means of query and key, pooled on the sequence shards ----------------------------------------
    def enable_pooling(self, block_size: int) -> None:
        """Allocates the halo and pooled-mean buffers for `pool_to_head` (collective: every rank calls it)."""
        import torch.distributed._symmetric_memory as symm_mem
        self.pool_bs = block_size
        self.pool_nb = (self.N + block_size - 1) // block_size
        self.pool_part = pool_partition(self.N, block_size, self.world, self.rank)
        self.halo = symm_mem.empty((2, self.H, block_size, self.D), dtype=self.dtype, device=self.device)
        self.halo_handle = symm_mem.rendezvous(self.halo, self.group)
        self.pooled = symm_mem.empty((2, 1, self.hp, self.pool_nb, self.D), dtype=torch.float32, device=self.device)
        self.pooled_handle = symm_mem.rendezvous(self.pooled, self.group)

    def pool_to_head(self, q: torch.Tensor, k: torch.Tensor, channel: int = 0, quiesced: bool = False):
        """Block means of this rank's (1, H, N/P, D) query and key shards, delivered to the head owners.

        Returns this rank's (1, H/P, nb, D) float32 means of query and key - equal, bit for bit, to pooling
        the gathered heads - without waiting for the bulk sequence->head exchange of query and key: only
        the rows of a block cut by a shard boundary (fewer than block_size per head) and the means
        themselves cross the links."""
        for x in (q, k):
            if tuple(x.shape) != (1, self.H, self.ns, self.D) or x.dtype != self.dtype or not x.is_contiguous():
                raise ValueError("inputs must be contiguous (1, H, N/P, D) tensors of the configured dtype")
        first, end, halo_rows, tail_rows = self.pool_part
        bs = self.pool_bs
        row = self.D * self.esize
        if not quiesced:
            self.halo_handle.barrier(channel=channel, timeout_ms=self.timeout_ms)   # last call's readers are done
        if tail_rows:
            nxt = self.rank + 1
            base = int(self.halo_handle.buffer_ptrs[nxt])
            src = [x.data_ptr() + (self.ns - tail_rows) * row for x in (q, k)]
            dst = [base + t * self.H * bs * row for t in range(2)]
            self._ops.copy_rows_multi(src, dst, self.ns * row, bs * row, tail_rows * row, self.H, self.device)
        self.halo_handle.barrier(channel=channel, timeout_ms=self.timeout_ms)   # halos have landed
        plane = self.hp * self.pool_nb * self.D * 4
        for t, x in enumerate((q, k)):
            peers = [int(p) + t * plane for p in self.pooled_handle.buffer_ptrs]
            halo_ptr = self.halo.data_ptr() + t * self.H * bs * row
            self._ops.pool_blocks_shard(x, halo_ptr, halo_rows, bs, bs, end - first, peers, self.hp, self.pool_nb,
                                        first)
        self.pooled_handle.barrier(channel=channel, timeout_ms=self.timeout_ms)  # every rank's means have landed
        return self.pooled[0], self.pooled[1]

    # ---- output re-shard fused into the attention kernel's epilogue ------------------------------------
    def begin_output(self, channel: int = 0, consumed: bool = False):
        """Call before a kernel that stores its output rows straight into the peers' buffers; returns the
        `scatter` argument for `ops.sparse_attn_fwd` (peer buffer pointers, first global head of this rank).
        consumed=True skips the barrier: for a caller that, on every rank, read the previous output on this stream
        and has since passed another of this class's barriers on it (`pool_to_head` ends with one)."""
        if not consumed:
            self.out_handle.barrier(channel=channel, timeout_ms=self.timeout_ms)   # previous output has been consumed
        return [int(p) for p in self.out_handle.buffer_ptrs], self.rank * self.hp

    def finish_output(self, channel: int = 0) -> torch.Tensor:
        """Call after that kernel: once every rank's stores have landed the local (1, H, N/P, D) shard is valid."""
        self.out_handle.barrier(channel=channel, timeout_ms=self.timeout_ms)
        return self.output
