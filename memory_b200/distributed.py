"""Data-parallel gradient reduction for the memory layer: batch sharded, bank replicated.

The reference trains with DDP, which all-reduces the dense 262,208 x 768 fp32 bank gradient every
step because ``torch.gather``'s backward materialises it (memory_bank.py:291).  Here only the chapters
some rank touched travel:

1. every rank marks its touched chapters in a ``[C]`` count vector; all-reduce(SUM);
2. all ranks derive the same ascending union list ``U`` from it;
3. each rank scatters its compact ``[U_local*T, d]`` rows into a zeroed ``[|U|*T, d]`` buffer;
4. one all-reduce of that buffer (fp32, or bf16 on request), divided by the world size like DDP;
5. the result is handed back as a ``SparseBankGrad`` keyed by ``U``.

Dense parameter gradients (projections, router) are flattened into one bucket and all-reduced.

The pipelined form (``snapshot`` + ``reduce_snapshot_async``, what a training loop that replays a captured
step uses) exchanges the same rows without any host synchronisation and without building the union: every
rank's compact ``(chapter ids, count, rows / world)`` triple has a fixed size, so three all-gathers deliver
all ranks' triples and the result is a ``SparseBankGrad`` with one entry per rank whose scatter-add is the
mean gradient.  It moves (world-1) x local rows per rank instead of 2 x union rows and needs no
compaction pass before or division pass after the collective.

With ``exchange="peer"`` (CUDA, one node) the three all-gathers are replaced by device-to-device copies into
receive buffers that every rank holds in symmetric memory: each rank pushes its block to every peer with the copy
engines over NVLink, bracketed by two one-element all-reduces that order the pushes against the readers.  No SM
runs for the bulk transfer, so the compute of the next step keeps the whole GPU.

Works on any ``torch.distributed`` backend (NCCL on GPUs; gloo in the CPU tests of the bookkeeping).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def union_of_touched(counts: torch.Tensor) -> torch.Tensor:
    """Ascending chapter ids with a non-zero count."""
    return torch.nonzero(counts > 0, as_tuple=False).flatten()


def compact_to_union(local_ids: torch.Tensor, local_rows: torch.Tensor, union_ids: torch.Tensor,
                     num_chapters: int, tokens_per_chapter: int) -> torch.Tensor:
    """Place ``local_rows`` ([n_local*T, d], chapter-major, for ``local_ids``) at their positions in the
    union ordering; untouched positions are zero."""
    t = tokens_per_chapter
    d = local_rows.shape[-1]
    pos = torch.full((num_chapters,), -1, dtype=torch.long, device=union_ids.device)
    pos[union_ids] = torch.arange(union_ids.numel(), device=union_ids.device)
    out = torch.zeros(union_ids.numel(), t, d, dtype=local_rows.dtype, device=local_rows.device)
    if local_ids.numel():
        out.index_copy_(0, pos[local_ids.long()], local_rows.view(-1, t, d)[: local_ids.numel()])
    return out.view(-1, d)


# Priority of the exchange streams (the compute graph of a data-parallel step is captured on a high-priority stream).
# Measured at eight GPUs: exchanges at the compute stream's priority, alternating between two streams, with a third
# set of step buffers, made the step longer (1.71 ms against 1.56) -- two exchanges in flight share the same links and
# each takes twice as long -- so the exchange keeps one default-priority stream.
_EXCHANGE_PRIORITY = 0


class _PeerPush:
    """Fixed-size all-gather of one (ids, count, rows) triple by peer-to-peer copies.

    Every rank owns ``parities`` receive buffers ``[world, ...]`` in symmetric memory.  ``exchange`` (on the
    current stream): wait until the local consumer released this parity, one-element all-reduce (every rank is
    past its consumer), copy the local block into slot ``rank`` of every rank's buffer (``cudaMemcpyAsync``
    device-to-device: copy engines, no kernel), one-element all-reduce (every push has landed everywhere).
    """

    def __init__(self, group, device, n_ids: int, rows_shape, parities: int = 2,
                 rows_dtype: torch.dtype = torch.float32, n_dense: int = 0):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n, self.m, self.d = int(n_ids), int(rows_shape[0]), int(rows_shape[1])
        self.parities = parities
        self.rows_dtype = rows_dtype
        w = self.world
        per_word = 4 // torch.empty(0, dtype=rows_dtype).element_size()      # row elements per fp32 word
        if (self.m * self.d) % per_word:
            raise ValueError("row block must fill whole 32-bit words")
        self.rows_words = w * self.m * self.d // per_word
        self.ids_words = -(-(w * self.n) // 4) * 4
        self.num_words = -(-w // 4) * 4
        # optional slots for a dense bucket of n_dense fp32 values per rank, and one flag word per rank for the
        # flag barrier (behind the parities)
        self.n_dense = int(n_dense)
        self.dense_ld = -(-self.n_dense // 4) * 4
        self.dense_words = w * self.dense_ld
        self.per_parity = self.rows_words + self.ids_words + self.num_words + self.dense_words
        total = parities * self.per_parity + 16
        self.buf = symm.empty(total, dtype=torch.float32, device=device)
        self.buf[parities * self.per_parity:].zero_()       # the flag words start at epoch 0
        torch.cuda.synchronize(device)
        handle = symm.rendezvous(self.buf, self.group)
        self.peers = [handle.get_buffer(r, (total,), torch.float32) for r in range(w)]
        self.flags = [p_[parities * self.per_parity:].view(torch.int32) for p_ in self.peers]
        self.epoch = 0
        self.handle = handle
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.consumed = [None] * parities
        # one stream per peer: the pushes to different peers run on different copy engines / links at once
        self.push_streams = [torch.cuda.Stream(device, priority=_EXCHANGE_PRIORITY) for _ in range(w - 1)]

    def _views(self, flat: torch.Tensor, parity: int):
        base = parity * self.per_parity
        rows = flat[base:base + self.rows_words].view(self.rows_dtype).view(self.world, self.m, self.d)
        ids = flat[base + self.rows_words:base + self.rows_words + self.world * self.n].view(torch.int32)
        nums = flat[base + self.rows_words + self.ids_words:
                    base + self.rows_words + self.ids_words + self.world].view(torch.int32)
        return rows, ids.view(self.world, self.n), nums

    def _dense(self, flat: torch.Tensor, parity: int) -> torch.Tensor:
        """[world, dense_ld] fp32: the ranks' dense buckets of this parity."""
        base = parity * self.per_parity + self.rows_words + self.ids_words + self.num_words
        return flat[base:base + self.dense_words].view(self.world, self.dense_ld)

    def barrier(self) -> None:
        """Flag barrier on the current stream (see ``ops.peer_barrier``): every rank's earlier work on this stream,
        its pushes included, is complete and visible once it returns."""
        from . import ops
        self.epoch += 1
        ops.peer_barrier(self.flags, self.rank, self.epoch)

    def exchange(self, parity: int, uniq: torch.Tensor, num_unique: torch.Tensor, rows: torch.Tensor,
                 handshake: bool = True, dense: Optional[torch.Tensor] = None):
        """``handshake=False`` leaves both one-element all-reduces out.  That is safe when (a) the only reader of
        a receive buffer is work queued on this same stream right after the exchange that filled it (the
        union-sum), and (b) the caller issues one collective of its own after this call and treats its completion
        as "every push has landed" (every rank enters it after its pushes, in stream order).  Then a rank can only
        push into parity p again after all ranks entered the collective of the exchange in between, which they
        do after their reader of parity p."""
        stream = torch.cuda.current_stream(self.buf.device)
        if self.consumed[parity] is not None:
            stream.wait_event(self.consumed[parity])
        if handshake:
            dist.all_reduce(self.token, group=self.group)
        start = torch.cuda.Event()
        start.record(stream)
        for k in range(1, self.world):          # the local block is used where it is: no copy to self
            r = (self.rank + k) % self.world
            p_rows, p_ids, p_nums = self._views(self.peers[r], parity)
            side = self.push_streams[k - 1]
            side.wait_event(start)
            with torch.cuda.stream(side):
                p_rows[self.rank].copy_(rows.view(self.m, self.d), non_blocking=True)
                p_ids[self.rank].copy_(uniq.view(torch.int32), non_blocking=True)
                p_nums[self.rank:self.rank + 1].copy_(num_unique.view(torch.int32).reshape(1), non_blocking=True)
                if dense is not None:           # the dense bucket travels the same way, into this rank's slot
                    self._dense(self.peers[r], parity)[self.rank, :self.n_dense].copy_(dense, non_blocking=True)
        if dense is not None:
            self._dense(self.buf, parity)[self.rank, :self.n_dense].copy_(dense, non_blocking=True)
        for side in self.push_streams:          # what follows on the calling stream is behind every push
            stream.wait_stream(side)
        work = dist.all_reduce(self.token, group=self.group, async_op=True) if handshake else None
        rows_all, ids_all, nums_all = self._views(self.buf, parity)
        # the local list also goes into its own slot (a few KB), so that [world, n] is one table for the merge;
        # the local rows stay where they are
        ids_all[self.rank].copy_(uniq.view(torch.int32), non_blocking=True)
        nums_all[self.rank:self.rank + 1].copy_(num_unique.view(torch.int32).reshape(1), non_blocking=True)
        return work, [(uniq, num_unique, rows) if r == self.rank else (ids_all[r], nums_all[r:r + 1], rows_all[r])
                      for r in range(self.world)], (ids_all, nums_all)

    def release(self, parity: int) -> None:
        """The consumer of this parity's buffers is done (recorded on the current stream)."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.buf.device))
        self.consumed[parity] = ev


class GradReducer:
    """Reduces one step's gradients across the data-parallel group (mean, as DDP does)."""

    def __init__(self, num_chapters: int, tokens_per_chapter: int, dim: int, device,
                 group: Optional[dist.ProcessGroup] = None, bank_dtype: torch.dtype = torch.float32,
                 exchange: str = "nccl", wire_dtype: torch.dtype = torch.float32, merge: bool = False,
                 record_timings: bool = False, merge_dtype: torch.dtype = torch.float32, sync: str = "collective",
                 parities: int = 2):
        """``wire_dtype`` bf16: the pipelined exchange sends the bf16 copy of the rows that the backward pass
        wrote next to the fp32 ones (the sink must be created with ``SparseBankGrad(torch.bfloat16)``); sums are
        still formed in fp32 at the receiver.  The reference's DDP reduces fp32; bf16 halves the volume at a
        rounding of 2^-9 relative per rank's contribution.  ``merge``: the exchange is followed, on the reducer's
        stream, by the union-sum kernel, so ``PendingReduction.result()`` holds ONE entry: the mean gradient rows
        over the union of all ranks' chapters (identical bits on every rank).  ``merge_dtype`` bf16 stores those
        mean rows in bf16 (sums still in fp32): half the bytes the union-sum writes, one more rounding of 2^-9.
        ``sync`` (peer exchange with ``merge``): "collective" -- the dense bucket is all-reduced by NCCL and that
        collective doubles as the exchange's synchronisation; "flags" -- the dense bucket is pushed like the rows,
        summed locally (rank order, identical bits everywhere), and a flag barrier over peer memory synchronises:
        no NCCL kernel holds SMs beside the compute of the next step."""
        if sync not in ("collective", "flags"):
            raise ValueError("sync must be 'collective' or 'flags'")
        self.sync = sync
        # receive-buffer sets of the peer exchange (and of the union-sum's output): a result stays valid until
        # `parities` exchanges later, so a caller that keeps k results in flight needs k + 1 ... at least 2
        self.parities = max(2, int(parities))
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        if wire_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("wire_dtype must be float32 or bfloat16")
        self.exchange = exchange
        self.wire_dtype = wire_dtype
        self.merge = merge
        if merge_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("merge_dtype must be float32 or bfloat16")
        self.merge_dtype = merge_dtype
        self.record_timings = record_timings
        self.timings = []          # (start, exchanged, merged) CUDA events on the reducer's stream, per exchange
        self._merge_out = {}       # per parity: output buffers of the union-sum kernel
        self._peer = None
        self._parity = 0
        self.c, self.t, self.d = int(num_chapters), int(tokens_per_chapter), int(dim)
        self.device = torch.device(device)
        self.group = group
        self.bank_dtype = bank_dtype
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.last_union_size = 0

    def reduce_dense(self, grads: Sequence[Optional[torch.Tensor]]) -> None:
        live = [g for g in grads if g is not None]
        if not live or self.world == 1:
            return
        flat = torch.cat([g.reshape(-1).float() for g in live])
        dist.all_reduce(flat, group=self.group)
        flat.div_(self.world)
        off = 0
        for g in live:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n

    def reduce_bank(self, sink):
        """``sink`` is a SparseBankGrad holding this rank's entries (left untouched, so entries captured in
        a CUDA graph stay valid).  Returns a new SparseBankGrad with one entry: the union chapter list
        and the mean gradient rows."""
        counts = torch.zeros(self.c, dtype=torch.int32, device=self.device)
        merged_ids, merged_rows = self._merge_local(sink)
        if merged_ids.numel():
            counts[merged_ids.long()] = 1
        if self.world > 1:
            dist.all_reduce(counts, group=self.group)
        union = union_of_touched(counts)
        self.last_union_size = int(union.numel())
        buf = compact_to_union(merged_ids, merged_rows, union, self.c, self.t).to(self.bank_dtype)
        if self.world > 1:
            dist.all_reduce(buf, group=self.group)
            buf.div_(self.world)
        out = type(sink)()
        out.add(union.to(torch.int32), torch.tensor([union.numel()], dtype=torch.int32, device=self.device),
                buf.float(), self.t)
        return out

    def reduce_async(self, dense_grads: Sequence[Optional[torch.Tensor]], sink) -> "PendingReduction":
        """Start the reduction without blocking later work on the calling stream.

        Gradients are first copied into fresh staging buffers (on the calling stream), so the caller may
        overwrite its gradient tensors -- e.g. by replaying a captured step -- while the all-reduces run on
        the communication stream.  The one host synchronisation is the read of the union size.
        """
        live = [g for g in dense_grads if g is not None]
        works = []
        flat = torch.cat([g.reshape(-1).float() for g in live]) if live else None
        if flat is not None and self.world > 1:
            works.append(dist.all_reduce(flat, group=self.group, async_op=True))
        bank = None
        if sink is not None:       # entered by every rank, whatever its own sink holds: the collectives must match
            counts = torch.zeros(self.c, dtype=torch.int32, device=self.device)
            ids, rows = self._merge_local(sink)
            if ids.numel():
                counts[ids.long()] = 1
            if self.world > 1:
                dist.all_reduce(counts, group=self.group)
            union = union_of_touched(counts)
            self.last_union_size = int(union.numel())
            buf = compact_to_union(ids, rows, union, self.c, self.t).to(self.bank_dtype)
            if self.world > 1:
                works.append(dist.all_reduce(buf, group=self.group, async_op=True))
            bank = (union, buf)
        return PendingReduction(self, works, flat, [g.shape for g in live], bank, type(sink) if sink is not None else None)

    # ---- pipelined form: snapshot on the compute stream, reduce on a side stream one step later ----------
    def snapshot(self, dense_grads: Sequence[Optional[torch.Tensor]], sink, copy: bool = True) -> "GradSnapshot":
        """Stage this step's gradients on the current stream (no host synchronisation).

        ``copy=True``: gradients are copied, already divided by the world size, so the caller may overwrite its
        gradient tensors right afterwards (e.g. by replaying the same captured step).
        ``copy=False``: nothing is copied; the snapshot references the caller's tensors, which must stay
        untouched until the reduction's ``wait()`` (e.g. two captured steps used alternately); the dense bucket
        is assembled on the reducer's stream and the bank rows travel unscaled, the result's ``scale`` says what
        the consumer still has to apply."""
        inv = 1.0 / self.world
        live = [g for g in dense_grads if g is not None]
        entries = []
        if copy:
            flat = torch.cat([g.reshape(-1).float() for g in live]) if live else None
            if flat is not None and self.world > 1:
                flat.mul_(inv)
            if sink is not None:
                for uniq, num_unique, rows, t in sink.entries:
                    staged = rows.float() * inv if self.world > 1 else rows.float().clone()
                    entries.append((uniq.clone(), num_unique.clone(), staged.to(self.wire_dtype), t))
        else:
            flat = None
            if sink is not None:
                for i, (u, n, r, t) in enumerate(sink.entries):
                    if self.wire_dtype == torch.bfloat16:
                        wire = sink.wire[i] if i < len(sink.wire) else None
                        if wire is None:
                            raise ValueError("bf16 exchange needs SparseBankGrad(wire_dtype=torch.bfloat16)")
                        entries.append((u, n, wire, t))
                    else:
                        entries.append((u, n, r if r.dtype == torch.float32 else r.float(), t))
        ev = torch.cuda.Event() if self.device.type == "cuda" else None
        if ev is not None:
            ev.record(torch.cuda.current_stream(self.device))
        snap = GradSnapshot(flat, [g.shape for g in live], entries, ev, type(sink) if sink is not None else None)
        if not copy:
            snap.dense_refs = live
            snap.bank_scale = inv if self.world > 1 else 1.0
        return snap

    def _all_gather(self, out: torch.Tensor, inp: torch.Tensor):
        """``out`` = the ranks' ``inp`` back to back; returns the async work handle."""
        try:
            return dist.all_gather_into_tensor(out, inp.contiguous(), group=self.group, async_op=True)
        except (RuntimeError, NotImplementedError):
            return dist.all_gather(list(out.chunk(self.world)), inp.contiguous(), group=self.group, async_op=True)

    def _gather_snapshot(self, snap: "GradSnapshot") -> "PendingReduction":
        works = []
        if snap.flat is None and snap.dense_refs:
            snap.flat = torch.cat([g.reshape(-1).float() for g in snap.dense_refs])
            if self.world > 1:
                snap.flat.mul_(1.0 / self.world)
        gathered = []
        merge_inputs = None
        use_peer = (self.exchange == "peer" and self.world > 1 and self.device.type == "cuda"
                    and len(snap.entries) == 1)
        # With the union-sum as the only reader of the receive buffers, the dense bucket's all-reduce, issued
        # after the pushes, is the one collective of the exchange (see _PeerPush.exchange).
        light = use_peer and self.merge and snap.flat is not None
        if snap.flat is not None and self.world > 1 and not light:
            works.append(dist.all_reduce(snap.flat, group=self.group, async_op=True))
        for uniq, num_unique, rows, t in snap.entries:
            if self.world == 1:
                gathered.append((uniq, num_unique, rows, t))
                continue
            if use_peer and self._peer is None:
                use_peer = self._open_peer(uniq.numel(), rows.shape, rows.dtype,
                                           snap.flat.numel() if snap.flat is not None else 0)
                if not use_peer and light:        # fell back to NCCL: the dense bucket travels on its own after all
                    light = False
                    works.append(dist.all_reduce(snap.flat, group=self.group, async_op=True))
            if use_peer:
                parity = self._parity
                self._parity = (parity + 1) % self._peer.parities
                flags = light and self.sync == "flags" and self._peer.n_dense == snap.flat.numel()
                work, triples, (ids_tab, num_tab) = self._peer.exchange(parity, uniq, num_unique, rows,
                                                                         handshake=not light,
                                                                         dense=snap.flat if flags else None)
                if work is not None:
                    works.append(work)
                elif flags:
                    # as below: this rank's reader of the previous exchange's buffers is over before it tells its
                    # peers (by arriving at the barrier) that they may overwrite them
                    if getattr(self, "_merge_done", None) is not None:
                        torch.cuda.current_stream(self.device).wait_event(self._merge_done)
                    self._peer.barrier()
                    from . import ops
                    dense_all = self._peer._dense(self._peer.buf, parity)
                    snap.flat = ops.sum_terms(dense_all.view(1, -1), snap.flat.numel(), self.world).view(-1)
                else:
                    # the reader of the previous exchange's receive buffers (the union-sum, on its own stream) must
                    # be over before this rank enters the collective that licenses its peers to overwrite them
                    if getattr(self, "_merge_done", None) is not None:
                        torch.cuda.current_stream(self.device).wait_event(self._merge_done)
                    works.append(dist.all_reduce(snap.flat, group=self.group, async_op=True))
                gathered += [(i, c, r, t) for i, c, r in triples]
                merge_inputs = ([r for _, _, r in triples], ids_tab, num_tab, t)
                pending_parity = parity
                continue
            n, m = uniq.numel(), rows.shape[0]
            ids_all = torch.empty(self.world * n, dtype=uniq.dtype, device=uniq.device)
            num_all = torch.empty(self.world, dtype=num_unique.dtype, device=uniq.device)
            rows_all = torch.empty(self.world * m, rows.shape[1], dtype=rows.dtype, device=rows.device)
            works += [self._all_gather(ids_all, uniq), self._all_gather(num_all, num_unique.reshape(1)),
                      self._all_gather(rows_all, rows)]
            for r in range(self.world):
                gathered.append((ids_all[r * n:(r + 1) * n], num_all[r:r + 1], rows_all[r * m:(r + 1) * m], t))
            if len(snap.entries) == 1:
                merge_inputs = ([rows_all[r * m:(r + 1) * m] for r in range(self.world)],
                                ids_all.view(self.world, n), num_all, t)
        pending = PendingReduction(self, works, snap.flat, snap.shapes, None, snap.sink_type, gathered=gathered)
        pending.bank_scale = snap.bank_scale
        pending.merge_inputs = merge_inputs
        if use_peer and self.world > 1 and snap.entries:
            pending.parity = pending_parity
        return pending

    def _open_peer(self, n_ids: int, rows_shape, rows_dtype=torch.float32, n_dense: int = 0) -> bool:
        """Create the symmetric-memory receive buffers; every rank must succeed or all fall back to NCCL."""
        ok = 1
        try:
            self._peer = _PeerPush(self.group, self.device, n_ids, rows_shape, parities=self.parities,
                                   rows_dtype=rows_dtype, n_dense=n_dense if self.sync == "flags" else 0)
        except Exception:                      # symmetric memory unavailable in this process / on this node
            self._peer, ok = None, 0
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self._peer = None
            self.exchange = "nccl"
            return False
        return True

    def prepare(self, sink, dense_grads: Optional[Sequence[Optional[torch.Tensor]]] = None) -> None:
        """Set up everything the pipelined exchange allocates or maps lazily -- the reducer's stream and, for
        ``exchange="peer"``, the symmetric-memory receive buffers and their peer mappings -- while the device is
        idle.  Mapping peer memory updates the GPU's page tables; done under running kernels it stalled their
        memory traffic long enough for a bounded device wait to give up.  Call once, on every rank, after the
        first backward pass has filled ``sink`` (its entry gives the block sizes) and before the timed loop.
        ``dense_grads`` (needed for ``sync="flags"``): the dense gradients of a step, for the size of their bucket."""
        if self.device.type != "cuda" or self.world == 1:
            return
        torch.cuda.synchronize(self.device)
        if getattr(self, "_streams", None) is None:
            self._streams = [torch.cuda.Stream(self.device, priority=_EXCHANGE_PRIORITY) for _ in range(2)]
        if self.merge and getattr(self, "_merge_stream", None) is None:
            self._merge_stream = torch.cuda.Stream(self.device)
        if self.exchange == "peer" and self._peer is None and sink is not None and len(sink.entries) == 1:
            uniq, _, rows, _ = sink.entries[0]
            if self.wire_dtype == torch.bfloat16 and sink.wire and sink.wire[0] is not None:
                rows = sink.wire[0]
            n_dense = sum(g.numel() for g in dense_grads if g is not None) if dense_grads is not None else 0
            self._open_peer(uniq.numel(), rows.shape, rows.dtype, n_dense)
        dist.barrier(group=self.group)
        torch.cuda.synchronize(self.device)

    def reduce_snapshot_async(self, snap: "GradSnapshot") -> "PendingReduction":
        """Exchange a snapshot on the reducer's own stream: one all-reduce of the dense bucket and three
        all-gathers per bank entry, all of fixed size, so nothing here waits for the device."""
        if self.device.type != "cuda":
            return self._gather_snapshot(snap)
        if getattr(self, "_streams", None) is None:
            self._streams = [torch.cuda.Stream(self.device, priority=_EXCHANGE_PRIORITY) for _ in range(2)]
        self._stream = self._streams[0]      # one exchange at a time (see _EXCHANGE_PRIORITY)
        with torch.cuda.stream(self._stream):
            self._stream.wait_event(snap.event)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if self.record_timings else None
            if ev:
                ev[0].record(self._stream)
            pending = self._gather_snapshot(snap)
            pending.stream = self._stream
            # completion of exactly this exchange (later exchanges queued on the same stream do not count)
            for w in pending.works:
                w.wait()
            pending.works = []
            if ev:
                ev[1].record(self._stream)
            if self.merge and pending.merge_inputs is not None:
                # The union-sum runs on a stream of its own, so the pushes of the next exchange (other parity) go
                # out beside it; that exchange's collective waits for it (see _gather_snapshot): every rank still
                # enters the collective after its reader of the parity before, which is what lets a peer overwrite
                # that parity afterwards.
                if getattr(self, "_merge_stream", None) is None:
                    self._merge_stream = torch.cuda.Stream(self.device)
                self._merge_stream.wait_stream(self._stream)
                with torch.cuda.stream(self._merge_stream):
                    self._merge(pending)
                    if ev:
                        ev[2].record(self._merge_stream)
                    self._merge_done = torch.cuda.Event()
                    self._merge_done.record(self._merge_stream)
                    pending.done = self._merge_done
                pending.stream = self._merge_stream
                if ev:
                    self.timings.append(tuple(ev))
            else:
                if ev:
                    ev[2].record(self._stream)
                    self.timings.append(tuple(ev))
                pending.done = torch.cuda.Event()
                pending.done.record(self._stream)
        return pending

    def _merge(self, pending: "PendingReduction") -> None:
        """Union-sum of the gathered rows on the current (reducer) stream.  The output buffers belong to the
        receive-buffer parity (or rotate over two sets), so a result stays valid until the exchange after next."""
        from . import ops
        rank_rows, ids_tab, num_tab, t = pending.merge_inputs
        if self.device.type == "cuda":      # allocated on the exchange stream, read on this one
            cur = torch.cuda.current_stream(self.device)
            for x in (*rank_rows, ids_tab, num_tab):
                x.record_stream(cur)
        slot = pending.parity if pending.parity is not None else (len(self.timings) & 1)
        out = ops.bank_grad_merge(rank_rows, ids_tab, num_tab, t, self.c, pending.bank_scale,
                                  out=self._merge_out.get(slot), out_dtype=self.merge_dtype)
        self._merge_out[slot] = out
        pending.merged = (out["uniq"], out["num_unique"], out["rows"], t)

    @staticmethod
    def _split(flat, shapes):
        out, off = [], 0
        if flat is None:
            return out
        for shp in shapes:
            n = 1
            for v in shp:
                n *= int(v)
            out.append(flat[off:off + n].view(shp))
            off += n
        return out

    def reduce(self, dense_grads: Sequence[Optional[torch.Tensor]], sink):
        """All-reduce the dense gradients in place and return the reduced bank gradient (or None)."""
        self.reduce_dense(dense_grads)
        if sink is not None:       # entered by every rank, whatever its own sink holds: the collectives must match
            return self.reduce_bank(sink)
        return None

    def _merge_local(self, sink):
        """Sum this rank's entries (several memory layers may share one bank) into one id list."""
        if len(sink.entries) == 0:
            return (torch.empty(0, dtype=torch.int32, device=self.device),
                    torch.empty(0, self.d, dtype=torch.float32, device=self.device))
        if len(sink.entries) == 1:
            uniq, num_unique, rows, _ = sink.entries[0]
            n = int(num_unique.item())
            return uniq[:n], rows[: n * self.t]
        dense_ids: List[torch.Tensor] = []
        for uniq, num_unique, rows, _ in sink.entries:
            n = int(num_unique.item())
            dense_ids.append(uniq[:n].long())
        ids = torch.unique(torch.cat(dense_ids)) if dense_ids else torch.empty(0, dtype=torch.long, device=self.device)
        pos = torch.full((self.c,), -1, dtype=torch.long, device=self.device)
        pos[ids] = torch.arange(ids.numel(), device=self.device)
        out = torch.zeros(ids.numel(), self.t, self.d, dtype=torch.float32, device=self.device)
        for uniq, num_unique, rows, _ in sink.entries:
            n = int(num_unique.item())
            out.index_add_(0, pos[uniq[:n].long()], rows[: n * self.t].view(n, self.t, self.d))
        return ids.to(torch.int32), out.view(-1, self.d)


class GradSnapshot:
    """Staged copy of one step's gradients (see :meth:`GradReducer.snapshot`)."""

    dense_refs = None     # zero-copy form: the caller's dense gradient tensors
    bank_scale = 1.0      # factor still to be applied to the bank rows by the consumer

    def __init__(self, flat, shapes, entries, event, sink_type):
        self.flat, self.shapes, self.entries, self.event, self.sink_type = flat, shapes, entries, event, sink_type


class PendingReduction:
    """Handle of a reduction started by :meth:`GradReducer.reduce_async`."""
    stream = None
    done = None

    def __init__(self, reducer, works, flat, shapes, bank, sink_type, gathered=None):
        self.reducer, self.works, self.flat, self.shapes, self.bank, self.sink_type = \
            reducer, works, flat, shapes, bank, sink_type
        self.gathered = gathered      # per-rank (ids, count, rows / world, T) of the pipelined form
        self.parity = None            # receive-buffer parity of the peer exchange, if that carried the rows
        self.bank_scale = 1.0
        self.merge_inputs = None      # (per-rank rows, [world, n] id table, [world] counts, T) for the union-sum
        self.merged = None            # (union ids, count, summed fp32 rows, T) once the union-sum has run

    def release(self) -> None:
        """Tell the reducer that the result's tensors are no longer read after the work queued so far on the
        current stream.  Needed with ``exchange="peer"``, whose receive buffers are reused every second step."""
        if self.parity is not None and self.reducer._peer is not None:
            self.reducer._peer.release(self.parity)

    def wait(self) -> None:
        """Make the current stream wait for the collectives (no host block)."""
        if self.done is not None:
            torch.cuda.current_stream(self.stream.device).wait_event(self.done)
        elif self.stream is not None:
            with torch.cuda.stream(self.stream):
                for w in self.works:
                    w.wait()
            torch.cuda.current_stream(self.stream.device).wait_stream(self.stream)
        else:
            for w in self.works:
                w.wait()
        self.works = []

    def result(self):
        """(list of mean dense gradients in the order given, reduced SparseBankGrad or None)."""
        self.wait()
        r = self.reducer
        if self.gathered is not None:
            bank = None
            if self.sink_type is not None:
                bank = self.sink_type()
                if self.merged is not None:
                    bank.add(*self.merged)        # one entry: the mean rows over the union (scale applied)
                else:
                    for e in self.gathered:
                        bank.add(*e)
                    bank.scale = self.bank_scale
            return GradReducer._split(self.flat, self.shapes), bank
        dense = []
        if self.flat is not None:
            flat = self.flat / r.world
            off = 0
            for shp in self.shapes:
                n = int(torch.tensor(shp).prod()) if len(shp) else 1
                dense.append(flat[off:off + n].view(shp))
                off += n
        bank = None
        if self.bank is not None:
            union, buf = self.bank
            bank = self.sink_type()
            bank.add(union.to(torch.int32), torch.tensor([union.numel()], dtype=torch.int32, device=r.device),
                     buf.float() / r.world, r.t)
        return dense, bank
