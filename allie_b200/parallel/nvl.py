"""Host side of the fused NVLink gradient path (kernels in ``csrc/comm.cu``).

The flat master / gradient / bf16-shadow arenas of the engine are allocated in PyTorch symmetric
memory, so every rank holds peer-mapped pointers (and, where the fabric offers it, a multicast
alias) to every other rank's arenas.  The replicated part of the arena is laid out in *buckets* in
the order in which backward finishes them, and every rank owns 1/N of each bucket
(:class:`ShardLayout`).  One optimizer step is then

    per bucket, on a side stream, as soon as backward has produced the bucket's last gradient:
        reduce-scatter of the bucket (+ its share of the sum of squares)
    after backward, on the compute stream:
        clip + sharded AdamW + parameter all-gather (one launch)  ->  wait for the peers' slices

with no NCCL call and no host synchronisation.  This is what ``DistributedDataParallel``'s bucketed
reducer hooks give the reference (``src/modeling/trainer.py:232-233``, fired from ``:280``), with
the optimizer sharded on top: Adam moments and the fp32 master of the weight-decayed parameters
live only on the rank that owns the slice; the other ranks receive the bf16 copy their GEMMs
read (and fp32 for the small non-decayed rest).  :meth:`NvlGradOptimizer.gather_state` brings
moments and masters back into the replicated layout for checkpoints.

The parameter all-gather always uses plain peer stores (measured faster than ``multimem.st`` on 2
and on 8 B200s); the gradient reduce-scatter uses plain peer loads up to 3 ranks and
``multimem.ld_reduce`` (the NVSwitch adds the eight copies) from 4 ranks up; ``ALLIE_NVL_MULTIMEM``
= ``0`` / ``rs`` / ``1`` forces plain / reduce-only / both.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import ptr, stream_ptr

MAX_BUCKETS = 32                       # csrc/comm.cu: MAX_BUCKETS
PHASE_DELIVERED = 2 * MAX_BUCKETS
FLAG_WORDS = (PHASE_DELIVERED + 1) * 32


def symmetric_empty(n: int, dtype: torch.dtype, device) -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem.empty(n, dtype=dtype, device=device)


def rendezvous(t: torch.Tensor):
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem.rendezvous(t, group=dist.group.WORLD)


def _ptr_array(ptrs) -> ctypes.Array:
    arr = (c_void_p * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = int(p)
    return arr


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """(offset, length) of the slice of a flat range of ``n`` elements that ``rank`` owns: equal
    contiguous slices rounded up to 64 elements (so every slice starts on a 256-byte boundary and
    the kernels' 16-byte vector accesses never straddle two owners); the last ranks may get a
    shorter or empty slice."""
    per = (n + world - 1) // world
    per = (per + 63) // 64 * 64
    off = min(n, per * rank)
    return off, max(0, min(n, per * (rank + 1)) - off)


class ShardLayout:
    """Who owns what: ``buckets`` is a list of ranges of the flat arena whose first and last
    entries are the bucket's start and end (the engine's ``(start, bf16_only_end, decay_end, end)``);
    rank r owns slice r of every bucket
    (:func:`shard_bounds` inside the bucket).  A rank's *shard* is its slices of all buckets back to
    back; that is the layout of its Adam moments.  Pure index arithmetic: usable on the CPU."""

    def __init__(self, buckets: list[tuple], world: int):
        assert 1 <= len(buckets) <= MAX_BUCKETS, f"{len(buckets)} gradient buckets (limit {MAX_BUCKETS})"
        self.buckets, self.world = [tuple(b) for b in buckets], world
        self.end = max((b[-1] for b in buckets), default=0)

    def slices(self, rank: int) -> list[tuple[int, int, int]]:
        """Per bucket: (offset in the arena, length, offset inside the rank's shard)."""
        out, m = [], 0
        for bk in self.buckets:
            start, end = bk[0], bk[-1]
            off, n = shard_bounds(end - start, self.world, rank)
            out.append((start + off, n, m))
            m += n
        return out

    def shard_numel(self, rank: int) -> int:
        return sum(n for _o, n, _m in self.slices(rank))

    def extract(self, full: torch.Tensor, rank: int) -> torch.Tensor:
        """``rank``'s shard cut out of a flat tensor in arena layout."""
        parts = [full[o:o + n] for o, n, _m in self.slices(rank)]
        return torch.cat(parts) if parts else full[:0]

    def place(self, shard: torch.Tensor, rank: int, full: torch.Tensor) -> None:
        """Writes ``rank``'s shard back into its places in a flat tensor in arena layout."""
        for o, n, m in self.slices(rank):
            full[o:o + n].copy_(shard[m:m + n])

    def assemble(self, shards: list[torch.Tensor], out: torch.Tensor | None = None) -> torch.Tensor:
        """The flat range [0, end) from all ranks' shards (the inverse of :meth:`extract`)."""
        if out is None:
            out = torch.zeros(self.end, dtype=shards[0].dtype, device=shards[0].device)
        for r, s in enumerate(shards):
            self.place(s, r, out)
        return out

    def all_gather(self, shard: torch.Tensor, rank: int, full: torch.Tensor, group=None) -> None:
        """Collective: every rank passes its shard; ``full`` ends up complete on every rank.  One
        padded ``all_gather`` per bucket (every slice of a bucket has the same padded length)."""
        for bk, (o, n, m) in zip(self.buckets, self.slices(rank)):
            start, end = bk[0], bk[-1]
            per = shard_bounds(end - start, self.world, 0)[1]
            if per == 0:
                continue
            mine = torch.zeros(per, dtype=shard.dtype, device=shard.device)
            mine[:n].copy_(shard[m:m + n])
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=group)
            full[start:end].copy_(torch.cat(parts)[: end - start])


    def gather(self, shard: torch.Tensor, rank: int, full: torch.Tensor | None, dst: int = 0, group=None) -> None:
        """Collective: like :meth:`all_gather`, but only rank ``dst`` receives (``full`` may be None
        elsewhere), so only that rank needs room for the whole range."""
        for bk, (o, n, m) in zip(self.buckets, self.slices(rank)):
            start, end = bk[0], bk[-1]
            per = shard_bounds(end - start, self.world, 0)[1]
            if per == 0:
                continue
            mine = torch.zeros(per, dtype=shard.dtype, device=shard.device)
            mine[:n].copy_(shard[m:m + n])
            parts = [torch.empty_like(mine) for _ in range(self.world)] if rank == dst else None
            dist.gather(mine, parts, dst=dst, group=group)
            if rank == dst:
                full[start:end].copy_(torch.cat(parts)[: end - start])


class NvlGradOptimizer:
    def __init__(self, engine):
        a = engine.arena
        if not getattr(a, "symmetric", False):
            raise RuntimeError("engine arenas are not in symmetric memory")
        self.engine = engine
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        assert self.world <= 8
        dev = engine.device
        self.h_grad = rendezvous(a.grad)
        self.h_master = rendezvous(a.master)
        self.h_shadow = rendezvous(a.shadow)
        self.flags = symmetric_empty(FLAG_WORDS, torch.int32, dev)
        self.flags.zero_()
        self.norm_part = symmetric_empty(8, torch.float32, dev)
        self.norm_part.zero_()
        self.h_flags = rendezvous(self.flags)
        self.h_norm = rendezvous(self.norm_part)
        self.ticket = torch.zeros(4, dtype=torch.int32, device=dev)
        # ALLIE_NVL_MULTIMEM: 0 = plain peer loads / stores; 1 = multimem.ld_reduce for the gradients
        # and multimem.st for the parameters; rs = multimem.ld_reduce for the gradients only.
        # Unset: rs from 4 ranks up (the reduce-scatter then issues one load per 16 bytes instead of
        # one per peer and leaves the SMs it shares with backward sooner: 84.2 against 85.2 ms per
        # step at 8 GPUs), plain below, and plain whenever NCCL_NVLS_ENABLE=0 asks for no multicast.
        mode = os.environ.get("ALLIE_NVL_MULTIMEM")
        if mode is None:
            mode = "rs" if self.world >= 4 and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0" else "0"
        mc = [int(getattr(h, "multicast_ptr", 0) or 0) for h in (self.h_grad, self.h_master, self.h_shadow)]
        self.multimem = mode == "1" and all(mc)
        self.mc_grad, self.mc_master, self.mc_shadow = mc if self.multimem else (0, 0, 0)
        if mode == "rs" and mc[0]:
            self.mc_grad = mc[0]
        # only the replicated region [0, sync_end) is reduced and sharded; rank-local (expert)
        # parameters behind it are updated in place by every rank for itself
        self.layout = ShardLayout(a.buckets, self.world)
        self.slices = self.layout.slices(self.rank)
        self.nb = len(self.slices)
        self.shard_n = self.layout.shard_numel(self.rank)
        self.total_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.has_local = a.total > a.sync_end
        self.exp_avg = torch.zeros(max(self.shard_n, 4), dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(max(self.shard_n, 4), dtype=torch.float32, device=dev)
        self.epoch = 0
        self._reduced = self.nb          # buckets of the current epoch already handed to the reduce kernel
        self._applied_epoch = 0          # epoch whose reduced gradients the optimizer has consumed
        self.side = torch.cuda.Stream(device=dev)
        self._ready = [torch.cuda.Event() for _ in range(self.nb)]
        self._all_reduced = torch.cuda.Event()
        ll = c_longlong * MAX_BUCKETS
        pad = [0] * (MAX_BUCKETS - self.nb)
        self._s_off = ll(*[o for o, _n, _m in self.slices], *pad)
        self._s_n = ll(*[n for _o, n, _m in self.slices], *pad)
        self._m_off = ll(*[m for _o, _n, m in self.slices], *pad)
        self._hend = ll(*[b[1] for b in a.buckets], *pad)
        self._dend = ll(*[b[2] for b in a.buckets], *pad)
        self._p_grad = _ptr_array(self.h_grad.buffer_ptrs)
        self._p_master = _ptr_array(self.h_master.buffer_ptrs)
        self._p_shadow = _ptr_array(self.h_shadow.buffer_ptrs)
        self._p_flags = _ptr_array(self.h_flags.buffer_ptrs)
        self._p_norm = _ptr_array(self.h_norm.buffer_ptrs)
        self.masters_complete = True     # False once a step left non-owned fp32 masters behind
        torch.cuda.synchronize()
        dist.barrier()

    # ---- the step -----------------------------------------------------------------------
    def _launch_reduce(self, b: int, grid: int) -> None:
        off, n, _m = self.slices[b]
        rc = _lib.cuda().ab_nvl_reduce_scatter(
            self._p_grad, self._p_flags, c_void_p(self.mc_grad), ptr(self.norm_part), ptr(self.ticket),
            c_longlong(off), c_longlong(n), c_int(self.rank), c_int(self.world), c_uint(self.epoch),
            c_int(b), c_int(int(b == 0)), c_int(grid), ptr(_lib.status_word()), stream_ptr())
        if rc:
            raise RuntimeError(f"ab_nvl_reduce_scatter failed: {rc}")
        _lib.count_launches(2)          # the bucket's one-warp sync kernel and the reduce-scatter itself

    def bucket_ready(self, b: int) -> None:
        """Backward hook: every gradient of bucket ``b`` has been enqueued on the current stream.
        Buckets arrive in order 0 .. nb-1 during the LAST micro-step of an optimizer step; the
        bucket's reduce-scatter goes to the side stream behind an event, so it runs under the rest
        of backward."""
        if b == 0:
            self.epoch += 1
            self._reduced = 0
        assert b == self._reduced, f"bucket {b} reported ready after {self._reduced} buckets"
        self._ready[b].record()
        last = b == self.nb - 1
        with torch.cuda.stream(self.side):
            self.side.wait_event(self._ready[b])
            if last and self.has_local:
                # this rank's expert gradients join the global norm through its published partial sum
                from ..ops import kernels as K

                a = self.engine.arena
                K.sumsq(a.grad[a.sync_end:], self.norm_part[self.epoch & 1: (self.epoch & 1) + 1])
            # one 128-thread block per SM sits beside the backward GEMMs; the last bucket has the GPU to itself
            self._launch_reduce(b, 148 * 4 if last else 148)
            if last:
                self._all_reduced.record()
        self._reduced = b + 1

    def step(self, lr, betas, eps, weight_decay, grad_clip) -> None:
        """Clip + sharded AdamW + parameter all-gather.  Buckets that no backward hook reported
        are reduced here first (a step driven without hooks is correct, only not overlapped)."""
        eng, a = self.engine, self.engine.arena
        lib = _lib.cuda()
        if self._applied_epoch == self.epoch:
            first = 0                       # no hook started this step's reductions
        else:
            first = self._reduced           # hooks covered buckets [0, _reduced)
        for b in range(first, self.nb):
            self.bucket_ready(b)
        torch.cuda.current_stream().wait_event(self._all_reduced)
        self._applied_epoch = self.epoch
        eng.step_count += 1
        st = _lib.status_word()
        rc = lib.ab_nvl_adamw_allgather(
            self._p_master, self._p_shadow, self._p_flags, self._p_norm, c_void_p(self.mc_master),
            c_void_p(self.mc_shadow), ptr(a.grad), ptr(self.exp_avg), ptr(self.exp_avg_sq),
            c_void_p(self.ticket.data_ptr() + 4), c_int(self.nb), self._s_off, self._s_n, self._hend,
            self._dend, self._m_off, c_int(self.rank), c_int(self.world), c_uint(self.epoch),
            c_float(lr), c_float(betas[0]), c_float(betas[1]), c_float(eps), c_float(weight_decay),
            c_int(eng.step_count), c_float(grad_clip), c_float(1.0 / self.world), ptr(self.total_norm), ptr(st),
            stream_ptr())
        if rc:
            raise RuntimeError(f"ab_nvl_adamw_allgather failed: {rc}")
        rc = lib.ab_nvl_wait(ptr(self.flags), c_int(PHASE_DELIVERED), c_int(self.world), c_uint(self.epoch),
                             ptr(st), stream_ptr())
        if rc:
            raise RuntimeError(f"ab_nvl_wait failed: {rc}")
        _lib.count_launches(2)
        self.masters_complete = False
        if self.has_local:
            from ..ops import kernels as K

            a.ensure_state()
            for start, end, decays in a.local_regions:
                if end > start:
                    K.adamw(a.master[start:end], a.grad[start:end], a.exp_avg[start:end], a.exp_avg_sq[start:end],
                            a.shadow[start:end], lr, betas[0], betas[1], eps, weight_decay if decays else 0.0,
                            eng.step_count, self.total_norm if grad_clip > 0 else None, grad_clip, 1.0 / self.world)

    # ---- optimizer state in the replicated (checkpoint) layout ---------------------------
    def gather_state(self, exp_avg: torch.Tensor | None, exp_avg_sq: torch.Tensor | None, dst: int = 0) -> None:
        """Collective, for checkpoints.  Completes the fp32 master arena on every rank (its
        weight-decayed part is only kept current by each slice's owner between checkpoints) and
        writes all ranks' moment shards into rank ``dst``'s flat arenas ``exp_avg`` /
        ``exp_avg_sq`` (arena layout; other ranks may pass None)."""
        self.gather_master()
        self.layout.gather(self.exp_avg, self.rank, exp_avg, dst)
        self.layout.gather(self.exp_avg_sq, self.rank, exp_avg_sq, dst)

    def gather_master(self) -> None:
        """Collective.  Makes the fp32 master arena complete on every rank."""
        if self.masters_complete:
            return
        a = self.engine.arena
        mine = self.layout.extract(a.master, self.rank)
        self.layout.all_gather(mine, self.rank, a.master)
        self.masters_complete = True

    def scatter_state(self, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor) -> None:
        self.exp_avg[: self.shard_n].copy_(self.layout.extract(exp_avg, self.rank))
        self.exp_avg_sq[: self.shard_n].copy_(self.layout.extract(exp_avg_sq, self.rank))
