"""Host side of the fused NVLink gradient path (kernels in ``csrc/comm.cu``).

The flat master / gradient / bf16-shadow arenas of the engine are allocated in PyTorch symmetric
memory, so every rank holds peer-mapped pointers (and, where the fabric offers it, a multicast
alias) to every other rank's arenas.  One optimizer step is then three launches on the compute
stream, with no NCCL call and no host synchronisation:

    reduce-scatter (+ sum of squares)  ->  clip + sharded AdamW + parameter all-gather  ->  wait

Rank r owns the r-th contiguous 1/N slice of the flat arenas; Adam moments exist only for that
slice (optimizer state sharded N ways).  The kernels move data with plain peer loads / stores by
default: measured on 2 and on 8 B200s that was faster than the ``multimem.ld_reduce`` /
``multimem.st`` variant (84.3 against 87.5 ms per medium step at 8 GPUs, 7.9 against 11.9 ms for the
phase at 2), so the multicast variant is opt-in with ``ALLIE_NVL_MULTIMEM=1``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import ptr, stream_ptr

FLAG_WORDS = 3 * 32


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
    """(offset, length) of the slice of a flat arena of ``n`` elements that ``rank`` owns: equal
    contiguous slices rounded up to 64 elements (so every shard starts on a 256-byte boundary and
    the kernels' 16-byte vector accesses never straddle two owners); the last ranks may get a
    shorter or empty slice."""
    per = (n + world - 1) // world
    per = (per + 63) // 64 * 64
    off = min(n, per * rank)
    return off, max(0, min(n, per * (rank + 1)) - off)


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
        use_mc = os.environ.get("ALLIE_NVL_MULTIMEM", "0") == "1"
        mc = [int(getattr(h, "multicast_ptr", 0) or 0) for h in (self.h_grad, self.h_master, self.h_shadow)]
        self.multimem = use_mc and all(mc)
        self.mc_grad, self.mc_master, self.mc_shadow = mc if self.multimem else (0, 0, 0)
        # only the replicated region [0, sync_end) is reduced and sharded; rank-local (expert)
        # parameters behind it are updated in place by every rank for itself
        self.shard_off, self.shard_n = shard_bounds(a.sync_end, self.world, self.rank)
        self.total_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.has_local = a.total > a.sync_end
        self.exp_avg = torch.zeros(max(self.shard_n, 4), dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(max(self.shard_n, 4), dtype=torch.float32, device=dev)
        self.epoch = 0
        self._p_grad = _ptr_array(self.h_grad.buffer_ptrs)
        self._p_master = _ptr_array(self.h_master.buffer_ptrs)
        self._p_shadow = _ptr_array(self.h_shadow.buffer_ptrs)
        self._p_flags = _ptr_array(self.h_flags.buffer_ptrs)
        self._p_norm = _ptr_array(self.h_norm.buffer_ptrs)
        torch.cuda.synchronize()
        dist.barrier()

    def step(self, lr, betas, eps, weight_decay, grad_clip) -> None:
        eng, a = self.engine, self.engine.arena
        lib = _lib.cuda()
        self.epoch += 1
        eng.step_count += 1
        st = _lib.status_word()
        if self.has_local:
            # this rank's expert gradients join the global norm through its published partial sum
            from ..ops import kernels as K

            K.sumsq(a.grad[a.sync_end:], self.norm_part[self.epoch & 1: (self.epoch & 1) + 1])
        rc = lib.ab_nvl_reduce_scatter(self._p_grad, self._p_flags, c_void_p(self.mc_grad),
                                       ptr(self.norm_part), ptr(self.ticket), c_longlong(self.shard_off),
                                       c_longlong(self.shard_n), c_int(self.rank), c_int(self.world),
                                       c_uint(self.epoch), ptr(st), stream_ptr())
        if rc:
            raise RuntimeError(f"ab_nvl_reduce_scatter failed: {rc}")
        rc = lib.ab_nvl_adamw_allgather(
            self._p_master, self._p_shadow, self._p_flags, self._p_norm, c_void_p(self.mc_master),
            c_void_p(self.mc_shadow), ptr(a.grad), ptr(self.exp_avg), ptr(self.exp_avg_sq),
            c_void_p(self.ticket.data_ptr() + 4), c_longlong(self.shard_off), c_longlong(self.shard_n),
            c_longlong(a.decay_end), c_int(self.rank), c_int(self.world), c_uint(self.epoch),
            c_float(lr), c_float(betas[0]), c_float(betas[1]), c_float(eps), c_float(weight_decay),
            c_int(eng.step_count), c_float(grad_clip), c_float(1.0 / self.world), ptr(self.total_norm), ptr(st),
            stream_ptr())
        if rc:
            raise RuntimeError(f"ab_nvl_adamw_allgather failed: {rc}")
        rc = lib.ab_nvl_wait(ptr(self.flags), c_int(2), c_int(self.world), c_uint(self.epoch), ptr(st),
                             stream_ptr())
        if rc:
            raise RuntimeError(f"ab_nvl_wait failed: {rc}")
        _lib.count_launches(3)
        if self.has_local:
            from ..ops import kernels as K

            a.ensure_state()
            for start, end, decays in a.regions[2:]:
                if end > start:
                    K.adamw(a.master[start:end], a.grad[start:end], a.exp_avg[start:end], a.exp_avg_sq[start:end],
                            a.shadow[start:end], lr, betas[0], betas[1], eps, weight_decay if decays else 0.0,
                            eng.step_count, self.total_norm if grad_clip > 0 else None, grad_clip, 1.0 / self.world)

    # ---- optimizer state in the replicated (checkpoint) layout ---------------------------
    def gather_state(self) -> tuple[torch.Tensor, torch.Tensor]:
        """All ranks' moment shards concatenated to full flat arenas (for checkpoints)."""
        a = self.engine.arena
        sizes = [torch.zeros(1, dtype=torch.int64, device=self.exp_avg.device) for _ in range(self.world)]
        dist.all_gather(sizes, torch.tensor([self.shard_n], dtype=torch.int64, device=self.exp_avg.device))
        mx = int(max(int(s) for s in sizes))
        outs = []
        for src in (self.exp_avg, self.exp_avg_sq):
            pad = torch.zeros(mx, dtype=torch.float32, device=src.device)
            pad[: self.shard_n] = src[: self.shard_n]
            parts = [torch.empty_like(pad) for _ in range(self.world)]
            dist.all_gather(parts, pad)
            outs.append(torch.cat([p[: int(s)] for p, s in zip(parts, sizes)])[: a.total])
        return outs[0], outs[1]

    def scatter_state(self, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor) -> None:
        self.exp_avg[: self.shard_n].copy_(exp_avg[self.shard_off:self.shard_off + self.shard_n])
        self.exp_avg_sq[: self.shard_n].copy_(exp_avg_sq[self.shard_off:self.shard_off + self.shard_n])
