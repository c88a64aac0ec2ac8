"""Data-parallel gradient path.

``GradSync`` combines the gradients of the ranks once per optimizer step.  Two implementations:

* ``fused`` (CUDA, one process per GPU of one NVSwitch domain): the flat gradient arena lives in
  symmetric memory; :mod:`allie_b200.parallel.nvl` runs reduce-scatter, global-norm clip, sharded
  AdamW and the bf16/fp32 parameter all-gather as sm_100a kernels that read and write peer memory
  directly (``allie_b200/csrc/comm.cu``).
* ``collective``: one ``all_reduce`` of the flat arena through ``torch.distributed`` (NCCL on GPUs,
  gloo on CPU ranks) followed by the replicated optimizer - the plain baseline and the CPU path.

The reference gets the same effect from ``DistributedDataParallel`` bucketed all-reduces
(``src/modeling/trainer.py:232-233``) followed by a replicated fused AdamW.
"""
from __future__ import annotations

import logging

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)


def broadcast_parameters(model: torch.nn.Module, engine=None, src: int = 0) -> None:
    """Rank 0's initial weights to every rank (what the DDP constructor does)."""
    if engine is not None:
        a = engine.arena
        dist.broadcast(a.master[:a.sync_end], src)     # rank-local (expert) parameters are not replicated
        engine.arena.refresh_shadow()
    else:
        for p in model.parameters():
            dist.broadcast(p.data, src)


class GradSync:
    def __init__(self, model: torch.nn.Module, engine=None, mode: str = "auto"):
        self.model, self.engine = model, engine
        self.world = dist.get_world_size()
        self.fused = False
        self.nvl = None
        if engine is not None and mode in ("auto", "fused") and self.world > 1:
            try:
                from .nvl import NvlGradOptimizer

                self.nvl = NvlGradOptimizer(engine)
                self.fused = True
            except Exception as e:  # pragma: no cover - depends on the machine
                if mode == "fused":
                    raise
                logger.warning(f"fused NVLink gradient path unavailable ({e}); using all_reduce")

    def all_reduce_sum(self) -> None:
        a = self.engine.arena
        dist.all_reduce(a.grad[:a.sync_end], op=dist.ReduceOp.SUM)   # rank-local (expert) gradients stay put

    def all_reduce_mean_torch(self) -> None:
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        flat /= self.world
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    def fused_step(self, lr, betas, eps, weight_decay, grad_clip) -> None:
        self.nvl.step(lr, betas, eps, weight_decay, grad_clip)
