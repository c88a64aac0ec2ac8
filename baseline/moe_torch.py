"""Plain-PyTorch expert-parallel MoE training step: the comparison arm for the MoE configuration
(the reference project has no MoE, so there is no reference implementation to run).

Stack: the oracle module tree in bf16 autocast, SDPA attention, the MoE feed-forward replaced by a
sort + ``all_to_all_single`` dispatch, one ``torch._grouped_mm`` per projection over all local
experts (a loop of cuBLAS GEMMs where that operator is missing, or with
``ALLIE_BASELINE_MOE_LOOP=1``), and an ``all_to_all_single`` combine; dense gradients all-reduced
with NCCL; torch fused AdamW.  No code of ``allie_b200``'s kernels or engine runs on this path.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from allie_b200.models.oracle import Attention, MoEMLP, gelu_new


GROUPED = hasattr(torch, "_grouped_mm") and os.environ.get("ALLIE_BASELINE_MOE_LOOP", "0") != "1"


class _A2A(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits):
        ctx.splits = (out_splits, in_splits)
        out = x.new_empty((sum(out_splits),) + x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits)
        return out

    @staticmethod
    def backward(ctx, g):
        out_splits, in_splits = ctx.splits
        gx = g.new_empty((sum(in_splits),) + g.shape[1:])
        dist.all_to_all_single(gx, g.contiguous(), in_splits, out_splits)
        return gx, None, None


def ep_moe_forward(self: MoEMLP, x):
    """Drop-in ``MoEMLP.forward`` for R ranks with E/R local experts each (weights pre-sliced)."""
    R = dist.get_world_size() if dist.is_initialized() else 1
    B, T, d = x.shape
    x2 = x.reshape(-1, d)
    gates, topi, self.aux_loss = self.route(x2)
    E = self.router.out_features
    El = E // R
    flat_e = topi.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // self.top_k
    xs = x2[tok]
    counts = torch.bincount(flat_e, minlength=E)
    if R > 1:
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts)              # [R, El] counts arriving here
        in_splits = counts.view(R, El).sum(1).tolist()
        out_splits = recv_counts.view(R, El).sum(1).tolist()
        xr = _A2A.apply(xs, out_splits, in_splits)
        rc = recv_counts.view(R, El)
        # received rows are grouped by source rank, then by local expert: regroup by expert
        idx = torch.arange(xr.size(0), device=x.device)
        seg_expert = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(R), rc.reshape(-1))
        perm = torch.argsort(seg_expert, stable=True)
        xr = xr[perm]
        per_expert = rc.sum(0).tolist()
    else:
        xr, per_expert, perm = xs, counts.tolist(), None
    if GROUPED and xr.is_cuda and xr.size(0) > 0:
        # one grouped GEMM per projection; expert banks are [E_local, in, out]
        n_rows = torch.tensor(per_expert, device=x.device)
        offs = torch.cumsum(n_rows, 0).to(torch.int32)
        row_expert = torch.repeat_interleave(torch.arange(len(per_expert), device=x.device), n_rows)
        dt = torch.bfloat16
        h = torch._grouped_mm(xr.to(dt), self.c_fc.weight.to(dt), offs=offs) + self.c_fc.bias.to(dt)[row_expert]
        yr = torch._grouped_mm(gelu_new(h).to(dt), self.c_proj.weight.to(dt), offs=offs) + self.c_proj.bias.to(dt)[row_expert]
    else:
        outs, s = [], 0
        for le, n in enumerate(per_expert):
            h = gelu_new(F.linear(xr[s:s + n], self.c_fc.weight[le].t(), self.c_fc.bias[le]))
            outs.append(F.linear(h, self.c_proj.weight[le].t(), self.c_proj.bias[le]))
            s += n
        yr = torch.cat(outs) if outs else xr.new_zeros(0, d)
    if R > 1:
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel(), device=x.device)
        ys = _A2A.apply(yr[inv], in_splits, out_splits)
    else:
        ys = yr
    w = gates.reshape(-1)[order].unsqueeze(1).to(ys.dtype)
    out = torch.zeros(x2.shape, dtype=ys.dtype, device=x2.device).index_add_(0, tok, ys * w).to(x2.dtype)
    return F.dropout(out.view(B, T, d), self.resid_pdrop, self.training)


def patch_model_for_baseline(model) -> None:
    """SDPA attention everywhere and the EP forward on every MoE layer; slices the expert banks
    to the local experts when running on several ranks."""
    R = dist.get_world_size() if dist.is_initialized() else 1
    r = dist.get_rank() if dist.is_initialized() else 0
    for m in model.modules():
        if isinstance(m, Attention):
            m.use_sdpa = True
        if isinstance(m, MoEMLP):
            if R > 1 and m.c_fc.weight.shape[0] == m.router.out_features:
                E = m.c_fc.weight.shape[0]
                for bank in (m.c_fc, m.c_proj):
                    for p in (bank.weight, bank.bias):
                        p.data = p.data[r * (E // R):(r + 1) * (E // R)].clone()
            m.forward = ep_moe_forward.__get__(m, MoEMLP)
