"""Expert-parallel MoE feed-forward on the engine (kernels in ``csrc/moe.cu`` and
``csrc/gemm_grouped.cu``).

Every rank owns ``E / R`` consecutive experts.  A layer's forward is five launches:

    router GEMM
    route + plan + dispatch  (softmax, top-2, load-balance loss; count exchange; token rows stored
                              directly into the owning rank's receive buffer, with an arrival
                              counter per 128-row block)
    grouped expert GEMM up   (fc + bias + GELU for all local experts in one persistent CTA-pair
                              launch; each tile starts once its rows have arrived)
    grouped expert GEMM down (proj + bias; the epilogue stores every result row back into the
                              source rank's combine buffer at its return address and releases a
                              flag when the whole launch is done)
    combine                  (waits for all ranks' flags; gate-weighted sum + dropout + residual)

and backward mirrors it (the weight gradients are grouped launches contracting over each expert's
live rows; the input-gradient GEMM scatters its rows back like the down projection).  Buffers that
other ranks write (receive rows, return addresses, combine rows, count matrix, counters, flags)
live in symmetric memory when R > 1; with R = 1 the same kernels run on plain tensors with the
rank as its own only peer.  Each local expert has a fixed region of ``cap_e`` rows
(``capacity_factor`` times the balanced share); rows beyond it are dropped and reported through
``overflow``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_uint, c_ulonglong, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib, kernels as K
from ..ops._lib import ptr, stream_ptr
from ..ops.gemm import gemm, gemm_grouped

PH_COUNTS, PH_RETURN, PH_BWD_RETURN = 0, 2, 4


def _ptrs(ps) -> ctypes.Array:
    arr = (c_void_p * 8)()
    for i, p in enumerate(ps):
        arr[i] = int(p)
    return arr


def _ck(rc: int, name: str, launches: int = 1) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    _lib.count_launches(launches)


class MoEContext:
    """Per-engine state shared by all MoE layers: the expert-parallel group, flags, shared
    backward buffers and the allocator for peer-visible memory."""

    def __init__(self, engine, M: int):
        cfg = engine.cfg
        self.eng = engine
        self.R, self.rank = engine.ep_world, engine.ep_rank      # 1, 0 unless experts are spread over the ranks
        self.E, self.k = cfg.num_experts, cfg.moe_top_k
        assert self.k == 2, "the routing kernels implement top-2"
        assert self.E % self.R == 0
        self.El = self.E // self.R
        self.M, self.d, self.F = M, cfg.n_embd, cfg.moe_ffn or cfg.ffn_dim
        balanced = self.R * M * self.k / self.E             # rows per expert if routing were uniform
        cap = int(min(self.R * M * self.k, max(128.0, cfg.capacity_factor * balanced)))
        self.cap_e = (cap + 255) // 256 * 256       # whole 256-row CTA-pair tiles
        self.rows = self.El * self.cap_e
        dev = engine.device
        self.flags, self.p_flags = self.shared(3 * 32 * 2, torch.int32)
        self.flags.zero_()
        self.all_counts, self.p_all_counts = self.shared(self.R * self.E, torch.int32)
        self.epoch = [0] * 8
        self.ticket = torch.zeros(8, dtype=torch.int32, device=dev)
        self.go = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        e = lambda *s, dt=bf: torch.zeros(*s, dtype=dt, device=dev)
        # backward buffers shared by the layers
        self.dyr, self.p_dyr = self.shared(self.rows * self.d, bf)
        self.dyr = self.dyr.view(self.rows, self.d)
        self.dxcomb, self.p_dxcomb = self.shared(M * 2 * self.d, bf)
        self.dxcomb = self.dxcomb.view(M * 2, self.d)
        self.dpre = e(self.rows, self.F)
        # arrival counters of the token rows this rank receives, one per 128 rows (cleared and used
        # within one layer's forward, so the layers share them)
        self.ready_fwd, self.p_ready_fwd = self.shared(self.rows // 128, torch.int32)
        self.dgate, self.dlogits = e(M * 2, dt=f32), e(M, self.E)
        self.aux_total = torch.zeros((), dtype=f32, device=dev)
        if self.R > 1:
            torch.cuda.synchronize()
            dist.barrier()

    def shared(self, n: int, dtype):
        """(tensor, pointer table of every rank's copy)."""
        if self.R == 1:
            t = torch.zeros(n, dtype=dtype, device=self.eng.device)
            return t, _ptrs([t.data_ptr()])
        from .nvl import rendezvous, symmetric_empty

        t = symmetric_empty(n, dtype, self.eng.device)
        t.zero_()
        h = rendezvous(t)
        return t, _ptrs(h.buffer_ptrs)

    def next_epoch(self, phase: int) -> int:
        self.epoch[phase] += 1
        return self.epoch[phase]


class MoELayer:
    def __init__(self, ctx: MoEContext, views: dict, train: bool):
        self.ctx, self.v = ctx, views
        c = ctx
        dev = c.eng.device
        f32, i32, bf = torch.float32, torch.int32, torch.bfloat16
        e = lambda *s, dt=bf: torch.zeros(*s, dtype=dt, device=dev)
        M, E = c.M, c.E
        self.logits, self.probs = e(M, E, dt=f32), e(M, E, dt=f32)
        self.topi, self.gates, self.dest = e(M * 2, dt=i32), e(M * 2, dt=f32), e(M * 2, dt=i32)
        self.cnt_ps = e(2 * E, dt=i32)                        # counts and probability sums, cleared together
        self.counts, self.psum = self.cnt_ps[:E], self.cnt_ps[E:].view(f32)
        self.send_off, self.cursor = e(E, dt=i32), e(E, dt=i32)
        self.rows_local, self.rows_pad = e(c.El, dt=i32), e(c.El, dt=i32)
        self.xr, self.p_xr = c.shared(c.rows * c.d, bf)
        self.xr = self.xr.view(c.rows, c.d)
        self.ret, self.p_ret = c.shared(c.rows, i32)
        self.ycomb, self.p_ycomb = c.shared(M * 2 * c.d, bf)
        self.ycomb = self.ycomb.view(M * 2, c.d)
        self.pre, self.act = e(c.rows, c.F), e(c.rows, c.F)
        # arrival counters of the gradient rows: cleared in this layer's forward, filled in its
        # backward, with other layers' backward passes in between - one set per layer
        self.ready_bwd, self.p_ready_bwd = c.shared(c.rows // 128, i32)

    # -------------------------------------------------------------------------------- forward
    def _scatter(self, peers, phase: int, epoch: int, ticket_slot: int) -> dict:
        c = self.ctx
        return dict(ret=self.ret, peers=peers, flags=c.p_flags, phase=phase, epoch=epoch, rank=c.rank, world=c.R,
                    ticket=c.ticket.data_ptr() + 4 * ticket_slot)

    def forward(self, ln2, resid, out, seed: int, stream_id: int, p_drop: float) -> None:
        c, v, lib = self.ctx, self.v, _lib.cuda()
        st = _lib.status_word()
        gemm(ln2, v["router_w"][1], b_mn=False, out=self.logits)
        self.cnt_ps.zero_()
        ep = c.next_epoch(PH_COUNTS)
        _ck(lib.ab_moe_route_plan_dispatch(
            ptr(self.logits), ptr(self.topi), ptr(self.gates), ptr(self.probs), ptr(self.counts), ptr(self.psum),
            ptr(c.aux_total), c.p_all_counts, c.p_flags, ptr(self.send_off), ptr(self.rows_local), ptr(self.rows_pad),
            ptr(self.cursor), ptr(c.overflow), ptr(c.ready_fwd), ptr(self.ready_bwd), ptr(c.ticket), ptr(c.go),
            self.p_xr, self.p_ret, c.p_ready_fwd, ptr(ln2), ptr(self.dest), c_int(c.M), c_int(c.E), c_int(c.El),
            c_int(c.R), c_int(c.rank), c_int(c.cap_e), c_int(c.d), c_int(PH_COUNTS), c_uint(ep), ptr(st),
            stream_ptr()), "ab_moe_route_plan_dispatch")
        # all local experts in one launch each; the first waits tile by tile for the dispatched rows
        gemm_grouped(self.xr, v["fc_w"][1], self.rows_local, c.cap_e, mode=1, b_mn=True, out=self.act,
                     bias=v["fc_b"][0], act=1, aux=self.pre, aux_grad=True, tile_ready=c.ready_fwd)
        ep = c.next_epoch(PH_RETURN)
        gemm_grouped(self.act, v["pr_w"][1], self.rows_local, c.cap_e, mode=1, b_mn=True, bias=v["pr_b"][0],
                     scatter=self._scatter(self.p_ycomb, PH_RETURN, ep, 1))
        _ck(lib.ab_moe_combine(ptr(self.ycomb), ptr(self.gates), ptr(self.dest), ptr(resid), ptr(out), c_int(c.M),
                               c_int(c.d), c_ulonglong(seed), c_uint(stream_id), c_uint(_lib.dropout_thr16(p_drop)),
                               ptr(c.flags), c_int(PH_RETURN), c_int(c.R), c_uint(ep), ptr(st), stream_ptr()),
            "ab_moe_combine")

    # ------------------------------------------------------------------------------- backward
    def backward(self, dyb, ln2, dln2_out, aux_coef: float) -> None:
        """dyb: bf16 gradient of the layer output; writes the gradient w.r.t. ``ln2`` (the layer
        input) into ``dln2_out`` and accumulates all parameter gradients."""
        c, v, lib = self.ctx, self.v, _lib.cuda()
        st = _lib.status_word()
        _ck(lib.ab_moe_combine_bwd_dispatch(c.p_dyr, self.p_ready_bwd, ptr(c.dyr), ptr(self.rows_local),
                                            ptr(self.rows_pad), c_int(c.El), c_int(c.cap_e), ptr(dyb),
                                            ptr(self.ycomb), ptr(self.gates), ptr(self.dest), ptr(c.dgate),
                                            c_int(c.M), c_int(c.d), c_int(c.rank), c_int(c.R), stream_ptr()),
            "ab_moe_combine_bwd_dispatch")
        rows, cap = self.rows_local, c.cap_e
        gemm_grouped(self.act, c.dyr, rows, cap, mode=2, out=v["pr_w"][2], tile_ready=self.ready_bwd)
        K.colsum_grouped_bf16(c.dyr, v["pr_b"][2], rows, cap)
        gemm_grouped(c.dyr, v["pr_w"][1], rows, cap, mode=1, b_mn=False, out=c.dpre, act=2, aux=self.pre, aux_grad=True)
        gemm_grouped(self.xr, c.dpre, rows, cap, mode=2, out=v["fc_w"][2])
        K.colsum_grouped_bf16(c.dpre, v["fc_b"][2], rows, cap)
        ep = c.next_epoch(PH_BWD_RETURN)
        gemm_grouped(c.dpre, v["fc_w"][1], rows, cap, mode=1, b_mn=False,
                     scatter=self._scatter(c.p_dxcomb, PH_BWD_RETURN, ep, 2))
        aux_scale = aux_coef * c.E / (float(c.M) * c.k * c.M)
        _ck(lib.ab_moe_router_bwd(ptr(self.probs), ptr(self.topi), ptr(self.gates), ptr(c.dgate), ptr(self.counts),
                                  c_float(aux_scale), c_float(1.0), c_int(c.M), c_int(c.E), ptr(c.dlogits),
                                  stream_ptr()), "ab_moe_router_bwd")
        gemm(c.dlogits, ln2, a_mn=True, b_mn=True, out=v["router_w"][2], accumulate=True)
        gemm(c.dlogits, v["router_w"][1], b_mn=True, out=dln2_out)
        _ck(lib.ab_moe_dx_sum(ptr(dln2_out), ptr(c.dxcomb), ptr(self.dest), c_int(c.M), c_int(c.d), ptr(c.flags),
                              c_int(PH_BWD_RETURN), c_int(c.R), c_uint(ep), ptr(st), stream_ptr()), "ab_moe_dx_sum")
