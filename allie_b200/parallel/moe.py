"""Expert-parallel MoE feed-forward on the engine (kernels in ``csrc/moe.cu``).

Every rank owns ``E / R`` consecutive experts.  A layer runs as

    router GEMM -> route (softmax, top-2, counts) -> count exchange + plan -> dispatch (token rows
    stored directly into the owning rank's receive buffer) -> per-expert tcgen05 GEMMs sized on
    the device (fc + GELU, proj) -> return (rows stored back at their return addresses) ->
    combine (gate-weighted sum + dropout + residual)

and backward mirrors it.  Buffers that other ranks write (receive rows, return addresses, combine
rows, count matrix, flags) live in symmetric memory when R > 1; with R = 1 the same kernels run on
plain tensors with the rank as its own only peer.  Each local expert has a fixed region of
``cap_e`` rows (``capacity_factor`` times the balanced share); rows beyond it are dropped and
reported through ``overflow``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_uint, c_ulonglong, c_void_p

import torch
import torch.distributed as dist

from ..ops import _lib, kernels as K
from ..ops._lib import ptr, stream_ptr
from ..ops.gemm import gemm

PH_COUNTS, PH_DISPATCH, PH_RETURN, PH_BWD_DISPATCH, PH_BWD_RETURN = 0, 1, 2, 3, 4


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
        self.cap_e = (cap + 127) // 128 * 128
        self.rows = self.El * self.cap_e
        dev = engine.device
        self.flags, self.p_flags = self.shared(3 * 32 * 2, torch.int32)
        self.flags.zero_()
        self.all_counts, self.p_all_counts = self.shared(self.R * self.E, torch.int32)
        self.epoch = [0] * 8
        self.ticket = torch.zeros(8, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        e = lambda *s, dt=bf: torch.zeros(*s, dtype=dt, device=dev)
        # forward scratch shared by the layers
        self.yr = e(self.rows, self.d)
        # backward buffers shared by the layers
        self.dyr, self.p_dyr = self.shared(self.rows * self.d, bf)
        self.dyr = self.dyr.view(self.rows, self.d)
        self.dxcomb, self.p_dxcomb = self.shared(M * 2 * self.d, bf)
        self.dxcomb = self.dxcomb.view(M * 2, self.d)
        self.dpre, self.dxr = e(self.rows, self.F), e(self.rows, self.d)
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

    def wait(self, phase: int, epoch: int) -> None:
        flags_local = self.flags
        _ck(_lib.cuda().ab_nvl_wait(ptr(flags_local), c_int(phase), c_int(self.R), c_uint(epoch),
                                    ptr(_lib.status_word()), stream_ptr()), "ab_nvl_wait")


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
        self.counts, self.psum = e(E, dt=i32), e(E, dt=f32)
        self.send_off, self.cursor = e(E, dt=i32), e(E, dt=i32)
        self.rows_local, self.rows_pad = e(c.El, dt=i32), e(c.El, dt=i32)
        self.xr, self.p_xr = c.shared(c.rows * c.d, bf)
        self.xr = self.xr.view(c.rows, c.d)
        self.ret, self.p_ret = c.shared(c.rows, i32)
        self.ycomb, self.p_ycomb = c.shared(M * 2 * c.d, bf)
        self.ycomb = self.ycomb.view(M * 2, c.d)
        self.pre, self.act = e(c.rows, c.F), e(c.rows, c.F)

    # -------------------------------------------------------------------------------- forward
    def forward(self, ln2, resid, out, seed: int, stream_id: int, p_drop: float) -> None:
        c, v, lib = self.ctx, self.v, _lib.cuda()
        st = _lib.status_word()
        gemm(ln2, v["router_w"][1], b_mn=False, out=self.logits)
        _ck(lib.ab_moe_route(ptr(self.logits), c_int(c.M), c_int(c.E), ptr(self.topi), ptr(self.gates),
                             ptr(self.probs), ptr(self.counts), ptr(self.psum), stream_ptr()), "ab_moe_route")
        ep = c.next_epoch(PH_COUNTS)
        _ck(lib.ab_moe_exchange_plan(c.p_all_counts, c.p_flags, ptr(self.counts), ptr(self.send_off),
                                     ptr(self.rows_local), ptr(self.rows_pad), ptr(self.cursor), ptr(c.overflow),
                                     c_int(c.R), c_int(c.E), c_int(c.El), c_int(c.cap_e), c_int(c.rank),
                                     c_int(PH_COUNTS), c_uint(ep), ptr(st), stream_ptr()), "ab_moe_exchange_plan")
        ep = c.next_epoch(PH_DISPATCH)
        _ck(lib.ab_moe_dispatch(self.p_xr, self.p_ret, c.p_flags, ptr(ln2), ptr(self.topi), ptr(self.send_off),
                                ptr(self.cursor), ptr(self.dest), ptr(c.ticket), c_int(c.M), c_int(c.d), c_int(c.El),
                                c_int(c.cap_e), c_int(c.rank), c_int(c.R), c_int(PH_DISPATCH), c_uint(ep),
                                stream_ptr()), "ab_moe_dispatch")
        c.wait(PH_DISPATCH, ep)
        for le in range(c.El):
            r0, r1 = le * c.cap_e, (le + 1) * c.cap_e
            lim = self.rows_local[le:le + 1]
            gemm(self.xr[r0:r1], v["fc_w"][1][le], b_mn=True, out=self.act[r0:r1], bias=v["fc_b"][0][le], act=1,
                 aux=self.pre[r0:r1], m_limit=lim)
            gemm(self.act[r0:r1], v["pr_w"][1][le], b_mn=True, out=c.yr[r0:r1], bias=v["pr_b"][0][le], m_limit=lim)
        ep = c.next_epoch(PH_RETURN)
        _ck(lib.ab_moe_return(self.p_ycomb, c.p_flags, ptr(c.yr), ptr(self.ret), ptr(self.rows_local),
                              c_void_p(c.ticket.data_ptr() + 4), c_int(c.d), c_int(c.El), c_int(c.cap_e),
                              c_int(c.rank), c_int(c.R), c_int(PH_RETURN), c_uint(ep), stream_ptr()), "ab_moe_return")
        c.wait(PH_RETURN, ep)
        _ck(lib.ab_moe_combine(ptr(self.ycomb), ptr(self.gates), ptr(self.dest), ptr(resid), ptr(out), c_int(c.M),
                               c_int(c.d), c_ulonglong(seed), c_uint(stream_id), c_uint(_lib.dropout_thr16(p_drop)),
                               stream_ptr()), "ab_moe_combine")
        # load-balance loss of this layer: E * sum_e f_e * P_e
        frac = self.counts.float() / (c.M * c.k)
        c.aux_total += c.E * (frac * (self.psum / c.M)).sum()

    # ------------------------------------------------------------------------------- backward
    def backward(self, dyb, ln2, dln2_out, aux_coef: float) -> None:
        """dyb: bf16 gradient of the layer output; writes the gradient w.r.t. ``ln2`` (the layer
        input) into ``dln2_out`` and accumulates all parameter gradients."""
        c, v, lib = self.ctx, self.v, _lib.cuda()
        ep = c.next_epoch(PH_BWD_DISPATCH)
        _ck(lib.ab_moe_combine_bwd_dispatch(c.p_dyr, c.p_flags, ptr(dyb), ptr(self.ycomb), ptr(self.gates),
                                            ptr(self.dest), ptr(c.dgate), c_void_p(c.ticket.data_ptr() + 8),
                                            c_int(c.M), c_int(c.d), c_int(c.rank), c_int(c.R),
                                            c_int(PH_BWD_DISPATCH), c_uint(ep), stream_ptr()),
            "ab_moe_combine_bwd_dispatch")
        c.wait(PH_BWD_DISPATCH, ep)
        _ck(lib.ab_moe_zero_pad(ptr(c.dyr), ptr(self.rows_local), ptr(self.rows_pad), c_int(c.El), c_int(c.cap_e),
                                c_int(c.d), stream_ptr()), "ab_moe_zero_pad")
        for le in range(c.El):
            r0, r1 = le * c.cap_e, (le + 1) * c.cap_e
            lim, pad = self.rows_local[le:le + 1], self.rows_pad[le:le + 1]
            dyr, dpre = c.dyr[r0:r1], c.dpre[r0:r1]
            gemm(self.act[r0:r1], dyr, a_mn=True, b_mn=True, out=v["pr_w"][2][le], accumulate=True, k_limit=pad)
            K.colsum_bf16(dyr, v["pr_b"][2][le], m_limit=pad)
            gemm(dyr, v["pr_w"][1][le], b_mn=False, out=dpre, act=2, aux=self.pre[r0:r1], m_limit=lim)
            gemm(self.xr[r0:r1], dpre, a_mn=True, b_mn=True, out=v["fc_w"][2][le], accumulate=True, k_limit=pad)
            K.colsum_bf16(dpre, v["fc_b"][2][le], m_limit=pad)
            gemm(dpre, v["fc_w"][1][le], b_mn=False, out=c.dxr[r0:r1], m_limit=lim)
        ep = c.next_epoch(PH_BWD_RETURN)
        _ck(lib.ab_moe_return(c.p_dxcomb, c.p_flags, ptr(c.dxr), ptr(self.ret), ptr(self.rows_local),
                              c_void_p(c.ticket.data_ptr() + 12), c_int(c.d), c_int(c.El), c_int(c.cap_e),
                              c_int(c.rank), c_int(c.R), c_int(PH_BWD_RETURN), c_uint(ep), stream_ptr()),
            "ab_moe_return")
        c.wait(PH_BWD_RETURN, ep)
        aux_scale = aux_coef * c.E / (float(c.M) * c.k * c.M)
        _ck(lib.ab_moe_router_bwd(ptr(self.probs), ptr(self.topi), ptr(self.gates), ptr(c.dgate), ptr(self.counts),
                                  c_float(aux_scale), c_float(1.0), c_int(c.M), c_int(c.E), ptr(c.dlogits),
                                  stream_ptr()), "ab_moe_router_bwd")
        gemm(c.dlogits, ln2, a_mn=True, b_mn=True, out=v["router_w"][2], accumulate=True)
        gemm(c.dlogits, v["router_w"][1], b_mn=True, out=dln2_out)
        _ck(lib.ab_moe_dx_sum(ptr(dln2_out), ptr(c.dxcomb), ptr(self.dest), c_int(c.M), c_int(c.d), stream_ptr()),
            "ab_moe_dx_sum")
