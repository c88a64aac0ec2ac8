"""KV-cached, batched leaf evaluator for MCTS on the sm_100a engine.

Every search tree owns a slice of a per-layer key/value cache: slots ``[0, prefix_len)`` hold the
game so far (filled once per move by a batched prefill), the following slots hold one entry per
evaluated tree node.  A search step evaluates one leaf per tree: the leaf's move token goes through
the network as a single new position whose attention reads the prefix slots plus the slots of the
leaf's ancestors (an index list produced by the C++ search), so a leaf costs one token of compute
instead of a re-encode of the whole game (the reference re-encodes, ``src/evaluation/decode.py:356-360``).
The step is a fixed sequence of kernels over static buffers and is replayed as a CUDA graph.
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong

import numpy as np
import torch

from ..ops import _lib, kernels as K
from ..ops._lib import ptr, stream_ptr
from ..ops.gemm import gemm


class KVLeafEvaluator:
    def __init__(self, engine, n_trees: int, max_prefix: int = 320, max_nodes: int = 512,
                 anc_max: int = 128, legal_max: int = 224, use_graph: bool = True):
        self.eng = engine
        cfg = engine.cfg
        self.n, self.S = n_trees, max_prefix + max_nodes
        self.max_prefix, self.anc_max, self.legal_max = max_prefix, anc_max, legal_max
        dev, d, F, V, L = engine.device, cfg.n_embd, cfg.ffn_dim, cfg.vocab_size, cfg.n_layer
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        self.kc = torch.zeros(L, n_trees, self.S, d, dtype=bf, device=dev)
        self.vc = torch.zeros(L, n_trees, self.S, d, dtype=bf, device=dev)
        n = n_trees
        # request block: one int32 buffer, one host->device copy per step
        self.off = {}
        o = 0
        for name, width in (("active", 1), ("tok", 1), ("pos", 1), ("slot", 1), ("prefix_len", 1),
                            ("n_anc", 1), ("n_legal", 1), ("anc", anc_max), ("legal", legal_max)):
            self.off[name] = (o, width)
            o += n * width
        self.req_host = torch.zeros(o, dtype=i32, pin_memory=True)
        self.req_dev = torch.zeros(o, dtype=i32, device=dev)
        self.out_stride = legal_max + 4
        self.out_dev = torch.zeros(n, self.out_stride, dtype=f32, device=dev)
        self.out_host = torch.zeros(n, self.out_stride, dtype=f32, pin_memory=True)
        e = lambda *s, dt=bf: torch.empty(*s, dtype=dt, device=dev)
        self.x = [e(n, d, dt=f32), e(n, d, dt=f32)]
        self.ln, self.qkv, self.att = e(n, d), e(n, 3 * d), e(n, d)
        self.act, self.h, self.logits = e(n, F), e(n, d), e(n, V)
        self.stat = [e(n, dt=f32) for _ in range(2)]
        self.value, self.time = e(n, dt=f32), e(n, dt=f32)
        self.resign_id = 1992
        self.graph = None
        self.use_graph = use_graph
        self.steps = 0

    def view(self, t: torch.Tensor, name: str) -> torch.Tensor:
        o, w = self.off[name]
        v = t[o:o + self.n * w]
        return v.view(self.n, w) if w > 1 else v

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, token_rows: list[np.ndarray]):
        """Runs the prompts (one per tree, raw token ids incl. ELO pseudo-ids) through the network,
        fills cache slots [0, len) of every tree and returns host tensors
        (last-position logits [n, V] fp32, value [n], time [n])."""
        eng, n = self.eng, self.n
        assert len(token_rows) == n
        lens = [len(r) for r in token_rows]
        Lp = max(lens)
        assert Lp <= self.max_prefix
        pad = eng.cfg.pad_token_id if eng.cfg.pad_token_id is not None else 0
        ids = np.full((n, Lp), pad, dtype=np.int64)
        for i, r in enumerate(token_rows):
            ids[i, :len(r)] = r
        batch = {"input_ids": torch.from_numpy(ids)}
        B, T = eng.load_batch(batch, False)
        len_dev = torch.tensor(lens, dtype=torch.int32, device=eng.device)
        d = eng.cfg.n_embd

        def hook(l, qkv):
            rc = _lib.cuda().ab_kv_store(ptr(qkv), ptr(self.kc[l]), ptr(self.vc[l]), ptr(len_dev), c_int(n),
                                         c_int(Lp), c_int(self.S), c_int(d), c_int(eng.cfg.head_dim), stream_ptr())
            assert rc == 0
            _lib.count_launches(1)

        buf = eng.forward(B, T, False, 0, False, False, kv_hook=hook)
        rows = torch.arange(n, device=eng.device) * Lp + (len_dev.long() - 1)
        logits = buf["logits"][rows].float().cpu()
        if eng.reg is not None:
            value, time = buf["value"][rows].cpu(), buf["time"][rows].cpu()
        else:
            value = time = torch.zeros(n)
        self.view(self.req_host, "prefix_len").copy_(torch.tensor(lens, dtype=torch.int32))
        return logits, value, time

    # --------------------------------------------------------------------- step
    def _launch_step(self) -> None:
        eng, cfg, n = self.eng, self.eng.cfg, self.n
        rd = self.req_dev
        V, eps = cfg.vocab_size, cfg.layer_norm_epsilon
        lib = _lib.cuda()
        K.embed_fwd(self.view(rd, "tok"), self.view(rd, "pos"), eng.wte[0], eng.wpe[0], eng.ctrl_w[0],
                    self.x[0], V, 0, 0, 0.0)
        x = self.x[0]
        scale = 1.0 / cfg.head_dim ** 0.5
        # the kernels of the step are programmatic dependents of the kernel before them: a GEMM's
        # set-up and first ring of weight tiles, the attention kernel's prompt-slot chunks and every
        # launch overlap the previous kernel (ALLIE_DECODE_PDL=0 turns it off)
        pdl = os.environ.get("ALLIE_DECODE_PDL", "1") != "0"
        for l, Ly in enumerate(eng.layers):
            K.layernorm_fwd(x, Ly["ln1_w"][0], Ly["ln1_b"][0], self.ln, self.stat[0], self.stat[1], eps, eng.rms,
                            dependent=pdl)
            gemm(self.ln, Ly["qkv_w"][1], b_mn=True, out=self.qkv, bias=Ly["qkv_b"][0], dependent=pdl)
            rc = lib.ab_decode_attn(ptr(self.qkv), ptr(self.kc[l]), ptr(self.vc[l]), ptr(self.view(rd, "active")),
                                    ptr(self.view(rd, "slot")), ptr(self.view(rd, "prefix_len")),
                                    ptr(self.view(rd, "anc")), c_int(self.anc_max), ptr(self.view(rd, "n_anc")),
                                    ptr(self.att), c_int(n), c_int(cfg.n_head), c_int(cfg.head_dim),
                                    c_int(self.S), c_float(scale), c_int(int(pdl)), ptr(_lib.status_word()),
                                    stream_ptr())
            assert rc == 0
            _lib.count_launches(1)
            # residual updates in place: with a few hundred rows they run as split-K reduce-adds
            gemm(self.att, Ly["o_w"][1], b_mn=True, out=x, bias=Ly["o_b"][0], resid=x, dependent=pdl)
            K.layernorm_fwd(x, Ly["ln2_w"][0], Ly["ln2_b"][0], self.ln, self.stat[0], self.stat[1], eps, eng.rms,
                            dependent=pdl)
            gemm(self.ln, Ly["fc_w"][1], b_mn=True, out=self.act, bias=Ly["fc_b"][0], act=3, dependent=pdl)
            gemm(self.act, Ly["pr_w"][1], b_mn=True, out=x, bias=Ly["pr_b"][0], resid=x, dependent=pdl)
        K.layernorm_fwd(x, eng.lnf_w[0], eng.lnf_b[0], self.h, self.stat[0], self.stat[1], eps, eng.rms,
                        dependent=pdl)
        gemm(self.h, eng.wte[1], b_mn=False, out=self.logits, dependent=pdl)
        has_heads = eng.reg is not None
        if has_heads:
            K.heads_fwd(self.h, eng.wv[0], eng.bv[0], eng.wt[0], eng.bt[0], None, None, eng.counts, 0.0, 0.0,
                        self.value, self.time, None, None, None)
        rc = lib.ab_policy_epilogue(ptr(self.logits), c_longlong(self.logits.stride(0)),
                                    ptr(self.view(rd, "active")), ptr(self.view(rd, "legal")),
                                    c_int(self.legal_max), ptr(self.view(rd, "n_legal")),
                                    ptr(self.value if has_heads else None), ptr(self.time if has_heads else None),
                                    c_int(self.resign_id), c_float(1.0), ptr(self.out_dev),
                                    c_int(self.out_stride), c_int(n), stream_ptr())
        assert rc == 0
        _lib.count_launches(1)

    @torch.no_grad()
    def step(self) -> np.ndarray:
        """Evaluates the requests currently in ``req_host``; returns the packed result rows
        (host, [n, legal_max + 4]: priors..., value, time, resign logit, best legal logit)."""
        self.req_dev.copy_(self.req_host, non_blocking=True)
        if self.use_graph:
            if self.graph is None:
                self._launch_step()                      # warm-up outside capture (first-launch set-up)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._launch_step()
                self.graph = g
            self.graph.replay()
        else:
            self._launch_step()
        self.out_host.copy_(self.out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.steps += 1
        return self.out_host.numpy()
