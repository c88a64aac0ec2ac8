"""The Blackwell execution engine: runs the model as an explicit schedule of sm_100a kernels.

There is no autograd and no tracing compiler on this path.  ``B200Engine`` takes the module tree
of :mod:`allie_b200.models.oracle` (which only *holds* the parameters, under the reference's
state-dict names), moves every parameter into one flat fp32 arena (with matching flat arenas for
gradients, Adam moments and the bf16 shadow copy the tensor cores read), and then executes

    forward  : unpack -> embed -> L x [LN, QKV GEMM, attention, proj GEMM(+bias+dropout+residual),
               LN, fc GEMM(+bias+GELU), proj GEMM(+bias+dropout+residual)] -> LN -> fused lm_head
               GEMM + cross-entropy (loss and d logits, logits never stored) -> fused value/time heads
    backward : hand-scheduled mirror image; weight gradients are accumulated in fp32 straight into
               the gradient arena by the GEMM epilogue (split-K with vector atomics)
    step     : global-norm clip + AdamW + bf16 refresh over the flat arenas (two launches)

which replaces the autocast + ``torch.compile`` + fused-AdamW stack of the reference trainer
(``src/modeling/trainer.py:193-289``).  The residual stream stays fp32 as it does there under
autocast; GEMM operands are bf16 with fp32 accumulation.
"""
from __future__ import annotations

import math
import os
import re

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..data import TIME_MEAN, TIME_STDEV
from ..ops import _lib, kernels as K
from ..ops._lib import ptr, stream_ptr
from ..ops.gemm import gemm
from . import unwrap
from .oracle import Conv1D, MoEMLP

ALIGN = 64  # elements; keeps every parameter view 256-byte (fp32) / 128-byte (bf16) aligned


def partition_parameter_names(model: nn.Module) -> tuple[list[str], list[str]]:
    """(decay, no_decay) parameter names, each sorted by name -- the optimizer ordering of the
    reference (``src/modeling/utils.py:58-98``): weights of linear layers decay; biases, norm and
    embedding weights (and an untied lm_head) do not."""
    decay, no_decay = set(), set()
    params = dict(model.named_parameters())
    for mn, m in model.named_modules():
        for pn, _p in m.named_parameters(recurse=False):
            fpn = f"{mn}.{pn}" if mn else pn
            if fpn not in params:
                continue  # tied duplicate
            if pn.endswith("bias"):
                no_decay.add(fpn)
            elif fpn.endswith("lm_head.weight"):
                no_decay.add(fpn)
            elif isinstance(m, (nn.Linear, Conv1D)) or type(m).__name__ == "ExpertBank":
                decay.add(fpn)
            else:
                no_decay.add(fpn)
    missing = params.keys() - (decay | no_decay)
    assert not missing and not (decay & no_decay), (missing, decay & no_decay)
    return sorted(decay), sorted(no_decay)


def layer_of(name: str) -> int | None:
    """Index of the transformer block a parameter belongs to (None for embeddings, final norm, heads)."""
    m = re.search(r"\.h\.(\d+)\.", name)
    return int(m.group(1)) if m else None


def bucket_of(name: str, n_layer: int, layers_per_bucket: int) -> int:
    """Gradient bucket of a parameter, numbered in the order backward completes them: the final
    norm and the regression heads go with the last blocks (bucket 0), every following bucket takes
    the next ``layers_per_bucket`` blocks going down, and the embeddings (whose gradient is only
    complete after the embedding backward, the very last kernel) go with block 0."""
    nb = max(1, -(-n_layer // layers_per_bucket))
    l = layer_of(name)
    if l is None:
        first = any(k in name for k in ("ln_f.", "value_head", "time_head"))
        return 0 if first else nb - 1
    return (n_layer - 1 - l) // layers_per_bucket


def arena_layout(model: nn.Module, local_names: frozenset = frozenset(), n_layer: int = 1,
                 layers_per_bucket: int | None = None) -> dict:
    """Where every parameter sits in the flat arenas.  The replicated parameters are laid out as
    gradient buckets of ``layers_per_bucket`` transformer blocks each, in the order backward
    finishes them (None: one bucket); inside a bucket come first the weight-decayed GEMM weights
    (which ranks other than a slice's owner need only as bf16), then the weight-decayed
    parameters the kernels read as fp32, then the rest.  Rank-local (expert-parallel) parameters
    follow behind ``sync_end``.  Pure index arithmetic, no device needed."""
    decay, no_decay = partition_parameter_names(model)
    params = dict(model.named_parameters())
    lpb = layers_per_bucket if layers_per_bucket else max(1, n_layer)
    nb = max(1, -(-n_layer // lpb))
    # weight-decayed matrices that the kernels read as fp32 (the two regression heads); every
    # other weight-decayed parameter is a GEMM operand and is only ever read from its bf16 copy
    fp32_read = [n for n in decay if "value_head" in n or "time_head" in n]
    groups: list[tuple[list[str], bool]] = []
    for b in range(nb):
        mine = lambda names: [n for n in names if n not in local_names and bucket_of(n, n_layer, lpb) == b]
        groups.append(([n for n in mine(decay) if n not in fp32_read], True))
        groups.append((mine(fp32_read), True))
        groups.append((mine(no_decay), False))
    n_repl = len(groups)
    groups.append(([n for n in decay if n in local_names], True))
    groups.append(([n for n in no_decay if n in local_names], False))
    offsets: dict[str, int] = {}
    off = 0
    bounds = []
    for g, _ in groups:
        start = off
        for n in g:
            offsets[n] = off
            off += (params[n].numel() + ALIGN - 1) // ALIGN * ALIGN
        bounds.append((start, off))
    # gradient buckets: (start, end of the part other ranks need only as bf16, end of the
    # weight-decayed part, end)
    buckets = [(bounds[3 * b][0], bounds[3 * b][1], bounds[3 * b + 1][1], bounds[3 * b + 2][1]) for b in range(nb)]
    # (start, end, apply weight decay) of every optimizer range, empty ones dropped and adjacent equal ones merged
    regions: list[tuple[int, int, bool]] = []
    for i, (s0, e0) in enumerate(bounds[:n_repl]):
        if e0 > s0:
            if regions and regions[-1][2] == groups[i][1] and regions[-1][1] == s0:
                regions[-1] = (regions[-1][0], e0, groups[i][1])
            else:
                regions.append((s0, e0, groups[i][1]))
    local_regions = [(s0, e0, groups[n_repl + i][1]) for i, (s0, e0) in enumerate(bounds[n_repl:]) if e0 > s0]
    return dict(names=[n for g, _ in groups for n in g], decay_names=frozenset(decay), offsets=offsets,
                buckets=buckets, sync_end=bounds[n_repl - 1][1], regions=regions + local_regions,
                local_regions=local_regions, total=off, layers_per_bucket=lpb,
                shapes={n: tuple(params[n].shape) for n in offsets})


class ParamArena:
    """Flat storage for parameters / gradients / Adam state / bf16 shadows."""

    def __init__(self, model: nn.Module, device: torch.device, symmetric: bool = False,
                 local_names: frozenset = frozenset(), n_layer: int = 1, layers_per_bucket: int | None = None):
        """``symmetric``: allocate the master / gradient / shadow arenas in symmetric memory so
        peer GPUs can address them (the fused NVLink gradient path needs that).
        ``local_names``: parameters that differ per rank (expert-parallel weights); they are laid
        out after the replicated ones and never take part in gradient synchronisation.
        ``layers_per_bucket``: see :func:`arena_layout`."""
        lay = arena_layout(model, local_names, n_layer, layers_per_bucket)
        params = dict(model.named_parameters())
        self.names, self.decay_names, self.offsets = lay["names"], lay["decay_names"], lay["offsets"]
        self.buckets, self.sync_end = lay["buckets"], lay["sync_end"]
        self.regions, self.local_regions = lay["regions"], lay["local_regions"]
        self.layers_per_bucket = lay["layers_per_bucket"]
        off = lay["total"]
        self.total = off
        self.symmetric = symmetric
        if symmetric:
            from ..parallel.nvl import symmetric_empty

            self.master = symmetric_empty(max(off, 64), torch.float32, device).zero_()
            self.grad = symmetric_empty(max(off, 64), torch.float32, device).zero_()
            self.shadow = symmetric_empty(max(off, 64), torch.bfloat16, device).zero_()
        else:
            self.master = torch.zeros(off, dtype=torch.float32, device=device)
            self.grad = torch.zeros(off, dtype=torch.float32, device=device)
            self.shadow = torch.zeros(off, dtype=torch.bfloat16, device=device)
        self.exp_avg: torch.Tensor | None = None
        self.exp_avg_sq: torch.Tensor | None = None
        self.shapes = {n: tuple(params[n].shape) for n in self.names}
        for n in self.names:
            p = params[n]
            view = self.view(self.master, n)
            view.copy_(p.data.to(device=device, dtype=torch.float32))
            p.data = view
            p.grad = self.view(self.grad, n)
        K.cast_bf16(self.master, self.shadow)

    def view(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        o = self.offsets[name]
        shape = self.shapes[name]
        return flat[o:o + math.prod(shape)].view(shape)

    def ensure_state(self) -> None:
        if self.exp_avg is None:
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)

    def refresh_shadow(self) -> None:
        K.cast_bf16(self.master, self.shadow)


class B200Engine:
    def __init__(self, model: nn.Module, device: str | torch.device = "cuda", seed: int = 1234,
                 symmetric: bool = False, layers_per_bucket: int | None = None, expert_parallel: bool = True):
        """``symmetric``: parameter arenas in symmetric memory, laid out as gradient buckets (the
        fused NVLink gradient path).  ``layers_per_bucket``: transformer blocks per gradient bucket
        (default with ``symmetric``: about a dozen buckets).  ``expert_parallel``: with several
        ranks, spread the experts of MoE layers over the ranks (tokens travel to their experts);
        False keeps every expert on every rank and treats expert weights like any other
        data-parallel parameter."""
        import torch.distributed as dist

        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        self.ep_world = dist.get_world_size() if multi and expert_parallel else 1
        self.ep_rank = dist.get_rank() if multi and expert_parallel else 0
        self.device = torch.device(device)
        assert self.device.type == "cuda"
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        _lib.cuda()  # fail loudly if the kernel library is missing
        self.model = model
        self.lm, self.ctrl, self.reg = unwrap(model)
        self.cfg: ModelConfig = self.lm.config
        assert self.cfg.activation_function == "gelu_new"
        model.to(self.device)
        local_names = self._shard_experts(model)
        if symmetric and layers_per_bucket is None:
            layers_per_bucket = max(1, -(-self.cfg.n_layer // 12))
        self.arena = ParamArena(model, self.device, symmetric=symmetric, local_names=local_names,
                                n_layer=self.cfg.n_layer, layers_per_bucket=layers_per_bucket)
        self._moe_ctx: dict = {}
        self._moe_layers: dict = {}
        self.rms = self.cfg.norm_type == "rmsnorm"
        self.seed = seed
        self.step_count = 0      # optimizer steps taken
        self.fwd_count = 0       # forward passes (dropout streams)
        self._bufs: dict[tuple, dict] = {}
        self.max_inference_shapes = 6
        self._names = {id(p): n for n, p in model.named_parameters()}
        self._bind()
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.loss_acc = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.loss_out = torch.zeros(4, dtype=torch.float32, device=self.device)
        self.counts = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.kernel_launches = 0
        # CUDA-graph replay of the micro-step (see enable_step_graph)
        self.step_graph = False
        self._step_graphs: dict[tuple, dict] = {}
        self._salt = torch.tensor([(seed * 0x9E3779B97F4A7C15) & ((1 << 63) - 1)], dtype=torch.int64,
                                  device=self.device)

    # ------------------------------------------------------------- experts
    def _shard_experts(self, model: nn.Module) -> frozenset:
        """Expert parallelism: with R ranks every rank keeps experts [rank*E/R, (rank+1)*E/R) of each
        expert bank.  Returns the names of those rank-local parameters."""
        world, rank = self.ep_world, self.ep_rank
        assert self.cfg.ep_world in (1, world), "the model was built for another expert-parallel layout"
        names = set()
        for mn, m in model.named_modules():
            if type(m).__name__ != "ExpertBank":
                continue
            for pn, p in m.named_parameters(recurse=False):
                names.add(f"{mn}.{pn}")
                if world > 1 and self.cfg.ep_world == 1:     # built with all experts: keep this rank's slice
                    E = p.shape[0]
                    assert E % world == 0, "experts must divide evenly over the ranks"
                    p.data = p.data[rank * (E // world):(rank + 1) * (E // world)].clone()
        return frozenset(names) if world > 1 else frozenset()

    def _moe(self, l: int, M: int, train: bool):
        from ..parallel.moe import MoEContext, MoELayer

        key = (M, train)
        if key not in self._moe_ctx:
            self._moe_ctx[key] = MoEContext(self, M)
        if (l, key) not in self._moe_layers:
            self._moe_layers[(l, key)] = MoELayer(self._moe_ctx[key], self.layers[l], train)
        return self._moe_layers[(l, key)]

    def moe_stats(self) -> dict | None:
        """Routing statistics of the last training forward pass of this rank (None for a dense
        model or before the first pass): the summed load-balance loss, whether any expert buffer
        overflowed its capacity, and per MoE layer how many (token, choice) pairs this rank's
        tokens sent to every expert.  Reads a few small device tensors; call it at logging time."""
        layers = {l: m for (l, key), m in self._moe_layers.items() if key[1]}
        if not layers:
            return None
        ctx = next(iter(layers.values())).ctx
        counts = {l: m.counts.tolist() for l, m in sorted(layers.items())}
        worst = max(max(c) / max(1.0, sum(c) / len(c)) for c in counts.values())
        return {"aux_loss": float(ctx.aux_total), "overflow": bool(int(ctx.overflow[0])),
                "expert_tokens": counts, "max_over_mean_load": worst}

    # ---------------------------------------------------------------- views
    def _n(self, p: nn.Parameter) -> str:
        return self._names[id(p)]

    def _views(self, p: nn.Parameter | None):
        """(fp32 master view, bf16 shadow view, fp32 grad view) of a parameter."""
        if p is None:
            return None, None, None
        n = self._n(p)
        a = self.arena
        return a.view(a.master, n), a.view(a.shadow, n), a.view(a.grad, n)

    def _bind(self) -> None:
        tr = self.lm.transformer
        self.wte = self._views(tr.wte.weight)
        self.wpe = self._views(tr.wpe.weight)
        self.ctrl_w = self._views(self.ctrl.control_embeds.weight) if self.ctrl is not None else (None,) * 3
        self.lnf_w = self._views(tr.ln_f.weight)
        self.lnf_b = self._views(getattr(tr.ln_f, "bias", None))
        self.layers = []
        for blk in tr.h:
            L = dict(
                ln1_w=self._views(blk.ln_1.weight), ln1_b=self._views(getattr(blk.ln_1, "bias", None)),
                ln2_w=self._views(blk.ln_2.weight), ln2_b=self._views(getattr(blk.ln_2, "bias", None)),
                qkv_w=self._views(blk.attn.c_attn.weight), qkv_b=self._views(blk.attn.c_attn.bias),
                o_w=self._views(blk.attn.c_proj.weight), o_b=self._views(blk.attn.c_proj.bias),
                moe=isinstance(blk.mlp, MoEMLP), block=blk)
            L.update(fc_w=self._views(blk.mlp.c_fc.weight), fc_b=self._views(blk.mlp.c_fc.bias),
                     pr_w=self._views(blk.mlp.c_proj.weight), pr_b=self._views(blk.mlp.c_proj.bias))
            if L["moe"]:
                L["router_w"] = self._views(blk.mlp.router.weight)
            self.layers.append(L)
        if self.reg is not None:
            self.wv = self._views(self.reg.value_head[0].weight)
            self.bv = self._views(self.reg.value_head[0].bias)
            self.wt = self._views(self.reg.time_head[0].weight)
            self.bt = self._views(self.reg.time_head[0].bias)

    # -------------------------------------------------------------- buffers
    def _buffers(self, B: int, T: int, train: bool) -> dict:
        key = (B, T, train)
        if key in self._bufs:
            self._bufs[key] = self._bufs.pop(key)          # most recently used goes last
            return self._bufs[key]
        # Inference shapes vary with every request batch (rows x longest game): keep only the most
        # recently used few sets, or a long-running server grows without bound.  Training shapes
        # are fixed by the configuration and stay.
        if not train:
            idle = [k for k in self._bufs if not k[2]]
            for k in idle[:max(0, len(idle) - (self.max_inference_shapes - 1))]:
                del self._bufs[k]
        cfg, dev = self.cfg, self.device
        if T > cfg.n_positions:
            raise ValueError(f"sequence length {T} exceeds the model's {cfg.n_positions} learned positions")
        M, d, F, V = B * T, cfg.n_embd, cfg.ffn_dim, cfg.vocab_size
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        e = lambda *s, dt=bf: torch.empty(*s, dtype=dt, device=dev)
        buf = dict(
            ids=e(M, dt=i32), pos=e(M, dt=i32), labels=e(M, dt=i32), vlab=e(M, dt=f32),
            tlab=e(M, dt=f32), h=e(M, d), meanf=e(M, dt=f32), rstdf=e(M, dt=f32),
            logits=e(M, V), value=e(M, dt=f32), time=e(M, dt=f32), dv=e(M, dt=f32), dt=e(M, dt=f32),
        )
        nl = cfg.n_layer
        if train:
            # every layer keeps what its backward needs
            buf["x"] = [e(M, d, dt=f32) for _ in range(nl + 1)]
            buf["xmid"] = [e(M, d, dt=f32) for _ in range(nl)]
            for name, width in (("ln1", d), ("qkv", 3 * d), ("attn", d), ("ln2", d), ("pre", F), ("act", F)):
                buf[name] = [e(M, width) for _ in range(nl)]
            for name in ("mean1", "rstd1", "mean2", "rstd2"):
                buf[name] = [e(M, dt=f32) for _ in range(nl)]
            buf["lse"] = [e(B, cfg.n_head, T, dt=f32) for _ in range(nl)]
            buf["dx"] = e(M, d, dt=f32)
            buf["delta"] = e(B, cfg.n_head, T, dt=f32)
            if cfg.head_dim == 64:
                buf["dq_acc"] = torch.zeros(M, d, dtype=f32, device=dev)   # kept all-zero between uses
            if T % 32 == 0 and cfg.attn_pdrop > 0:
                buf["dmask"] = [e(B, cfg.n_head, T, T // 32, dt=i32) for _ in range(nl)]
            buf["dyb"] = e(M, d)
            buf["dpre"] = e(M, F)
            buf["dqkv"] = e(M, 3 * d)
            buf["dsmall"] = e(M, d)
        else:
            # inference: two ping-pong residual buffers and one set of scratch activations
            x0, x1 = e(M, d, dt=f32), e(M, d, dt=f32)
            buf["x"] = [x0 if i % 2 == 0 else x1 for i in range(nl + 1)]
            xm = e(M, d, dt=f32)
            buf["xmid"] = [xm] * nl
            shared = {n: e(M, w) for n, w in (("ln1", d), ("qkv", 3 * d), ("attn", d), ("ln2", d), ("act", F))}
            for n, t in shared.items():
                buf[n] = [t] * nl
            for name in ("mean1", "rstd1", "mean2", "rstd2"):
                t = e(M, dt=f32)
                buf[name] = [t] * nl
            lse = e(B, cfg.n_head, T, dt=f32)
            buf["lse"] = [lse] * nl
        self._bufs[key] = buf
        return buf

    # ------------------------------------------------------------ attention
    def _attention_fwd(self, qkv, out, lse, B, T, p_drop, seed, stream_id, drop_mask=None):
        from ..ops.attention import attention_fwd

        attention_fwd(qkv, out, lse, B, T, self.cfg.n_head, self.cfg.head_dim, p_drop, seed, stream_id,
                      drop_mask if p_drop > 0 else None)

    def _attention_bwd(self, qkv, out, lse, dout, dqkv, B, T, p_drop, seed, stream_id, drop_mask=None):
        from ..ops.attention import attention_bwd

        buf = self._buffers(B, T, True)
        attention_bwd(qkv, out, lse, dout, dqkv, buf["delta"], B, T, self.cfg.n_head, self.cfg.head_dim,
                      p_drop, seed, stream_id, drop_mask if p_drop > 0 else None, buf.get("dq_acc"))

    # -------------------------------------------------------------- forward
    def _drop(self, train: bool):
        cfg = self.cfg
        if not train:
            return 0.0, 0.0, 0.0
        return cfg.embd_pdrop, cfg.resid_pdrop, cfg.attn_pdrop

    def forward(self, B: int, T: int, train: bool, seed: int, compute_loss: bool,
                write_grad: bool, kv_hook=None) -> dict:
        """Runs the forward schedule on the ids / labels already placed in the buffers.
        ``kv_hook(layer, qkv)`` is called right after each layer's QKV GEMM (the KV-cache prefill
        uses it to copy keys/values out of the shared inference scratch)."""
        cfg = self.cfg
        buf = self._buffers(B, T, train)
        d, V, eps = cfg.n_embd, cfg.vocab_size, cfg.layer_norm_epsilon
        p_emb, p_res, p_att = self._drop(train)
        x = buf["x"]
        self._has_moe = any(L["moe"] for L in self.layers)
        if self._has_moe:
            for ctx in self._moe_ctx.values():
                ctx.aux_total.zero_()
        K.embed_fwd(buf["ids"], buf["pos"], self.wte[0], self.wpe[0], self.ctrl_w[0], x[0], V, seed, 0, p_emb)
        for l, L in enumerate(self.layers):
            K.layernorm_fwd(x[l], L["ln1_w"][0], L["ln1_b"][0], buf["ln1"][l], buf["mean1"][l],
                            buf["rstd1"][l], eps, self.rms)
            gemm(buf["ln1"][l], L["qkv_w"][1], b_mn=True, out=buf["qkv"][l], bias=L["qkv_b"][0])
            if kv_hook is not None:
                kv_hook(l, buf["qkv"][l])
            self._attention_fwd(buf["qkv"][l], buf["attn"][l], buf["lse"][l], B, T, p_att, seed, 3 + 3 * l,
                                buf["dmask"][l] if "dmask" in buf else None)
            gemm(buf["attn"][l], L["o_w"][1], b_mn=True, out=buf["xmid"][l], bias=L["o_b"][0],
                 resid=x[l], drop_p=p_res, drop_seed=seed, drop_stream=1 + 3 * l)
            K.layernorm_fwd(buf["xmid"][l], L["ln2_w"][0], L["ln2_b"][0], buf["ln2"][l], buf["mean2"][l],
                            buf["rstd2"][l], eps, self.rms)
            if L["moe"]:
                self._moe(l, B * T, train).forward(buf["ln2"][l], buf["xmid"][l], x[l + 1], seed, 2 + 3 * l, p_res)
                continue
            if train:
                # buf["pre"] receives GELU'(pre-activation), all that backward needs of it
                gemm(buf["ln2"][l], L["fc_w"][1], b_mn=True, out=buf["act"][l], bias=L["fc_b"][0], act=1,
                     aux=buf["pre"][l], aux_grad=True)
            else:       # inference: nothing needs the pre-activation
                gemm(buf["ln2"][l], L["fc_w"][1], b_mn=True, out=buf["act"][l], bias=L["fc_b"][0], act=3)
            gemm(buf["act"][l], L["pr_w"][1], b_mn=True, out=x[l + 1], bias=L["pr_b"][0],
                 resid=buf["xmid"][l], drop_p=p_res, drop_seed=seed, drop_stream=2 + 3 * l)
        nl = cfg.n_layer
        K.layernorm_fwd(x[nl], self.lnf_w[0], self.lnf_b[0], buf["h"], buf["meanf"], buf["rstdf"], eps, self.rms)
        lm_coef = self.reg.lm_loss_coef if self.reg is not None else 1.0
        if compute_loss and write_grad:
            # training: output-embedding GEMM, softmax cross entropy and d logits in one kernel;
            # buf["logits"] receives the gradient, the logits themselves are never stored
            self.loss_acc.zero_()
            K.lmhead_ce(buf["h"], self.wte[1], buf["labels"], self.counts[0:1], lm_coef, buf["logits"],
                        self.loss_acc[0:1])
        else:
            gemm(buf["h"], self.wte[1], b_mn=False, out=buf["logits"])
            if compute_loss:
                self.loss_acc.zero_()
                K.ce_fwd_bwd(buf["logits"], buf["labels"], self.counts[0:1], lm_coef, self.loss_acc[0:1], write_grad)
        if self.reg is not None:
            vc = self.reg.value_loss_coef
            K.heads_fwd(buf["h"], self.wv[0], self.bv[0], self.wt[0], self.bt[0],
                        buf["vlab"] if compute_loss else None, buf["tlab"] if compute_loss else None,
                        self.counts, vc, vc, buf["value"], buf["time"], buf["dv"], buf["dt"],
                        self.loss_acc if compute_loss else None)
        if compute_loss:
            lm_coef = self.reg.lm_loss_coef if self.reg is not None else 1.0
            vc = self.reg.value_loss_coef if self.reg is not None else 0.0
            K.loss_finalize(self.loss_acc, self.counts, lm_coef, vc, vc, self.loss_out)
            if self._has_moe:
                aux = self._moe_ctx[(B * T, train)].aux_total
                self.loss_out[0] += self._aux_coef() * aux
        return buf

    def _aux_coef(self) -> float:
        return self.reg.aux_loss_coef if self.reg is not None else self.cfg.aux_loss_coef

    # ------------------------------------------------------------- backward
    def backward(self, B: int, T: int, seed: int, bucket_hook=None) -> None:
        """``bucket_hook(b)`` is called right after the last kernel that writes a gradient of bucket
        ``b`` of the parameter arena has been enqueued (buckets complete in order 0, 1, ...)."""
        cfg = self.cfg
        buf = self._buffers(B, T, True)
        d, V = cfg.n_embd, cfg.vocab_size
        p_emb, p_res, p_att = self._drop(True)
        nl = cfg.n_layer
        dx, dyb, dsmall = buf["dx"], buf["dyb"], buf["dsmall"]
        dpre, dqkv = buf["dpre"], buf["dqkv"]
        F = cfg.ffn_dim
        dlogits = buf["logits"]
        lpb = self.arena.layers_per_bucket
        # lm head: d h = dlogits @ wte ; d wte += dlogits^T @ h
        gemm(dlogits, self.wte[1], b_mn=True, out=dsmall)
        gemm(dlogits, buf["h"], a_mn=True, b_mn=True, out=self.wte[2], accumulate=True)
        s0 = w0 = s1 = w1 = None
        if self.reg is not None:
            K.heads_bwd_w(buf["h"], buf["dv"], buf["dt"], self.wv[2].view(-1), self.bv[2],
                          self.wt[2].view(-1), self.bt[2])
            s0, w0, s1, w1 = buf["dv"], self.wv[0].view(-1), buf["dt"], self.wt[0].view(-1)
        # every LayerNorm backward also emits the masked bf16 gradient of the branch below it and,
        # when that branch ends in a dense projection, the column sums that are its bias gradient
        def proj_bias_grad(layer):
            return None if layer["moe"] else layer["pr_b"][2]

        K.layernorm_bwd(dsmall, buf["x"][nl], buf["meanf"], buf["rstdf"], self.lnf_w[0], None, dx, dyb,
                        self.lnf_w[2], self.lnf_b[2], s0=s0, w0=w0, s1=s1, w1=w1, rms=self.rms,
                        drop_seed=seed, drop_stream=2 + 3 * (nl - 1), drop_p=p_res,
                        dbias=proj_bias_grad(self.layers[nl - 1]))
        for l in range(nl - 1, -1, -1):
            L = self.layers[l]
            # ---- MLP
            if L["moe"]:
                self._moe(l, B * T, True).backward(dyb, buf["ln2"][l], dsmall, self._aux_coef())
            else:
                gemm(buf["act"][l], dyb, a_mn=True, b_mn=True, out=L["pr_w"][2], accumulate=True)
                gemm(dyb, L["pr_w"][1], b_mn=False, out=dpre, act=2, aux=buf["pre"][l], aux_grad=True)
                gemm(buf["ln2"][l], dpre, a_mn=True, b_mn=True, out=L["fc_w"][2], accumulate=True)
                K.colsum_bf16(dpre, L["fc_b"][2])
                gemm(dpre, L["fc_w"][1], b_mn=False, out=dsmall)
            K.layernorm_bwd(dsmall, buf["xmid"][l], buf["mean2"][l], buf["rstd2"][l], L["ln2_w"][0], dx, dx,
                            dyb, L["ln2_w"][2], L["ln2_b"][2], rms=self.rms, drop_seed=seed,
                            drop_stream=1 + 3 * l, drop_p=p_res, dbias=L["o_b"][2])
            # ---- attention
            gemm(buf["attn"][l], dyb, a_mn=True, b_mn=True, out=L["o_w"][2], accumulate=True)
            gemm(dyb, L["o_w"][1], b_mn=False, out=dsmall)
            self._attention_bwd(buf["qkv"][l], buf["attn"][l], buf["lse"][l], dsmall, dqkv, B, T, p_att,
                                seed, 3 + 3 * l, buf["dmask"][l] if "dmask" in buf else None)
            gemm(buf["ln1"][l], dqkv, a_mn=True, b_mn=True, out=L["qkv_w"][2], accumulate=True)
            K.colsum_bf16(dqkv, L["qkv_b"][2])
            gemm(dqkv, L["qkv_w"][1], b_mn=False, out=dsmall)
            K.layernorm_bwd(dsmall, buf["x"][l], buf["mean1"][l], buf["rstd1"][l], L["ln1_w"][0], dx, dx,
                            dyb if l > 0 else None, L["ln1_w"][2], L["ln1_b"][2], rms=self.rms,
                            drop_seed=seed, drop_stream=max(0, 2 + 3 * (l - 1)), drop_p=p_res if l > 0 else 0.0,
                            dbias=proj_bias_grad(self.layers[l - 1]) if l > 0 else None)
            # block l was the lowest of its bucket (the bucket that also holds the embeddings is
            # only complete after the embedding backward below)
            if bucket_hook is not None and l > 0 and (nl - l) % lpb == 0:
                bucket_hook((nl - 1 - l) // lpb)
        K.embed_bwd(buf["ids"], buf["pos"], dx, self.wte[2], self.wpe[2], self.ctrl_w[2], V, seed, 0, p_emb)
        if bucket_hook is not None:
            bucket_hook(len(self.arena.buckets) - 1)

    # ------------------------------------------------------------- public API
    def load_window(self, words: torch.Tensor) -> tuple[int, int]:
        """words: uint32/int32 [B, T] raw training words already on the device."""
        B, T = words.shape
        buf = self._buffers(B, T, True)
        tok_pad = self.cfg.pad_token_id if self.cfg.pad_token_id is not None else -1
        K.unpack_window(words, self.cfg.vocab_size, tok_pad, TIME_MEAN, TIME_STDEV, buf["ids"], buf["pos"],
                        buf["labels"], buf["vlab"], buf["tlab"], self.counts)
        return B, T

    def load_batch(self, batch: dict, train: bool) -> tuple[int, int]:
        """Collated batch (input_ids / position_ids / labels / value_labels / time_labels)."""
        ids = batch["input_ids"]
        B, T = ids.shape
        buf = self._buffers(B, T, train)
        dev = self.device
        buf["ids"].copy_(ids.reshape(-1).to(dev, non_blocking=True))
        if "position_ids" in batch and batch["position_ids"] is not None:
            buf["pos"].copy_(batch["position_ids"].reshape(-1).to(dev, non_blocking=True))
        else:
            buf["pos"].copy_(torch.arange(T, device=dev, dtype=torch.int32).repeat(B))
        if batch.get("labels") is not None:
            lab = batch["labels"].to(dev)
            shifted = torch.full_like(lab, -100)
            shifted[:, :-1] = lab[:, 1:]
            buf["labels"].copy_(shifted.reshape(-1))
            vl = batch.get("value_labels")
            tl = batch.get("time_labels")
            buf["vlab"].copy_((vl if vl is not None else torch.full((B, T), -100.0)).reshape(-1).to(dev))
            buf["tlab"].copy_((tl if tl is not None else torch.full((B, T), -100.0)).reshape(-1).to(dev))
            self.counts[0] = (buf["labels"] >= 0).sum()
            self.counts[1] = (buf["vlab"] != -100).sum()
            self.counts[2] = (buf["tlab"] != -100).sum()
        return B, T

    def _next_seed(self) -> int:
        self.fwd_count += 1
        return (self.seed * 0x9E3779B97F4A7C15 + self.fwd_count * 0xD1B54A32D192ED03) & ((1 << 64) - 1)

    # ------------------------------------------------------- captured micro-step
    def enable_step_graph(self, on: bool = True) -> bool:
        """Replays the micro-step (window unpack, forward, backward: a few thousand launches for
        the medium model) as one CUDA graph per batch shape instead of launching its kernels one
        by one.  A captured launch freezes the arguments it was given by value, and the dropout seed
        is one of them, so while capturing, every kernel that draws a mask is also handed the address
        of a device word (``_salt``) that it folds into its seed; the first node of the graph advances
        that word, which gives every replay fresh masks that its forward and backward kernels agree
        on.  Micro-steps that carry a bucket hook (their reduce-scatter launches take the cross-rank
        epoch by value) and models with MoE layers (same, for every dispatch) keep the ordinary
        launches.  Returns whether the mode is on."""
        self.step_graph = bool(on) and not any(L["moe"] for L in self.layers)
        if not self.step_graph:
            self._step_graphs.clear()
        return self.step_graph

    def _capture_step(self, words: torch.Tensor) -> dict:
        lib = _lib.cuda()
        static = torch.empty_like(words)
        seed = self._next_seed()
        graph = torch.cuda.CUDAGraph()
        launches0 = _lib.LAUNCHES
        assert lib.ab_set_seed_salt(ptr(self._salt)) == 0
        # ALLIE_TRAIN_PDL=1: the captured kernels become links of a programmatic chain (each may take
        # its place on the SMs while the one before it drains).  Off by default: on the medium model
        # the chained graph measured 1.7 % SLOWER than ordinary graph edges (654.6 / 655.1 ms against
        # 644.0 ms per step, same box, alternating runs), unlike the decode step, where it pays.
        lib.ab_set_pdl_chain(int(os.environ.get("ALLIE_TRAIN_PDL", "0") == "1"))
        try:
            # thread-local capture mode: the window-prefetch thread may wait on a copy event
            # (cudaEventSynchronize) while this thread captures
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                assert lib.ab_seed_salt_advance(ptr(self._salt), stream_ptr()) == 0
                _lib.count_launches(1)
                B, T = self.load_window(static)
                self.forward(B, T, True, seed, True, True)
                self.backward(B, T, seed, None)
        finally:
            lib.ab_set_seed_salt(None)
            lib.ab_set_pdl_chain(0)
        captured = _lib.LAUNCHES - launches0
        _lib.count_launches(-captured)       # nothing ran yet: the launches are counted per replay
        return {"graph": graph, "words": static, "launches": captured, "seed": seed}

    def _graph_micro_step(self, words: torch.Tensor) -> torch.Tensor:
        key = (tuple(words.shape), words.dtype)
        entry = self._step_graphs.get(key)
        if entry is None:
            # the first micro-step of a shape runs the ordinary way: it creates the buffers and
            # does every kernel's first-launch set-up, neither of which may happen under capture
            self._step_graphs[key] = {}
            return self.micro_step(words, _no_graph=True)
        if not entry:
            torch.cuda.current_stream().synchronize()
            launches0 = _lib.LAUNCHES
            try:
                entry = self._step_graphs[key] = self._capture_step(words)
            except Exception as e:      # nothing ran during the failed capture: go on with ordinary launches
                import logging

                logging.getLogger(__name__).warning(f"CUDA-graph capture of the micro-step failed ({e}); "
                                                    "continuing with ordinary launches")
                _lib.count_launches(launches0 - _lib.LAUNCHES)
                self.enable_step_graph(False)
                return self.micro_step(words, _no_graph=True)
        entry["words"].copy_(words, non_blocking=True)
        entry["graph"].replay()
        self.fwd_count += 1
        _lib.count_launches(entry["launches"])
        return self.loss_out

    def micro_step(self, words: torch.Tensor, bucket_hook=None, _no_graph: bool = False) -> torch.Tensor:
        """Forward + backward of one micro-batch of raw words; gradients accumulate.  Returns the
        device tensor [loss, lm_loss, value_loss, time_loss] (no host sync).  ``bucket_hook``: see
        :meth:`backward` (given on the last micro-step of an optimizer step)."""
        if self.step_graph and bucket_hook is None and not _no_graph:
            return self._graph_micro_step(words)
        B, T = self.load_window(words)
        seed = self._next_seed()
        self.forward(B, T, True, seed, True, True)
        self.backward(B, T, seed, bucket_hook)
        return self.loss_out

    def micro_step_batch(self, batch: dict) -> torch.Tensor:
        B, T = self.load_batch(batch, True)
        seed = self._next_seed()
        self.forward(B, T, True, seed, True, True)
        self.backward(B, T, seed)
        return self.loss_out

    @torch.no_grad()
    def evaluate_batch(self, batch: dict, with_loss: bool = True) -> dict:
        """Inference forward (no dropout).  Returns logits [B,T,V] bf16, value/time logits and, if
        the batch has labels, the four losses."""
        B, T = self.load_batch(batch, False)
        has_labels = with_loss and batch.get("labels") is not None
        buf = self.forward(B, T, False, 0, has_labels, False)
        V = self.cfg.vocab_size
        out = {"logits": buf["logits"].view(B, T, V), "hidden_states": (buf["h"].view(B, T, -1),)}
        if self.reg is not None:
            out["value_logits"] = buf["value"].view(B, T)
            out["time_logits"] = buf["time"].view(B, T)
        if has_labels:
            lo = self.loss_out.clone()
            out.update(loss=lo[0], lm_loss=lo[1], value_loss=lo[2], time_loss=lo[3])
        return out

    def zero_grad(self) -> None:
        self.arena.grad.zero_()

    def optimizer_step(self, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0,
                       grad_clip: float = 0.0, grad_scale: float = 1.0) -> None:
        a = self.arena
        a.ensure_state()
        self.step_count += 1
        gn = None
        if grad_clip > 0:
            self.gnorm_sq.zero_()
            K.sumsq(a.grad, self.gnorm_sq)
            gn = self.gnorm_sq
        if a.total > a.sync_end and gn is not None:
            import torch.distributed as dist

            if dist.is_initialized() and dist.get_world_size() > 1:
                # rank-local (expert) gradients differ per rank: the global norm needs all of them
                self.gnorm_sq.zero_()
                K.sumsq(a.grad[a.sync_end:], self.gnorm_sq)
                dist.all_reduce(self.gnorm_sq)
                K.sumsq(a.grad[:a.sync_end], self.gnorm_sq)
        for start, end, decays in a.regions:
            if end > start:
                K.adamw(a.master[start:end], a.grad[start:end], a.exp_avg[start:end], a.exp_avg_sq[start:end],
                        a.shadow[start:end], lr, betas[0], betas[1], eps, weight_decay if decays else 0.0,
                        self.step_count, gn, grad_clip, grad_scale)
