"""Plain-PyTorch statement of the model: the CPU path and the numerical ground truth for every
sm_100a kernel.

It is a GPT-2 decoder (learned absolute positions, pre-LayerNorm blocks, ``gelu_new`` MLP, tied
output embedding) with the two wrappers of the reference:

* soft ELO conditioning -- input ids >= vocab_size are ratings, embedded as
  ``[e, 1-e] @ control_embeds`` with ``e = (clamp(id - V, 500, 3000) - 500) / 2500``
  (reference ``src/modeling/model.py:13-57``);
* a value head (``tanh``) and a think-time head on the final hidden state with masked-MSE losses,
  total = lm*lm_coef + value*value_coef + time*value_coef -- the think-time loss really is scaled
  by ``value_loss_coef`` (reference ``src/modeling/model.py:60-147``).

Module nesting and parameter names reproduce the reference state-dict keys
(``model.model.transformer.h.0.attn.c_attn.weight`` with the GPT-2 ``[in, out]`` weight layout,
``model.control_embeds.weight``, ``value_head.0.weight`` ...), so checkpoints are interchangeable.
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig

IGNORE = -100


def gelu_new(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


class Conv1D(nn.Module):
    """Linear layer with the weight stored ``[in_features, out_features]`` (GPT-2 convention)."""

    def __init__(self, nf: int, nx: int):
        super().__init__()
        self.nf = nf
        self.weight = nn.Parameter(torch.empty(nx, nf))
        self.bias = nn.Parameter(torch.zeros(nf))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.addmm(self.bias, x.reshape(-1, x.size(-1)), self.weight).view(*x.shape[:-1], self.nf)


class RMSNorm(nn.Module):
    def __init__(self, d: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


def make_norm(cfg: ModelConfig) -> nn.Module:
    if cfg.norm_type == "rmsnorm":
        return RMSNorm(cfg.n_embd, cfg.layer_norm_epsilon)
    return nn.LayerNorm(cfg.n_embd, eps=cfg.layer_norm_epsilon)


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.n_head, self.head_dim = cfg.n_head, cfg.head_dim
        self.c_attn = Conv1D(3 * cfg.n_embd, cfg.n_embd)
        self.c_proj = Conv1D(cfg.n_embd, cfg.n_embd)
        self.attn_pdrop, self.resid_pdrop = cfg.attn_pdrop, cfg.resid_pdrop

    def forward(self, x, key_mask: Optional[torch.Tensor] = None, past=None):
        """``past`` = (k, v) [B,H,Tp,hd] of earlier positions (KV cache) or None.  Returns
        (out, (k, v))."""
        B, T, d = x.shape
        q, k, v = self.c_attn(x).split(d, dim=2)
        sh = lambda t: t.view(B, T, self.n_head, self.head_dim).transpose(1, 2)
        q, k, v = sh(q), sh(k), sh(v)
        if past is not None:
            k = torch.cat([past[0], k], dim=2)
            v = torch.cat([past[1], v], dim=2)
        Tk = k.size(2)
        if getattr(self, "use_sdpa", False) and past is None and key_mask is None:
            # library attention (used by the plain-PyTorch baselines, not by the oracle tests)
            y = F.scaled_dot_product_attention(q, k, v, is_causal=True,
                                               dropout_p=self.attn_pdrop if self.training else 0.0)
            y = y.transpose(1, 2).reshape(B, T, d)
            return F.dropout(self.c_proj(y), self.resid_pdrop, self.training), (k, v)
        att = (q @ k.transpose(-1, -2)) / math.sqrt(self.head_dim)
        causal = torch.ones(Tk, Tk, dtype=torch.bool, device=x.device).tril()[Tk - T:]
        att = att.masked_fill(~causal, float("-inf"))
        if key_mask is not None:
            att = att.masked_fill(~key_mask[:, None, None, :].bool(), torch.finfo(att.dtype).min)
        att = F.dropout(F.softmax(att, dim=-1), self.attn_pdrop, self.training)
        y = (att @ v).transpose(1, 2).reshape(B, T, d)
        return F.dropout(self.c_proj(y), self.resid_pdrop, self.training), (k, v)


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.c_fc = Conv1D(cfg.ffn_dim, cfg.n_embd)
        self.c_proj = Conv1D(cfg.n_embd, cfg.ffn_dim)
        self.resid_pdrop = cfg.resid_pdrop

    def forward(self, x):
        return F.dropout(self.c_proj(gelu_new(self.c_fc(x))), self.resid_pdrop, self.training)


class ExpertBank(nn.Module):
    """Weights of all experts of one layer, stacked on a leading expert dimension."""

    def __init__(self, n_experts: int, nx: int, nf: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_experts, nx, nf))
        self.bias = nn.Parameter(torch.zeros(n_experts, nf))
        nn.init.normal_(self.weight, std=0.02)


class MoEMLP(nn.Module):
    """Top-k softmax-routed mixture of GELU MLP experts (dense reference: every expert is applied
    to every token and masked by the gate, no capacity limit).  ``aux_loss`` is the load-balance
    term  E * sum_e f_e * P_e  (f_e: fraction of routed assignments, P_e: mean router probability)."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        E, d = cfg.num_experts, cfg.n_embd
        Fe = cfg.moe_ffn or cfg.ffn_dim
        self.top_k = cfg.moe_top_k
        self.router = nn.Linear(d, E, bias=False)
        nn.init.normal_(self.router.weight, std=0.02)
        assert E % cfg.ep_world == 0
        n_local = E // cfg.ep_world          # all experts unless built for one expert-parallel rank
        self.c_fc = ExpertBank(n_local, d, Fe)
        self.c_proj = ExpertBank(n_local, Fe, d)
        self.resid_pdrop = cfg.resid_pdrop
        self.aux_loss: torch.Tensor | None = None

    def route(self, x2: torch.Tensor):
        probs = F.softmax(self.router(x2).float(), dim=-1)
        topv, topi = probs.topk(self.top_k, dim=-1)
        gates = topv / topv.sum(-1, keepdim=True)
        E = probs.size(-1)
        frac = F.one_hot(topi, E).float().sum(1).mean(0) / self.top_k
        aux = E * (frac * probs.mean(0)).sum()
        return gates, topi, aux

    def forward(self, x):
        B, T, d = x.shape
        x2 = x.reshape(-1, d)
        gates, topi, self.aux_loss = self.route(x2)
        E = self.router.out_features
        dense_gate = torch.zeros(x2.size(0), E, dtype=x.dtype, device=x.device)
        dense_gate.scatter_(1, topi, gates.to(x.dtype))
        h = torch.einsum("nd,edf->enf", x2, self.c_fc.weight) + self.c_fc.bias[:, None, :]
        y = torch.einsum("enf,efd->end", gelu_new(h), self.c_proj.weight) + self.c_proj.bias[:, None, :]
        out = (y * dense_gate.t().unsqueeze(-1)).sum(0)
        return F.dropout(out.view(B, T, d), self.resid_pdrop, self.training)


class Block(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        self.ln_1 = make_norm(cfg)
        self.attn = Attention(cfg)
        self.ln_2 = make_norm(cfg)
        self.mlp = MoEMLP(cfg) if cfg.is_moe_layer(layer_idx) else MLP(cfg)

    def forward(self, x, key_mask=None, past=None):
        a, present = self.attn(self.ln_1(x), key_mask, past)
        x = x + a
        return x + self.mlp(self.ln_2(x)), present


class Transformer(nn.Module):
    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.wte = nn.Embedding(cfg.vocab_size, cfg.n_embd)
        self.wpe = nn.Embedding(cfg.n_positions, cfg.n_embd)
        self.h = nn.ModuleList([Block(cfg, i) for i in range(cfg.n_layer)])
        self.ln_f = make_norm(cfg)
        self.embd_pdrop = cfg.embd_pdrop


class GPT2LM(nn.Module):
    """Decoder with tied LM head.  ``forward`` accepts ``input_ids`` or ``inputs_embeds``."""

    def __init__(self, cfg: ModelConfig):
        super().__init__()
        self.config = cfg
        self.transformer = Transformer(cfg)
        self.lm_head = nn.Linear(cfg.n_embd, cfg.vocab_size, bias=False)
        self.lm_head.weight = self.transformer.wte.weight  # tied
        self.reset_parameters()

    def reset_parameters(self) -> None:
        cfg = self.config
        std = cfg.initializer_range
        for name, p in self.named_parameters():
            if name.endswith("bias"):
                nn.init.zeros_(p)
            elif "ln_" in name:
                nn.init.ones_(p)
            elif name.endswith("c_proj.weight"):
                nn.init.normal_(p, std=std / math.sqrt(2 * cfg.n_layer))
            else:
                nn.init.normal_(p, std=std)

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, position_ids=None,
                labels=None, output_hidden_states: bool = True, past_key_values=None,
                use_cache: bool = False, **_: Any) -> dict:
        tr = self.transformer
        if inputs_embeds is None:
            inputs_embeds = tr.wte(input_ids)
        B, T, _d = inputs_embeds.shape
        past_len = 0 if past_key_values is None else past_key_values[0][0].size(2)
        if position_ids is None:
            position_ids = torch.arange(past_len, past_len + T, device=inputs_embeds.device)[None].expand(B, T)
        x = F.dropout(inputs_embeds + tr.wpe(position_ids), tr.embd_pdrop, self.training)
        # like the reference stack, padding only matters for batched evaluation
        key_mask = attention_mask if (attention_mask is not None and not self.training and B > 1) else None
        presents = []
        aux = None
        for i, blk in enumerate(tr.h):
            x, present = blk(x, key_mask, None if past_key_values is None else past_key_values[i])
            if use_cache:
                presents.append(present)
            if isinstance(blk.mlp, MoEMLP) and blk.mlp.aux_loss is not None:
                aux = blk.mlp.aux_loss if aux is None else aux + blk.mlp.aux_loss
        h = tr.ln_f(x)
        logits = self.lm_head(h)
        out = {"logits": logits, "hidden_states": (h,)}
        if use_cache:
            out["past_key_values"] = presents
        if aux is not None:
            out["aux_loss"] = aux
        if labels is not None:
            out["loss"] = F.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)).float(),
                                          labels[:, 1:].reshape(-1), ignore_index=IGNORE)
        return out


class CausalLMWithControlToken(nn.Module):
    def __init__(self, model: GPT2LM):
        super().__init__()
        self.config = model.config
        self.model = model
        self.vocab_size = model.transformer.wte.num_embeddings
        self.control_embeds = nn.Embedding(2, model.config.n_embd)
        self.control_embeds.weight.data.normal_(mean=0.0, std=0.02)
        self.elo_min, self.elo_max = 500, 3000

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        is_elo = (input_ids >= self.vocab_size).unsqueeze(-1)
        e = ((input_ids - self.vocab_size).clamp(self.elo_min, self.elo_max) - self.elo_min) / (
            self.elo_max - self.elo_min)
        ctrl = torch.stack((e, 1 - e), dim=2).to(self.control_embeds.weight.dtype) @ self.control_embeds.weight
        tok = self.model.transformer.wte(input_ids.clamp(0, self.vocab_size - 1))
        return torch.where(is_elo, ctrl, tok)

    def forward(self, input_ids, attention_mask=None, output_hidden_states: bool = True, **kwargs):
        return self.model(inputs_embeds=self.embed(input_ids), attention_mask=attention_mask,
                          output_hidden_states=output_hidden_states, **kwargs)


def masked_mse(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """Mean squared error over entries whose target is not -100 (0 when none is valid)."""
    target = target.to(device=pred.device, dtype=pred.dtype)
    se = (pred - target) ** 2
    valid = target != IGNORE
    if not bool(valid.any()):
        return (se * 0.0).mean()
    return se[valid].mean()


class CausalLMWithRegressionHead(nn.Module):
    def __init__(self, model: nn.Module, lm_loss_coef: float = 1.0, value_loss_coef: float = 1.0,
                 time_loss_coef: float = 1.0, aux_loss_coef: float | None = None):
        super().__init__()
        self.config = model.config
        self.model = model
        d = model.config.n_embd
        self.value_head = nn.Sequential(nn.Linear(d, 1), nn.Flatten(start_dim=1), nn.Tanh())
        self.time_head = nn.Sequential(nn.Linear(d, 1), nn.Flatten(start_dim=1))
        self.lm_loss_coef = lm_loss_coef
        self.value_loss_coef = value_loss_coef
        self.time_loss_coef = time_loss_coef  # stored, unused: see module docstring
        self.aux_loss_coef = model.config.aux_loss_coef if aux_loss_coef is None else aux_loss_coef

    def forward(self, input_ids, attention_mask=None, value_labels=None, time_labels=None,
                output_hidden_states: bool = True, **kwargs) -> dict:
        assert output_hidden_states
        out = dict(self.model(input_ids=input_ids, attention_mask=attention_mask,
                              output_hidden_states=True, **kwargs))
        h = out["hidden_states"][-1]
        out["value_logits"] = self.value_head(h)
        out["time_logits"] = self.time_head(h)
        if value_labels is not None:
            out["value_loss"] = masked_mse(out["value_logits"], value_labels)
        if time_labels is not None:
            out["time_loss"] = masked_mse(out["time_logits"], time_labels)
        loss = torch.zeros((), dtype=torch.float, device=h.device)
        if "loss" in out:
            out["lm_loss"] = out["loss"]
            loss = loss + out["lm_loss"] * self.lm_loss_coef
        if "value_loss" in out:
            loss = loss + out["value_loss"] * self.value_loss_coef
        if "time_loss" in out:
            loss = loss + out["time_loss"] * self.value_loss_coef
        if "aux_loss" in out and ("lm_loss" in out):
            loss = loss + out["aux_loss"] * self.aux_loss_coef
        out["loss"] = loss
        return out
