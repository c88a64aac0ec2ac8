"""Throughput bookkeeping for the trainer log: model FLOPs per token and model-FLOPs utilisation.

The reference logs only the wall time per ``log_interval`` (``src/modeling/trainer.py:291-298``);
this adds tokens/s, the step time as the maximum over ranks and MFU against the dense bf16 peak of
the device (B200: 2.25e15 FLOP/s nominal; a measured peak can be passed instead).
"""
from __future__ import annotations

B200_BF16_DENSE_FLOPS = 2.25e15


def matmul_params_per_token(cfg) -> float:
    """Weights a token passes through in matrix products: attention projections and FFN of every
    block (top-k experts plus the router in MoE blocks), and the tied output projection."""
    d, L, V = cfg.n_embd, cfg.n_layer, cfg.vocab_size
    attn = 4 * d * d
    dense_ffn = 2 * d * cfg.ffn_dim
    total = 0.0
    for i in range(L):
        if cfg.is_moe_layer(i):
            f = cfg.moe_ffn if cfg.moe_ffn is not None else cfg.ffn_dim
            total += attn + cfg.moe_top_k * 2 * d * f + d * cfg.num_experts
        else:
            total += attn + dense_ffn
    return total + d * V


def train_flops_per_token(cfg, seq_len: int) -> float:
    """Forward + backward FLOPs per token: 6 per matrix-product weight, plus causal attention
    (QK^T and PV: 2 * 2 * T/2 * d per layer forward, times three for forward + backward)."""
    attention = cfg.n_layer * 3 * 2 * seq_len * cfg.n_embd
    return 6.0 * matmul_params_per_token(cfg) + attention


def mfu(tokens_per_s: float, flops_per_token: float, n_gpus: int = 1,
        peak_flops: float = B200_BF16_DENSE_FLOPS) -> float:
    return tokens_per_s * flops_per_token / (n_gpus * peak_flops)
