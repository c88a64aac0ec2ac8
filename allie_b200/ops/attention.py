"""Causal self-attention over the packed QKV activation.

``qkv`` is the [B*T, 3*d] bf16 output of the QKV GEMM (q | k | v, head h in columns
h*hd .. (h+1)*hd of each third); ``out`` is [B*T, d] bf16 in the layout the output projection GEMM
reads.  ``lse`` [B, H, T] keeps the log-sum-exp of each row for the backward pass.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_uint, c_ulonglong

from . import _lib
from ._lib import ptr, stream_ptr


def attention_fwd(qkv, out, lse, B: int, T: int, H: int, hd: int, p_drop: float, seed: int,
                  stream_id: int, drop_mask=None) -> None:
    """``drop_mask``: optional int32 [B, H, T, T//32] that receives the dropout keep bits so the
    backward pass can read them back instead of re-running the generator."""
    rc = _lib.cuda().ab_attn_fwd(ptr(qkv), ptr(out), ptr(lse), ptr(drop_mask), c_int(B), c_int(T), c_int(H), c_int(hd),
                                 c_float(1.0 / hd ** 0.5), c_ulonglong(seed), c_uint(stream_id),
                                 c_uint(_lib.dropout_thr16(p_drop)), ptr(_lib.status_word()),
                                 stream_ptr())
    if rc != 0:
        raise RuntimeError(f"ab_attn_fwd failed with code {rc} (B={B} T={T} H={H} hd={hd})")
    _lib.count_launches(1)


def attention_bwd(qkv, out, lse, dout, dqkv, delta, B: int, T: int, H: int, hd: int, p_drop: float,
                  seed: int, stream_id: int, drop_mask=None, dq_acc=None) -> None:
    """``delta`` is fp32 scratch [B, H, T] (row sums of dO*O, filled here).  ``dq_acc``: optional
    all-zero fp32 [B*T, H*hd] accumulator (head_dim 64 only) that selects the single-kernel
    backward; it is handed back all zero."""
    rc = _lib.cuda().ab_attn_bwd(ptr(qkv), ptr(out), ptr(lse), ptr(dout), ptr(dqkv), ptr(delta),
                                 ptr(drop_mask), ptr(dq_acc), c_int(B), c_int(T),
                                 c_int(H), c_int(hd), c_float(1.0 / hd ** 0.5), c_ulonglong(seed),
                                 c_uint(stream_id), c_uint(_lib.dropout_thr16(p_drop)),
                                 ptr(_lib.status_word()), stream_ptr())
    if rc != 0:
        raise RuntimeError(f"ab_attn_bwd failed with code {rc} (B={B} T={T} H={H} hd={hd})")
    _lib.count_launches(3)  # delta + (two backward kernels | fused backward + dQ conversion)


def set_backward_schedule(mode: int) -> None:
    """Schedule of the single-kernel head_dim-64 backward: 0 = chosen from the problem shape
    (persistent walk when there are at least four (batch, head) slices per SM), 1 = one key tile
    per CTA, 2 = persistent walk over (batch, head) slices."""
    rc = _lib.cuda().ab_attn_bwd_schedule(c_int(mode))
    if rc != 0:
        raise ValueError(f"bad attention backward schedule {mode}")
