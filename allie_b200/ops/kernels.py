"""Python entries to the non-GEMM sm_100a kernels (norms, embedding, loss heads, optimizer).

Every function launches on the current CUDA stream, allocates nothing unless an output argument is
omitted, and never synchronises with the host.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_uint, c_ulonglong

from . import _lib
from ._lib import ptr, stream_ptr


def _ck(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    _lib.count_launches(1)


# ------------------------------------------------------------------ norms ---
def layernorm_fwd(x, gamma, beta, y, mean, rstd, eps: float, rms: bool = False, dependent: bool = False) -> None:
    """``dependent``: launch as a programmatic dependent of the previous kernel in the stream (the
    launch overlaps that kernel's tail; the kernel waits for it before it reads ``x``)."""
    M, d = x.shape
    fn = _lib.cuda().ab_layernorm_fwd_dependent if dependent else _lib.cuda().ab_layernorm_fwd
    _ck(fn(ptr(x), ptr(gamma), ptr(beta), ptr(y), ptr(mean), ptr(rstd),
           c_int(M), c_int(d), c_float(eps), c_int(int(rms)), stream_ptr()), "ab_layernorm_fwd")


def layernorm_bwd(dy, x, mean, rstd, gamma, dres_in, dx, dbranch, dgamma, dbeta, *, s0=None, w0=None,
                  s1=None, w1=None, rms: bool = False, drop_seed: int = 0, drop_stream: int = 0,
                  drop_p: float = 0.0, dbias=None) -> None:
    """``dbias`` (optional, fp32 [d], accumulated): column sums of ``dbranch``, i.e. the bias gradient
    of the projection whose output gradient ``dbranch`` is; needs ``dgamma``."""
    M, d = x.shape
    _ck(_lib.cuda().ab_layernorm_bwd(
        ptr(dy), ptr(x), ptr(mean), ptr(rstd), ptr(gamma), ptr(dres_in), ptr(dx), ptr(dbranch),
        ptr(dgamma), ptr(dbeta), ptr(dbias), ptr(s0), ptr(w0), ptr(s1), ptr(w1), c_int(M), c_int(d),
        c_int(int(rms)), c_ulonglong(drop_seed), c_uint(drop_stream),
        c_uint(_lib.dropout_thr16(drop_p)), stream_ptr()), "ab_layernorm_bwd")


# -------------------------------------------------------------- embedding ---
def unpack_window(words, vocab: int, pad_id: int, time_mean: float, time_std: float, ids, pos,
                  lm_labels, value_labels, time_labels, counts) -> None:
    B, T = words.shape
    _ck(_lib.cuda().ab_unpack_window(ptr(words), c_int(B), c_int(T), c_int(vocab), c_int(pad_id),
                                     c_float(time_mean), c_float(time_std), ptr(ids), ptr(pos),
                                     ptr(lm_labels), ptr(value_labels), ptr(time_labels), ptr(counts),
                                     stream_ptr()), "ab_unpack_window")


def embed_fwd(ids, pos, wte, wpe, ctrl, x, vocab: int, drop_seed: int, drop_stream: int,
              drop_p: float) -> None:
    M, d = x.shape
    _ck(_lib.cuda().ab_embed_fwd(ptr(ids), ptr(pos), ptr(wte), ptr(wpe), ptr(ctrl), ptr(x), c_int(M),
                                 c_int(d), c_int(vocab), c_ulonglong(drop_seed), c_uint(drop_stream),
                                 c_uint(_lib.dropout_thr16(drop_p)), stream_ptr()), "ab_embed_fwd")


def embed_bwd(ids, pos, dx, dwte, dwpe, dctrl, vocab: int, drop_seed: int, drop_stream: int,
              drop_p: float) -> None:
    M, d = dx.shape
    _ck(_lib.cuda().ab_embed_bwd(ptr(ids), ptr(pos), ptr(dx), ptr(dwte), ptr(dwpe), ptr(dctrl),
                                 c_int(M), c_int(d), c_int(vocab), c_ulonglong(drop_seed),
                                 c_uint(drop_stream), c_uint(_lib.dropout_thr16(drop_p)),
                                 stream_ptr()), "ab_embed_bwd")


# ------------------------------------------------------------------ losses ---
def ce_fwd_bwd(logits, labels, n_valid, coef: float, loss_acc, write_grad: bool = True) -> None:
    M, V = logits.shape
    _ck(_lib.cuda().ab_ce_fwd_bwd(ptr(logits), ptr(labels), ptr(n_valid), c_float(coef), c_int(M),
                                  c_int(V), c_longlong(logits.stride(0)), ptr(loss_acc),
                                  c_int(int(write_grad)), stream_ptr()), "ab_ce_fwd_bwd")


def lmhead_ce(h, wte, labels, n_valid, coef: float, dlogits, loss_acc) -> None:
    """Fused output-embedding GEMM + cross entropy (``csrc/lmhead_ce.cu``): ``loss_acc[0]`` += the summed
    negative log likelihood of the labelled rows, ``dlogits`` [M, V] bf16 = d loss / d logits (mean over
    ``n_valid`` rows, times ``coef``); the logits are never stored."""
    from .gemm import num_sms

    M, K = h.shape
    V = wte.shape[0]
    assert h.dtype == wte.dtype == dlogits.dtype and dlogits.shape == (M, V) and wte.shape[1] == K
    _ck(_lib.cuda().ab_lmhead_ce(ptr(h), c_longlong(h.stride(0)), ptr(wte), c_longlong(wte.stride(0)), ptr(labels),
                                 ptr(n_valid), c_float(coef), ptr(dlogits), c_longlong(dlogits.stride(0)),
                                 ptr(loss_acc), c_int(M), c_int(V), c_int(K), c_int(num_sms()),
                                 ptr(_lib.status_word()), stream_ptr()), "ab_lmhead_ce")


def heads_fwd(h, wv, bv, wt, bt, value_labels, time_labels, counts, value_coef: float,
              time_coef: float, value_out, time_out, dv, dt, acc) -> None:
    M, d = h.shape
    _ck(_lib.cuda().ab_heads_fwd(ptr(h), ptr(wv), ptr(bv), ptr(wt), ptr(bt), ptr(value_labels),
                                 ptr(time_labels), ptr(counts), c_float(value_coef),
                                 c_float(time_coef), ptr(value_out), ptr(time_out), ptr(dv), ptr(dt),
                                 ptr(acc), c_int(M), c_int(d), stream_ptr()), "ab_heads_fwd")


def heads_bwd_w(h, dv, dt, dwv, dbv, dwt, dbt) -> None:
    M, d = h.shape
    _ck(_lib.cuda().ab_heads_bwd_w(ptr(h), ptr(dv), ptr(dt), ptr(dwv), ptr(dbv), ptr(dwt), ptr(dbt),
                                   c_int(M), c_int(d), stream_ptr()), "ab_heads_bwd_w")


def loss_finalize(acc, counts, lm_coef: float, value_coef: float, time_coef: float, out) -> None:
    _ck(_lib.cuda().ab_loss_finalize(ptr(acc), ptr(counts), c_float(lm_coef), c_float(value_coef),
                                     c_float(time_coef), ptr(out), stream_ptr()), "ab_loss_finalize")


# --------------------------------------------------------------- optimizer ---
def sumsq(g, out) -> None:
    _ck(_lib.cuda().ab_sumsq(ptr(g), c_longlong(g.numel()), ptr(out), stream_ptr()), "ab_sumsq")


def adamw(p, g, m, v, p_bf16, lr: float, beta1: float, beta2: float, eps: float, wd: float,
          step: int, gnorm_sq=None, max_norm: float = 0.0, grad_scale: float = 1.0) -> None:
    _ck(_lib.cuda().ab_adamw(ptr(p), ptr(g), ptr(m), ptr(v), ptr(p_bf16), c_longlong(p.numel()),
                             c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(wd),
                             c_int(step), ptr(gnorm_sq), c_float(max_norm), c_float(grad_scale),
                             stream_ptr()), "ab_adamw")


def cast_bf16(src, dst) -> None:
    _ck(_lib.cuda().ab_cast_bf16(ptr(src), ptr(dst), c_longlong(src.numel()), stream_ptr()),
        "ab_cast_bf16")


def colsum_bf16(x, out, m_limit=None) -> None:
    """out[n] += sum over rows of the bf16 matrix x (bias gradients); ``m_limit`` is an optional
    int32 device scalar limiting the rows that take part."""
    M, N = x.shape
    _ck(_lib.cuda().ab_colsum_bf16(ptr(x), c_longlong(x.stride(0)), c_int(M), c_int(N), ptr(out),
                                   ptr(m_limit), stream_ptr()), "ab_colsum_bf16")


def colsum_grouped_bf16(x, out, rows, cap: int) -> None:
    """Grouped form: ``x`` [G*cap, N] bf16, ``out`` [G, N] fp32 accumulated, ``rows`` int32 [G] = rows of
    every group that take part."""
    G = rows.numel()
    N = x.shape[1]
    assert x.shape[0] == G * cap and out.numel() == G * N
    _ck(_lib.cuda().ab_colsum_grouped_bf16(ptr(x), c_longlong(x.stride(0)), c_int(G), c_int(cap), c_int(N),
                                           ptr(out), ptr(rows), stream_ptr()), "ab_colsum_grouped_bf16")
