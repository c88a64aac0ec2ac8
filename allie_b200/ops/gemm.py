"""Python entry to the tcgen05 GEMM (``csrc/gemm_tc.cu``).

``gemm(a, b, a_mn=..., b_mn=..., ...)`` computes ``C[M,N] = A[M,K] @ B[K,N]``
where each operand may be given K-major or MN-major in memory:

=========  ======================  ==========================
flag       tensor passed           meaning
=========  ======================  ==========================
a_mn=False ``a`` of shape [M, K]   A as is
a_mn=True  ``a`` of shape [K, M]   A = a.T
b_mn=False ``b`` of shape [N, K]   B = b.T   (nn.Linear weight layout)
b_mn=True  ``b`` of shape [K, N]   B as is   (GPT-2 Conv1D weight layout)
=========  ======================  ==========================
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong

import torch

from . import _lib

_NUM_SMS: dict[int, int] = {}


def num_sms() -> int:
    dev = torch.cuda.current_device()
    if dev not in _NUM_SMS:
        _NUM_SMS[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _NUM_SMS[dev]


def pick_k_splits(M: int, N: int, K: int) -> int:
    """Split K when the output alone has too few 128x256 tiles to fill the GPU
    (the weight-gradient case: small output, very long contraction)."""
    bn = 128 if N <= 128 else 256
    tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
    sms = num_sms()
    if tiles >= 4 * sms:
        return 1
    kb = (K + 63) // 64
    best, best_eff = 1, 0.0
    for s in (1, 2, 3, 4, 6, 8, 12, 16, 24, 32):
        if kb // s < 8:
            break
        units = tiles * s
        waves = (units + sms - 1) // sms
        eff = units / (waves * sms)
        # prefer fewer splits on near-ties: each split re-reads/atomically adds C
        if eff > best_eff + 0.04:
            best, best_eff = s, eff
    return best


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False, bias: torch.Tensor | None = None, act: int = 0,
         aux: torch.Tensor | None = None, resid: torch.Tensor | None = None,
         drop_p: float = 0.0, drop_seed: int = 0, drop_stream: int = 0,
         alpha: float = 1.0, k_splits: int | None = None, m_limit: torch.Tensor | None = None,
         k_limit: torch.Tensor | None = None, dependent: bool = False,
         aux_grad: bool = False) -> torch.Tensor:
    """``dependent``: launch as a programmatic dependent of the previous kernel in the stream
    (honoured by the small-M kernel): its set-up and first weight tiles overlap that kernel.  ``b``
    must then be data the previous kernel does not write (weights).
    ``aux_grad``: with ``act=1`` store GELU'(pre-activation) in ``aux`` instead of the
    pre-activation, with ``act=2`` multiply by ``aux`` as it is: the derivative is computed once,
    beside the activation it shares its tanh with, and the backward epilogue (bound by instruction
    issue) shrinks to a multiply."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        assert not accumulate
    assert out.shape == (M, N) and out.stride(1) == 1
    assert out.dtype in (torch.bfloat16, torch.float32)
    out_fp32 = out.dtype == torch.float32
    if accumulate:
        assert out_fp32
    if (k_splits is None and resid is not None and resid.data_ptr() == out.data_ptr() and drop_p == 0.0
            and act == 0 and M <= 512 and m_limit is None and k_limit is None):
        # Skinny in-place residual update (decode steps): x += a @ b + bias.  A few output tiles
        # with a long K loop leave most SMs idle, so the contraction is split over more CTAs and
        # the partial products are reduce-added into x; the first split adds the bias.
        tiles = -(-M // 128) * -(-N // 128)
        ks = max(1, min(K // 256, 128 // max(tiles, 1)))
        if ks > 1:
            accumulate, resid, k_splits = True, None, ks
    if k_splits is None:
        k_splits = pick_k_splits(M, N, K) if (accumulate and out_fp32) else 1
    ep = _lib.GemmEpilogue()
    ep.out = out.data_ptr()
    ep.ldo = out.stride(0)
    ep.out_fp32 = int(out_fp32)
    ep.accumulate = int(accumulate)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
        ep.bias = bias.data_ptr()
    ep.act = act            # 1: GELU, pre-activation saved in aux; 2: times GELU'(aux); 3: GELU, nothing saved
    if act in (1, 2):
        assert aux is not None and aux.dtype == torch.bfloat16 and aux.shape == (M, N)
        ep.aux = aux.data_ptr()
        ep.ldaux = aux.stride(0)
    if resid is not None:
        assert resid.dtype == torch.float32 and resid.shape == (M, N) and out_fp32
        ep.resid = resid.data_ptr()
        ep.ldr = resid.stride(0)
        ep.drop_seed = drop_seed
        ep.drop_stream = drop_stream
        ep.drop_thr16 = _lib.dropout_thr16(drop_p)
    ep.alpha = alpha
    if m_limit is not None:      # int32 device scalar: rows actually present
        ep.m_limit = m_limit.data_ptr()
    if k_limit is not None:      # int32 device scalar: contraction length actually present
        ep.k_limit = k_limit.data_ptr()
    ep.pdl = int(dependent)
    ep.aux_grad = int(aux_grad)
    rc = _lib.cuda().ab_gemm_bf16(
        _lib.ptr(a), c_int(int(a_mn)), c_longlong(a.stride(0)),
        _lib.ptr(b), c_int(int(b_mn)), c_longlong(b.stride(0)),
        c_int(M), c_int(N), c_int(K), ctypes.byref(ep), c_int(k_splits), c_int(num_sms()),
        _lib.ptr(_lib.status_word()), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"ab_gemm_bf16 failed with code {rc} for M={M} N={N} K={K}")
    _lib.count_launches(1)
    return out


def gemm_grouped(a: torch.Tensor, b: torch.Tensor, rows: torch.Tensor, cap: int, *, mode: int, b_mn: bool = True,
                 out: torch.Tensor | None = None, bias: torch.Tensor | None = None, act: int = 0,
                 aux: torch.Tensor | None = None, tile_ready: torch.Tensor | None = None,
                 scatter: dict | None = None, aux_grad: bool = False) -> None:
    """One launch of the grouped CTA-pair GEMM (``csrc/gemm_grouped.cu``) over all local experts.

    ``rows`` (int32 [G], device): live rows per group; ``cap``: rows reserved per group.
    mode 1: ``a`` [G*cap, K] bf16, ``b`` [G, K, N] (``b_mn``) or [G, N, K]; ``out`` / ``aux`` [G*cap, N] bf16,
            ``bias`` [G, N] fp32, ``act`` as in :func:`gemm`.
    mode 2: ``a`` [G*cap, M] bf16, ``b`` [G*cap, N] bf16; ``out`` [G, M, N] fp32, accumulated with
            ``a[g]^T @ b[g]`` over each group's live rows (rounded up to 128).
    ``tile_ready`` (uint32 / int32 [G*cap/128]): arrival counters the producer waits on.
    ``scatter`` (mode 1): ``dict(ret=, peers=, flags=, phase=, epoch=, rank=, world=, ticket=)`` - rows
    leave to the peers' buffers from the epilogue instead of being written to ``out``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1
    G = rows.numel()
    assert rows.dtype == torch.int32 and a.shape[0] == G * cap and cap % 256 == 0
    ep = _lib.GemmEpilogue()
    grp = _lib.GroupedGemm()
    grp.groups, grp.cap, grp.mode = G, cap, mode
    grp.rows = rows.data_ptr()
    if tile_ready is not None:
        assert tile_ready.numel() >= G * cap // 128
        grp.tile_ready = tile_ready.data_ptr()
    ep.alpha = 1.0
    if mode == 1:
        K = a.shape[1]
        assert b.dim() == 3 and b.shape[0] == G and b.is_contiguous()
        N = b.shape[2] if b_mn else b.shape[1]
        assert (b.shape[1] if b_mn else b.shape[2]) == K
        M = cap
        ldb = b.shape[2]
        if scatter is not None:
            assert act == 0 and out is None
            grp.ret = scatter["ret"].data_ptr()
            for i in range(8):
                grp.peers[i] = scatter["peers"][i]
                grp.flags[i] = scatter["flags"][i]
            grp.phase, grp.epoch = scatter["phase"], scatter["epoch"]
            grp.rank, grp.world = scatter["rank"], scatter["world"]
            grp.ticket = scatter["ticket"]
        else:
            assert out is not None and out.dtype == torch.bfloat16 and out.shape == (G * cap, N) and out.stride(1) == 1
            ep.out, ep.ldo = out.data_ptr(), out.stride(0)
        if bias is not None:
            assert bias.dtype == torch.float32 and bias.numel() == G * N and bias.is_contiguous()
            ep.bias = bias.data_ptr()
        ep.act = act
        ep.aux_grad = int(aux_grad)
        if act:
            assert aux is not None and aux.dtype == torch.bfloat16 and aux.shape == (G * cap, N)
            ep.aux, ep.ldaux = aux.data_ptr(), aux.stride(0)
    else:
        assert mode == 2 and b.dim() == 2 and b.shape[0] == G * cap and b.stride(1) == 1 and b_mn
        M, N, K = a.shape[1], b.shape[1], cap
        ldb = b.stride(0)
        assert out is not None and out.dtype == torch.float32 and out.shape == (G, M, N) and out.is_contiguous()
        ep.out, ep.ldo, ep.out_fp32, ep.accumulate = out.data_ptr(), N, 1, 1
    rc = _lib.cuda().ab_gemm_grouped_bf16(
        _lib.ptr(a), c_longlong(a.stride(0)), _lib.ptr(b), c_int(int(b_mn)), c_longlong(ldb),
        c_int(M), c_int(N), c_int(K), ctypes.byref(ep), ctypes.byref(grp), c_int(num_sms()),
        _lib.ptr(_lib.status_word()), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"ab_gemm_grouped_bf16 failed with code {rc} (mode {mode}, G={G}, cap={cap}, M={M}, N={N}, K={K})")
    _lib.count_launches(1)
