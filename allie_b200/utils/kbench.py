"""Kernel micro-benchmarks: one kernel, one shape, CUDA-event timing after warm-up, achieved
TFLOP/s or GB/s against the measured peaks of the machine (``MEASURED_PEAKS.json`` when present).

    python -m allie_b200.utils.kbench gemm --m 32768 --n 4096 --k 1024 [--epilogue bias|gelu|dgelu|resid|none] [--wgrad]
    python -m allie_b200.utils.kbench attn --batch 64 --seq 512 --heads 16 --hd 64 [--dropout 0.1] [--bwd]
    python -m allie_b200.utils.kbench layernorm --rows 32768 --d 1024 [--bwd]
    python -m allie_b200.utils.kbench adamw --n 300000000
    python -m allie_b200.utils.kbench colsum --rows 32768 --d 4096
    python -m allie_b200.utils.kbench lmhead_ce --m 32768 --n 2048 --k 1024
    python -m allie_b200.utils.kbench gemm_grouped --groups 8 --cap 8192 --live 4096 --n 4096 --k 2048 [--wgrad]
    python -m allie_b200.utils.kbench nvl --n 300000000      # gradient-path kernels with the rank as its own only peer
    python -m allie_b200.utils.kbench moe --rows 16384 --d 2048 --experts 8   # routing / dispatch / combine, one rank
    python -m allie_b200.utils.kbench decode_attn --batch 256 --heads 16 --hd 64 --seq 160

Also the workload to put under ``ncu`` (``--iters`` small).  Inputs are sized beyond the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def _peaks() -> dict:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        return json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


def main(argv=None) -> dict:
    from ..ops import _lib, kernels as K
    from ..ops.attention import attention_bwd, attention_fwd
    from ..ops.gemm import gemm

    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn", "layernorm", "adamw", "colsum", "lmhead_ce", "gemm_grouped",
                                       "nvl", "moe", "decode_attn"])
    ap.add_argument("--groups", type=int, default=8); ap.add_argument("--cap", type=int, default=8192)
    ap.add_argument("--live", type=int, default=4096); ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--m", type=int, default=32768); ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--epilogue", default="none", choices=["none", "bias", "gelu", "dgelu", "resid"])
    ap.add_argument("--aux-grad", action="store_true",
                    help="gelu / dgelu: the second tensor holds GELU'(pre-activation), as the training engine runs them")
    ap.add_argument("--wgrad", action="store_true")
    ap.add_argument("--batch", type=int, default=64); ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--heads", type=int, default=16); ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--dropout", type=float, default=0.0); ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--rows", type=int, default=32768); ap.add_argument("--d", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=20); ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)
    dev, peaks = "cuda", _peaks()
    out: dict = {"kernel": a.kernel}
    if a.kernel == "gemm":
        M, N, Kd = a.m, a.n, a.k
        if a.wgrad:      # dW[M,N] += X^T[M,K] dY[K,N], both operands MN-major, fp32 reduce-add epilogue
            x = torch.randn(Kd, M, device=dev).bfloat16(); dy = torch.randn(Kd, N, device=dev).bfloat16()
            dw = torch.zeros(M, N, device=dev)
            fn = lambda: gemm(x, dy, a_mn=True, b_mn=True, out=dw, accumulate=True)
        else:
            x = torch.randn(M, Kd, device=dev).bfloat16(); w = (torch.randn(Kd, N, device=dev) * 0.02).bfloat16()
            bias = torch.randn(N, device=dev)
            if a.epilogue == "resid":
                res = torch.randn(M, N, device=dev)
                fn = lambda: gemm(x, w, b_mn=True, bias=bias, resid=res, out=res, drop_p=0.1, drop_seed=1, drop_stream=1)
            elif a.epilogue == "gelu":
                o = torch.empty(M, N, device=dev, dtype=torch.bfloat16); pre = torch.empty_like(o)
                fn = lambda: gemm(x, w, b_mn=True, bias=bias, act=1, aux=pre, out=o, aux_grad=a.aux_grad)
            elif a.epilogue == "dgelu":   # dgrad through GELU: out = (x @ w) * gelu'(saved pre-activation)
                o = torch.empty(M, N, device=dev, dtype=torch.bfloat16); pre = torch.randn(M, N, device=dev).bfloat16()
                fn = lambda: gemm(x, w, b_mn=True, act=2, aux=pre, out=o, aux_grad=a.aux_grad)
            else:
                o = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
                fn = lambda: gemm(x, w, b_mn=True, bias=bias if a.epilogue == "bias" else None, out=o)
        s = _time(fn, a.iters, a.warmup)
        tf = 2.0 * M * N * Kd / s / 1e12
        out.update(shape=[M, N, Kd], seconds=s, tflops=tf, frac_of_measured_bf16=tf / peaks["bf16_tflops"])
    elif a.kernel == "attn":
        B, T, H, hd = a.batch, a.seq, a.heads, a.hd
        d = H * hd
        qkv = (torch.randn(B * T, 3 * d, device=dev) * 0.5).bfloat16()
        o = torch.zeros(B * T, d, device=dev, dtype=torch.bfloat16); lse = torch.zeros(B, H, T, device=dev)
        bits = torch.zeros(B, H, T, max(T // 32, 1), device=dev, dtype=torch.int32) if T % 32 == 0 else None
        attention_fwd(qkv, o, lse, B, T, H, hd, a.dropout, 1, 2, bits)
        if a.bwd:
            do = torch.randn(B * T, d, device=dev).bfloat16(); dq = torch.zeros_like(qkv)
            delta = torch.zeros(B, H, T, device=dev)
            acc = torch.zeros(B * T, d, device=dev) if hd == 64 else None
            fn = lambda: attention_bwd(qkv, o, lse, do, dq, delta, B, T, H, hd, a.dropout, 1, 2, bits, acc)
            flops = 5 * 2.0 * B * H * T * T * hd / 2
        else:
            fn = lambda: attention_fwd(qkv, o, lse, B, T, H, hd, a.dropout, 1, 2, bits)
            flops = 2 * 2.0 * B * H * T * T * hd / 2
        s = _time(fn, a.iters, a.warmup)
        out.update(shape=[B, T, H, hd], seconds=s, causal_tflops=flops / s / 1e12)
    elif a.kernel == "layernorm":
        M, d = a.rows, a.d
        x = torch.randn(M, d, device=dev); g = torch.ones(d, device=dev); b = torch.zeros(d, device=dev)
        y = torch.empty(M, d, device=dev, dtype=torch.bfloat16); mean = torch.empty(M, device=dev); rstd = torch.empty(M, device=dev)
        K.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
        if a.bwd:
            dy = torch.randn(M, d, device=dev).bfloat16(); dx = torch.randn(M, d, device=dev); dyb = torch.empty_like(dy)
            dg = torch.zeros(d, device=dev); db = torch.zeros(d, device=dev)
            fn = lambda: K.layernorm_bwd(dy, x, mean, rstd, g, dx, dx, dyb, dg, db, drop_p=0.1, drop_seed=1, drop_stream=1)
            nbytes = M * d * (2 + 4 + 4 + 4 + 2)      # dy, x, residual gradient in; dx, masked bf16 copy out
        else:
            fn = lambda: K.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
            nbytes = M * d * 6
        s = _time(fn, a.iters, a.warmup)
        out.update(shape=[M, d], seconds=s, gbs=nbytes / s / 1e9, frac_of_measured_hbm=nbytes / s / 1e9 / peaks["hbm_gbs"])
    elif a.kernel == "colsum":
        M, d = a.rows, a.d
        x = torch.randn(M, d, device=dev).bfloat16(); o = torch.zeros(d, device=dev)
        fn = lambda: K.colsum_bf16(x, o)
        s = _time(fn, a.iters, a.warmup)
        nbytes = M * d * 2
        out.update(shape=[M, d], seconds=s, gbs=nbytes / s / 1e9, frac_of_measured_hbm=nbytes / s / 1e9 / peaks["hbm_gbs"])
    elif a.kernel == "lmhead_ce":
        M, V, Kd = a.m, a.n, a.k
        h = torch.randn(M, Kd, device=dev).bfloat16(); wte = (torch.randn(V, Kd, device=dev) * 0.05).bfloat16()
        labels = torch.randint(0, V, (M,), device=dev, dtype=torch.int32)
        nval = torch.tensor([M], device=dev, dtype=torch.int32)
        dl = torch.empty(M, V, device=dev, dtype=torch.bfloat16); loss = torch.zeros(1, device=dev)
        fn = lambda: K.lmhead_ce(h, wte, labels, nval, 1.0, dl, loss)
        s = _time(fn, a.iters, a.warmup)
        tf = 2 * 2.0 * M * V * Kd / s / 1e12          # two sweeps of the GEMM
        out.update(shape=[M, V, Kd], seconds=s, tflops_two_sweeps=tf, frac_of_measured_bf16=tf / peaks["bf16_tflops"])
    elif a.kernel == "gemm_grouped":
        from ..ops.gemm import gemm_grouped

        G, cap, N, Kd, live = a.groups, a.cap, a.n, a.k, a.live
        rows = torch.full((G,), live, device=dev, dtype=torch.int32)
        if a.wgrad:       # dW[g] += X[g]^T dY[g] over the live rows
            x = torch.randn(G * cap, Kd, device=dev).bfloat16(); dy = torch.randn(G * cap, N, device=dev).bfloat16()
            dw = torch.zeros(G, Kd, N, device=dev)
            fn = lambda: gemm_grouped(x, dy, rows, cap, mode=2, out=dw)
        else:
            x = torch.randn(G * cap, Kd, device=dev).bfloat16(); w = (torch.randn(G, Kd, N, device=dev) * 0.02).bfloat16()
            bias = torch.randn(G, N, device=dev)
            o = torch.empty(G * cap, N, device=dev, dtype=torch.bfloat16); pre = torch.empty_like(o)
            fn = lambda: gemm_grouped(x, w, rows, cap, mode=1, b_mn=True, out=o, bias=bias, act=1, aux=pre)
        s = _time(fn, a.iters, a.warmup)
        tf = 2.0 * G * live * N * Kd / s / 1e12
        out.update(shape=[G, cap, live, N, Kd], seconds=s, tflops=tf, frac_of_measured_bf16=tf / peaks["bf16_tflops"])
    elif a.kernel == "nvl":
        # the two kernels of the fused data-parallel gradient path on ONE rank (world 1: the rank is
        # its own peer, flags and arenas are plain local tensors): what they cost as memory passes
        import ctypes
        from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

        n = a.n if a.n > 1 << 20 else 300_000_000
        n -= n % 64
        lib = _lib.cuda()
        grad = torch.randn(n, device=dev); master = torch.randn(n, device=dev); shadow = torch.empty(n, device=dev, dtype=torch.bfloat16)
        m1 = torch.zeros(n, device=dev); m2 = torch.zeros(n, device=dev)
        flags = torch.zeros(lib.ab_nvl_flag_words(), device=dev, dtype=torch.int32)
        norm = torch.zeros(8, device=dev); ticket = torch.zeros(4, device=dev, dtype=torch.int32)
        arr = lambda t: (c_void_p * 8)(t.data_ptr(), *([None] * 7))
        st = _lib.status_word()
        ll = c_longlong * 32
        z = [0] * 31
        epoch = [0]

        def rs():
            epoch[0] += 1
            assert lib.ab_nvl_reduce_scatter(arr(grad), arr(flags), c_void_p(0), _lib.ptr(norm), _lib.ptr(ticket), c_longlong(0),
                                             c_longlong(n), c_int(0), c_int(1), c_uint(epoch[0]), c_int(0), c_int(1),
                                             c_int(148 * 4), _lib.ptr(st), _lib.stream_ptr()) == 0

        def ag():
            assert lib.ab_nvl_adamw_allgather(arr(master), arr(shadow), arr(flags), arr(norm), c_void_p(0), c_void_p(0),
                                              _lib.ptr(grad), _lib.ptr(m1), _lib.ptr(m2), c_void_p(ticket.data_ptr() + 4),
                                              c_int(1), ll(0, *z), ll(n, *z), ll(n, *z), ll(n, *z), ll(0, *z), c_int(0),
                                              c_int(1), c_uint(epoch[0]), c_float(1e-3), c_float(0.9), c_float(0.95),
                                              c_float(1e-8), c_float(0.01), c_int(10), c_float(1.0), c_float(1.0),
                                              c_void_p(0), _lib.ptr(st), _lib.stream_ptr()) == 0

        s_rs = _time(rs, a.iters, a.warmup)
        s_ag = _time(lambda: (rs(), ag()), a.iters, a.warmup) - s_rs
        out.update(n=n, reduce_scatter_seconds=s_rs, reduce_scatter_gbs=n * 8 / s_rs / 1e9,
                   adamw_allgather_seconds=s_ag, adamw_allgather_gbs=n * 30 / s_ag / 1e9,
                   frac_of_measured_hbm=[n * 8 / s_rs / 1e9 / peaks["hbm_gbs"], n * 30 / s_ag / 1e9 / peaks["hbm_gbs"]])
    elif a.kernel == "moe":
        # one MoE layer forward + backward on one rank (the rank is its own peer): the routing /
        # dispatch / combine kernels and the grouped expert GEMMs in their real sequence
        from ..config import ModelConfig
        from ..data import UCITokenizer
        from ..models import initialize_model
        from ..models.engine import B200Engine

        T = 512
        B = max(1, a.rows // T)
        tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
        model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1, n_embd=a.d,
                                 n_head=a.d // 128, n_positions=T, num_experts=a.experts, moe_ffn=2 * a.d,
                                 moe_layer_freq=1, capacity_factor=2.0)
        eng = B200Engine(model, dev)
        w = torch.randint(0, 1968, (B, T), device=dev, dtype=torch.int32) | (5 << 16)

        def fn():
            eng.micro_step(w)
            eng.zero_grad()

        s = _time(fn, a.iters, a.warmup)
        out.update(shape=[B * T, a.d, a.experts], seconds_per_micro_step=s, moe=eng.moe_stats())
    elif a.kernel == "decode_attn":
        import ctypes
        from ctypes import c_float, c_int

        n, H, hd, P = a.batch, a.heads, a.hd, a.seq
        d, S = H * hd, P + 64
        qkv = (torch.randn(n, 3 * d, device=dev) * 0.5).bfloat16()
        kc = (torch.randn(n, H, S, hd, device=dev) * 0.5).bfloat16(); vc = (torch.randn(n, H, S, hd, device=dev) * 0.5).bfloat16()
        i32 = dict(device=dev, dtype=torch.int32)
        active = torch.ones(n, **i32); slot = torch.full((n,), P + 8, **i32); plen = torch.full((n,), P, **i32)
        anc = (torch.arange(128, **i32)[None, :] % 8 + P).repeat(n, 1).contiguous(); n_anc = torch.full((n,), 8, **i32)
        att = torch.empty(n, d, device=dev, dtype=torch.bfloat16)
        lib = _lib.cuda()
        fn = lambda: lib.ab_decode_attn(_lib.ptr(qkv), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(active), _lib.ptr(slot),
                                        _lib.ptr(plen), _lib.ptr(anc), c_int(128), _lib.ptr(n_anc), _lib.ptr(att), c_int(n),
                                        c_int(H), c_int(hd), c_int(S), c_float(hd ** -0.5), c_int(0),
                                        _lib.ptr(_lib.status_word()), _lib.stream_ptr())
        s = _time(fn, a.iters, a.warmup)
        nbytes = n * H * (P + 8) * hd * 2 * 2
        out.update(shape=[n, H, hd, P], seconds=s, gbs=nbytes / s / 1e9, frac_of_measured_hbm=nbytes / s / 1e9 / peaks["hbm_gbs"])
    else:
        n = a.n if a.n > 1 << 20 else 300_000_000
        n -= n % 4
        p = torch.randn(n, device=dev); g = torch.randn(n, device=dev); m = torch.zeros(n, device=dev); v = torch.zeros(n, device=dev)
        sh = torch.empty(n, device=dev, dtype=torch.bfloat16)
        fn = lambda: K.adamw(p, g, m, v, sh, 1e-3, 0.9, 0.95, 1e-8, 0.01, 10)
        s = _time(fn, a.iters, a.warmup)
        nbytes = n * (4 * 4 + 3 * 4 + 2)
        out.update(n=n, seconds=s, gbs=nbytes / s / 1e9, frac_of_measured_hbm=nbytes / s / 1e9 / peaks["hbm_gbs"])
    torch.cuda.synchronize()
    _lib.check_status()
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
