"""Kernel micro-benchmarks: one kernel, one shape, CUDA-event timing after warm-up, achieved
TFLOP/s or GB/s against the measured peaks of the machine (``MEASURED_PEAKS.json`` when present).

    python -m allie_b200.utils.kbench gemm --m 32768 --n 4096 --k 1024 [--epilogue bias|gelu|dgelu|resid|none] [--wgrad]
    python -m allie_b200.utils.kbench attn --batch 64 --seq 512 --heads 16 --hd 64 [--dropout 0.1] [--bwd]
    python -m allie_b200.utils.kbench layernorm --rows 32768 --d 1024 [--bwd]
    python -m allie_b200.utils.kbench adamw --n 300000000
    python -m allie_b200.utils.kbench colsum --rows 32768 --d 4096

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
    ap.add_argument("kernel", choices=["gemm", "attn", "layernorm", "adamw", "colsum"])
    ap.add_argument("--m", type=int, default=32768); ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--epilogue", default="none", choices=["none", "bias", "gelu", "dgelu", "resid"])
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
                fn = lambda: gemm(x, w, b_mn=True, bias=bias, act=1, aux=pre, out=o)
            elif a.epilogue == "dgelu":   # dgrad through GELU: out = (x @ w) * gelu'(saved pre-activation)
                o = torch.empty(M, N, device=dev, dtype=torch.bfloat16); pre = torch.randn(M, N, device=dev).bfloat16()
                fn = lambda: gemm(x, w, b_mn=True, act=2, aux=pre, out=o)
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
