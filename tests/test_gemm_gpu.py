"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (384, 768, 1024), (200, 264, 136),
                                   (1000, 128, 512), (64, 64, 64),
                                   # large enough for the CTA-pair kernel, with ragged edges
                                   (1000, 264, 136), (640, 768, 320), (2304, 1024, 192),
                                   (512, 256, 64), (768, 512, 40)])      # one K block; ragged K
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    torch.manual_seed(0)
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (out - ref).abs().max().item()
    assert err < 2e-2 * (K ** 0.5), (err, M, N, K)
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2 * (K ** 0.5) * 0.1)


def test_gemm_epilogues():
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    torch.manual_seed(1)
    dev = "cuda"
    M, N, K = 512, 768, 256
    a = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(K, N, device=dev) * 0.05).bfloat16()
    bias = torch.randn(N, device=dev)
    ref = a.float() @ w.float() + bias
    # bias, bf16 out
    out = gemm(a, w, b_mn=True, bias=bias)
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    # bias + gelu, preact saved
    pre = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    out = gemm(a, w, b_mn=True, bias=bias, act=1, aux=pre)
    assert torch.allclose(pre.float(), ref, rtol=2e-2, atol=2e-2)
    g = torch.nn.functional.gelu(ref, approximate="tanh")
    assert torch.allclose(out.float(), g, rtol=2e-2, atol=2e-2)
    # gelu backward multiply
    dy = torch.randn(M, K, device=dev).bfloat16()
    wt = (torch.randn(N, K, device=dev) * 0.05).bfloat16()  # dX[M,N] = dy[M,K] @ wt[N,K]^T
    o2 = gemm(dy, wt, act=2, aux=pre)
    x = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(x, approximate="tanh").backward(dy.float() @ wt.float().t())
    assert torch.allclose(o2.float(), x.grad, rtol=3e-2, atol=3e-2)
    # residual (no dropout), fp32 out, in place
    resid = torch.randn(M, N, device=dev)
    r0 = resid.clone()
    gemm(a, w, b_mn=True, bias=bias, resid=resid, out=resid)
    assert torch.allclose(resid, r0 + ref, rtol=1e-2, atol=2e-2)
    # residual with dropout: kept fraction and scaling
    resid = torch.zeros(M, N, device=dev)
    gemm(a, w, b_mn=True, bias=bias, resid=resid, out=resid, drop_p=0.25, drop_seed=123, drop_stream=7)
    kept = resid != 0
    frac = kept.float().mean().item()
    assert abs(frac - 0.75) < 0.01, frac
    assert torch.allclose(resid[kept], (ref / 0.75)[kept], rtol=1e-2, atol=3e-2)
    # accumulate with split-K (wgrad shape): dW[K,N] += a^T @ dyy
    dyy = torch.randn(M, N, device=dev).bfloat16()
    dw = torch.ones(K, N, device=dev)
    gemm(a, dyy, a_mn=True, b_mn=True, out=dw, accumulate=True, k_splits=4)
    refw = 1.0 + a.float().t() @ dyy.float()
    assert torch.allclose(dw, refw, rtol=1e-3, atol=5e-2)
    torch.cuda.synchronize()
    _lib.check_status()


def test_gemm_big_and_timing():
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    dev = "cuda"
    torch.manual_seed(2)
    M, N, K = 16384, 4096, 1024
    a = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(K, N, device=dev) * 0.03).bfloat16()
    out = gemm(a, w, b_mn=True)
    ref = (a @ w).float()
    assert torch.allclose(out.float(), ref, rtol=3e-2, atol=3e-2)
    _lib.check_status()


def test_gemm_pair_split_k_accumulate():
    """Weight-gradient shape on the CTA-pair kernel: MN-major operands, split-K, TMA reduce-add."""
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    torch.manual_seed(3)
    dev = "cuda"
    T, I, O = 4096, 1024, 768
    x = torch.randn(T, I, device=dev).bfloat16()
    dy = torch.randn(T, O, device=dev).bfloat16()
    dw = torch.full((I, O), 2.0, device=dev)
    gemm(x, dy, a_mn=True, b_mn=True, out=dw, accumulate=True, k_splits=4)
    ref = 2.0 + x.float().t() @ dy.float()
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.allclose(dw, ref, rtol=1e-3, atol=0.2)


def test_gemm_skinny_residual_update_in_place():
    """Decode-sized x += a @ w + bias: few output tiles, long K (taken by the split-K route)."""
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    torch.manual_seed(4)
    dev = "cuda"
    for M, N, K in ((256, 1024, 4096), (192, 1024, 1024), (40, 768, 2048)):
        a = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(K, N, device=dev) * 0.03).bfloat16()
        bias = torch.randn(N, device=dev)
        x = torch.randn(M, N, device=dev)
        want = x + a.float() @ w.float() + bias
        gemm(a, w, b_mn=True, bias=bias, resid=x, out=x)
        torch.cuda.synchronize()
        _lib.check_status()
        assert torch.allclose(x, want, rtol=1e-3, atol=3e-2), (M, N, K, (x - want).abs().max().item())


@pytest.mark.parametrize("M,N,K", [(1000, 328, 192), (2048, 1024, 256), (640, 72, 128)])
def test_gemm_gelu_backward_epilogue_ragged(M, N, K):
    """out = (dy @ w^T) * gelu'(pre) on shapes with ragged row / column tiles (the CTA-pair kernel
    fetches the pre-activation tiles by TMA one tile ahead)."""
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    torch.manual_seed(5)
    dev = "cuda"
    dy = torch.randn(M, K, device=dev).bfloat16()
    wt = (torch.randn(N, K, device=dev) * 0.05).bfloat16()
    pre = torch.randn(M, N, device=dev).bfloat16()
    out = gemm(dy, wt, act=2, aux=pre)
    torch.cuda.synchronize()
    _lib.check_status()
    x = pre.float().requires_grad_(True)
    torch.nn.functional.gelu(x, approximate="tanh").backward(dy.float() @ wt.float().t())
    assert torch.allclose(out.float(), x.grad, rtol=3e-2, atol=3e-2), (out.float() - x.grad).abs().max().item()


def test_gemm_gelu_derivative_kept_in_aux():
    """act=1 / act=2 with aux_grad: the forward launch stores GELU'(pre-activation), the backward
    launch multiplies by it; same results as the pre-activation form."""
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm

    torch.manual_seed(6)
    dev = "cuda"
    M, N, K = 1000, 1152, 256
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(K, N, device=dev) * 0.08).bfloat16()
    bias = torch.randn(N, device=dev)
    act = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    dact = torch.empty_like(act)
    gemm(x, w, b_mn=True, bias=bias, act=1, aux=dact, out=act, aux_grad=True)
    dy = torch.randn(M, 512, device=dev).bfloat16()
    w2 = (torch.randn(N, 512, device=dev) * 0.05).bfloat16()
    dpre = gemm(dy, w2, act=2, aux=dact, aux_grad=True)
    torch.cuda.synchronize()
    _lib.check_status()
    pre = (x.float() @ w.float() + bias).requires_grad_(True)
    ref = torch.nn.functional.gelu(pre, approximate="tanh")
    (want_d,) = torch.autograd.grad(ref.sum(), pre)
    assert torch.allclose(act.float(), ref.detach(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(dact.float(), want_d, rtol=1e-2, atol=1e-2), (dact.float() - want_d).abs().max().item()
    want = (dy.float() @ w2.float().t()) * want_d
    assert torch.allclose(dpre.float(), want, rtol=3e-2, atol=3e-2), (dpre.float() - want).abs().max().item()
