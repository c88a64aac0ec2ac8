"""Non-GEMM sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _done():
    from allie_b200.ops import _lib

    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("M,d", [(300, 256), (1024, 1024), (77, 2048)])
def test_layernorm_forward(M, d, rms):
    from allie_b200.ops import kernels as K

    torch.manual_seed(0)
    x = torch.randn(M, d, device=DEV) * 2 + 0.3
    g = torch.randn(d, device=DEV)
    b = torch.randn(d, device=DEV)
    y = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    mean = torch.empty(M, device=DEV)
    rstd = torch.empty(M, device=DEV)
    K.layernorm_fwd(x, g, None if rms else b, y, mean, rstd, 1e-5, rms=rms)     # RMSNorm has no shift
    _done()
    if rms:
        ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * g
    else:
        ref = F.layer_norm(x, (d,), g, b, 1e-5)
        assert torch.allclose(mean, x.mean(-1), atol=1e-5)
    assert torch.allclose(y.float(), ref, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("M,d,rms", [(520, 1024, False), (520, 1024, True), (77, 256, False), (131, 1280, False),
                                     (66, 2048, True), (3, 128, False)])
def test_layernorm_backward_with_residual_and_params(M, d, rms):
    from allie_b200.ops import kernels as K

    torch.manual_seed(1)
    x = (torch.randn(M, d, device=DEV) * 1.5).requires_grad_(True)
    g = torch.randn(d, device=DEV, requires_grad=True)
    b = torch.randn(d, device=DEV, requires_grad=True)
    dy = torch.randn(M, d, device=DEV).bfloat16()
    dres = torch.randn(M, d, device=DEV)
    if rms:
        yref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * g
    else:
        yref = F.layer_norm(x, (d,), g, b, 1e-5)
    yref.backward(dy.float())
    y = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    mean = torch.empty(M, device=DEV)
    rstd = torch.empty(M, device=DEV)
    K.layernorm_fwd(x.detach(), g.detach(), None if rms else b.detach(), y, mean, rstd, 1e-5, rms=rms)
    dx = torch.empty(M, d, device=DEV)
    dbranch = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    dgamma = torch.zeros(d, device=DEV)
    dbeta = torch.zeros(d, device=DEV)
    K.layernorm_bwd(dy, x.detach(), mean, rstd, g.detach(), dres, dx, dbranch, dgamma,
                    None if rms else dbeta, rms=rms)
    _done()
    ref_dx = x.grad + dres
    assert torch.allclose(dx, ref_dx, rtol=1e-3, atol=2e-3)
    assert torch.allclose(dbranch.float(), ref_dx, rtol=1e-2, atol=3e-2)     # no dropout: a bf16 copy
    assert torch.allclose(dgamma, g.grad, rtol=1e-3, atol=5e-2)
    if not rms:
        assert torch.allclose(dbeta, b.grad, rtol=1e-3, atol=5e-2)


def test_layernorm_backward_dropout_copy_is_masked_and_scaled():
    from allie_b200.ops import kernels as K

    torch.manual_seed(2)
    M, d = 256, 1024
    x = torch.randn(M, d, device=DEV)
    g = torch.ones(d, device=DEV)
    b = torch.zeros(d, device=DEV)
    y = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    mean = torch.empty(M, device=DEV)
    rstd = torch.empty(M, device=DEV)
    K.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
    dy = torch.randn(M, d, device=DEV).bfloat16()
    dres = torch.randn(M, d, device=DEV) + 3.0     # keeps dx away from zero
    dx = torch.empty(M, d, device=DEV)
    dbranch = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    dgamma = torch.zeros(d, device=DEV)
    dbeta = torch.zeros(d, device=DEV)
    dbias = torch.full((d,), 0.5, device=DEV)
    K.layernorm_bwd(dy, x, mean, rstd, g, dres, dx, dbranch, dgamma, dbeta, drop_seed=11, drop_stream=5,
                    drop_p=0.25, dbias=dbias)
    _done()
    # fused bias gradient of the projection below: column sums of the masked copy, accumulated
    assert torch.allclose(dbias, 0.5 + dbranch.float().sum(0), rtol=1e-2, atol=0.5)
    kept = dbranch != 0
    frac = kept.float().mean().item()
    assert abs(frac - 0.75) < 0.01, frac
    assert torch.allclose(dbranch.float()[kept], (dx / 0.75)[kept], rtol=1e-2, atol=3e-2)


@pytest.mark.parametrize("M,d,params", [(37, 1280, True), (21, 1024, True), (19, 2048, True), (37, 1280, False)])
def test_layernorm_backward_dropout_mask_is_the_element_indexed_one(M, d, params):
    """The masked copy keeps exactly the elements that the generator keeps for element index
    row * d + column (the mask the projection's forward epilogue applied), in both backward kernels
    (with and without parameter gradients) and at widths where a thread owns two column groups."""
    import ctypes

    import numpy as np

    from allie_b200.ops import _lib
    from allie_b200.ops import kernels as K

    torch.manual_seed(4)
    x = torch.randn(M, d, device=DEV)
    g = torch.ones(d, device=DEV)
    y = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    mean = torch.empty(M, device=DEV)
    rstd = torch.empty(M, device=DEV)
    K.layernorm_fwd(x, g, torch.zeros(d, device=DEV), y, mean, rstd, 1e-5)
    dy = torch.randn(M, d, device=DEV).bfloat16()
    dres = torch.randn(M, d, device=DEV) + 5.0     # keeps dx away from zero
    dx = torch.empty(M, d, device=DEV)
    dbranch = torch.empty(M, d, device=DEV, dtype=torch.bfloat16)
    dgamma = torch.zeros(d, device=DEV) if params else None
    dbeta = torch.zeros(d, device=DEV) if params else None
    seed, stream, p = 1234567, 9, 0.3
    K.layernorm_bwd(dy, x, mean, rstd, g, dres, dx, dbranch, dgamma, dbeta, drop_seed=seed, drop_stream=stream,
                    drop_p=p)
    _done()
    host = np.empty(M * d, dtype=np.uint8)
    assert _lib.cuda().ab_dropout_mask_host(ctypes.c_ulonglong(seed), ctypes.c_uint(stream), ctypes.c_longlong(M * d),
                                            ctypes.c_uint(_lib.dropout_thr16(p)),
                                            host.ctypes.data_as(ctypes.c_void_p)) == 0
    want = torch.from_numpy(host).view(M, d).bool()
    assert torch.equal((dbranch != 0).cpu(), want)


def test_cross_entropy_loss_and_gradient():
    from allie_b200.ops import kernels as K

    torch.manual_seed(3)
    M, V = 700, 2048
    logits = (torch.randn(M, V, device=DEV) * 2).bfloat16()
    labels = torch.randint(0, V, (M,), device=DEV, dtype=torch.int32)
    labels[::7] = -100
    n_valid = (labels != -100).sum().to(torch.int32).reshape(1)
    ref_in = logits.float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, labels.long(), ignore_index=-100)
    (ref * 0.5).backward()
    acc = torch.zeros(4, device=DEV)
    work = logits.clone()
    K.ce_fwd_bwd(work, labels, n_valid, 0.5, acc, write_grad=True)
    _done()
    assert abs(acc[0].item() / n_valid.item() - ref.item()) < 2e-3 * max(1.0, ref.item())
    assert torch.allclose(work.float(), ref_in.grad, rtol=2e-2, atol=2e-6)
    # loss only: logits stay untouched
    acc.zero_()
    work = logits.clone()
    K.ce_fwd_bwd(work, labels, n_valid, 0.5, acc, write_grad=False)
    _done()
    assert torch.equal(work, logits)


@pytest.mark.parametrize("M,N", [(32768, 1024), (1000, 3072), (129, 4096), (64, 8)])
def test_column_sums(M, N):
    from allie_b200.ops import kernels as K

    torch.manual_seed(4)
    x = torch.randn(M, N, device=DEV).bfloat16()
    out = torch.full((N,), 1.5, device=DEV)
    K.colsum_bf16(x, out)
    _done()
    assert torch.allclose(out, 1.5 + x.float().sum(0), rtol=1e-3, atol=2e-2)
    # device-side row limit
    lim = torch.tensor([M // 3], device=DEV, dtype=torch.int32)
    out.zero_()
    K.colsum_bf16(x, out, m_limit=lim)
    _done()
    assert torch.allclose(out, x[: M // 3].float().sum(0), rtol=1e-3, atol=2e-2)


def test_adamw_with_clipping_matches_torch():
    from allie_b200.ops import kernels as K

    torch.manual_seed(5)
    n = 1 << 20
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 0.01
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    shadow = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in (1, 2, 3):
        ref_p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        nsq = torch.zeros(1, device=DEV)
        K.sumsq(g, nsq)
        K.adamw(p, g, m, v, shadow, 1e-3, 0.9, 0.95, 1e-8, 0.1, step, gnorm_sq=nsq, max_norm=1.0)
        _done()
        assert abs(nsq.item() - (g.double() ** 2).sum().item()) < 1e-3 * nsq.item()
        assert torch.allclose(p, ref_p.detach(), rtol=1e-5, atol=2e-6), step
        assert torch.allclose(shadow.float(), p, rtol=1e-2, atol=1e-3)
        g = g * 1.7 + 0.003


def test_cast_to_bf16():
    from allie_b200.ops import kernels as K

    src = torch.randn(100_003 * 8, device=DEV)
    dst = torch.empty_like(src, dtype=torch.bfloat16)
    K.cast_bf16(src, dst)
    _done()
    assert torch.equal(dst, src.bfloat16())


@pytest.mark.parametrize("M,V,K", [(1000, 2048, 256), (384, 1000, 128), (128 * 150 + 7, 2048, 1024)])
def test_fused_lmhead_cross_entropy_matches_fp32(M, V, K):
    """Fused output-embedding GEMM + cross entropy: summed loss and d logits against plain PyTorch
    fp32 on the same bf16 operands; ragged row count, ignored rows, a vocabulary that is not a
    multiple of the 256-column tile, more row tiles than SMs (second unit per CTA)."""
    import torch.nn.functional as F

    from allie_b200.ops import _lib, kernels as K_

    torch.manual_seed(M + V)
    h = (torch.randn(M, K, device="cuda") * 1.0).bfloat16()
    wte = (torch.randn(V, K, device="cuda") * 0.08).bfloat16()
    labels = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    labels[torch.rand(M, device="cuda") < 0.2] = -100
    n_valid = (labels >= 0).sum().to(torch.int32).reshape(1)
    coef = 0.7
    dlogits = torch.full((M, V), 3.0, device="cuda", dtype=torch.bfloat16)
    loss = torch.zeros(1, device="cuda")
    K_.lmhead_ce(h, wte, labels, n_valid, coef, dlogits, loss)
    torch.cuda.synchronize()
    _lib.check_status()
    logits = (h.float() @ wte.float().t()).requires_grad_(True)
    ref = F.cross_entropy(logits, labels.long(), ignore_index=-100, reduction="sum")
    (ref * coef / int(n_valid)).backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * ref.item()
    g = logits.grad
    err = (dlogits.float() - g).abs().max().item()
    assert err < 0.02 * g.abs().max().item() + 1e-7, (err, g.abs().max().item())
    assert (dlogits[labels < 0].float() == 0).all()
