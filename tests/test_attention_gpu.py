"""tcgen05 causal attention (forward and backward) against a plain PyTorch fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(qkv, B, T, H, hd, mask=None, scale_keep=1.0):
    q5 = qkv.float().view(B, T, 3, H, hd)
    q, k, v = (q5[:, :, i].transpose(1, 2) for i in range(3))
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    causal = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~causal, float("-inf"))
    p = s.softmax(-1)
    lse = torch.logsumexp(s, -1)
    if mask is not None:
        p = p * mask * scale_keep
    o = (p @ v).transpose(1, 2).reshape(B * T, H * hd)
    return o, lse


@pytest.mark.parametrize("B,T,H,hd", [(2, 128, 2, 64), (2, 512, 3, 64), (1, 200, 2, 64), (2, 256, 2, 128),
                                      (1, 40, 1, 128), (20, 384, 16, 64)])
def test_attention_fwd_bwd_no_dropout(B, T, H, hd):
    from allie_b200.ops import _lib
    from allie_b200.ops.attention import attention_bwd, attention_fwd

    torch.manual_seed(0)
    dev = "cuda"
    d = H * hd
    qkv = (torch.randn(B * T, 3 * d, device=dev) * 0.7).bfloat16()
    out = torch.zeros(B * T, d, device=dev, dtype=torch.bfloat16)
    lse = torch.zeros(B, H, T, device=dev)
    attention_fwd(qkv, out, lse, B, T, H, hd, 0.0, 0, 0)
    torch.cuda.synchronize()
    _lib.check_status()
    leaf = qkv.float().requires_grad_(True)
    o_ref, lse_ref = _ref(leaf, B, T, H, hd)
    assert torch.allclose(out.float(), o_ref, rtol=2e-2, atol=2e-2), (out.float() - o_ref).abs().max()
    assert torch.allclose(lse, lse_ref, rtol=1e-3, atol=1e-2)
    dout = (torch.randn(B * T, d, device=dev) * 0.5).bfloat16()
    delta = torch.zeros(B, H, T, device=dev)
    o_ref.backward(dout.float())
    g = leaf.grad
    # two-kernel backward, and for head_dim 64 also the single-kernel one with its fp32 dQ
    # accumulator under both of its schedules (1 = one key tile per CTA, 2 = persistent walk)
    from allie_b200.ops.attention import set_backward_schedule

    variants = [(None, 0)] + ([(torch.zeros(B * T, d, device=dev), 1), (torch.zeros(B * T, d, device=dev), 2)]
                              if hd == 64 else [])
    for dq_acc, schedule in variants:
        set_backward_schedule(schedule)
        dqkv = torch.zeros(B * T, 3 * d, device=dev, dtype=torch.bfloat16)
        attention_bwd(qkv, out, lse, dout, dqkv, delta, B, T, H, hd, 0.0, 0, 0, None, dq_acc)
        torch.cuda.synchronize()
        _lib.check_status()
        err = (dqkv.float() - g).abs().max().item()
        assert err < 3e-2 * max(1.0, g.abs().max().item()), err
        for i, name in enumerate("qkv"):
            a, b_ = dqkv.float()[:, i * d:(i + 1) * d], g[:, i * d:(i + 1) * d]
            rel = (a - b_).norm() / (b_.norm() + 1e-9)
            assert rel < 2e-2, (name, rel.item(), dq_acc is not None)
        if dq_acc is not None:
            assert float(dq_acc.abs().max()) == 0.0     # handed back cleared
    set_backward_schedule(0)


def test_attention_dropout_mask_consistency():
    """Recover the dropped attention matrix through its linearity in V, check the keep rate and
    scaling, and check the backward pass against autograd with that same mask."""
    from allie_b200.ops import _lib
    from allie_b200.ops.attention import attention_bwd, attention_fwd

    torch.manual_seed(1)
    dev = "cuda"
    B, T, H, hd, p = 1, 256, 2, 64, 0.25
    d = H * hd
    seed, stream = 987654321, 5
    qkv = (torch.randn(B * T, 3 * d, device=dev) * 0.5).bfloat16()
    A = torch.zeros(B, H, T, T, device=dev)
    lse = torch.zeros(B, H, T, device=dev)
    for blk in range(T // hd):
        probe = qkv.clone()
        v = torch.zeros(B, T, H, hd, device=dev)
        for c in range(hd):
            v[:, blk * hd + c, :, c] = 1.0
        probe[:, 2 * d:] = v.view(B * T, d).bfloat16()
        out = torch.zeros(B * T, d, device=dev, dtype=torch.bfloat16)
        attention_fwd(probe, out, lse, B, T, H, hd, p, seed, stream)
        A[:, :, :, blk * hd:(blk + 1) * hd] = out.float().view(B, T, H, hd).permute(0, 2, 1, 3)
    torch.cuda.synchronize()
    _lib.check_status()
    causal = torch.ones(T, T, dtype=torch.bool, device=dev).tril()
    mask = (A != 0)
    keep_rate = mask[..., causal].float().mean().item()
    assert abs(keep_rate - (1 - p)) < 0.01, keep_rate
    assert not mask[..., ~causal].any()
    thr = _lib.dropout_thr16(p)
    scale_keep = 65536.0 / (65536 - thr)
    leaf = qkv.float().requires_grad_(True)
    o_ref, _ = _ref(leaf, B, T, H, hd, mask.float(), scale_keep)
    out = torch.zeros(B * T, d, device=dev, dtype=torch.bfloat16)
    bits = torch.zeros(B, H, T, T // 32, device=dev, dtype=torch.int32)
    attention_fwd(qkv, out, lse, B, T, H, hd, p, seed, stream, bits)
    assert torch.allclose(out.float(), o_ref, rtol=3e-2, atol=3e-2)
    # the stored keep bits are the mask recovered above
    unpacked = ((bits.unsqueeze(-1) >> torch.arange(32, device=dev)) & 1).view(B, H, T, T).bool()
    assert torch.equal(unpacked & causal, mask & causal)
    dout = (torch.randn(B * T, d, device=dev) * 0.5).bfloat16()
    delta = torch.zeros(B, H, T, device=dev)
    o_ref.backward(dout.float())
    # regenerate the mask / read the stored bits; two-kernel / single-kernel backward
    from allie_b200.ops.attention import set_backward_schedule

    for use_bits, fused in ((False, 0), (True, 0), (False, 1), (True, 1), (False, 2), (True, 2)):
        set_backward_schedule(fused)           # 0: two-kernel backward; 1, 2: the fused kernel's schedules
        dqkv = torch.zeros(B * T, 3 * d, device=dev, dtype=torch.bfloat16)
        dq_acc = torch.zeros(B * T, d, device=dev) if fused else None
        attention_bwd(qkv, out, lse, dout, dqkv, delta, B, T, H, hd, p, seed, stream,
                      bits if use_bits else None, dq_acc)
        torch.cuda.synchronize()
        _lib.check_status()
        rel = (dqkv.float() - leaf.grad).norm() / leaf.grad.norm()
        assert rel < 3e-2, (rel.item(), use_bits, fused)
    set_backward_schedule(0)
