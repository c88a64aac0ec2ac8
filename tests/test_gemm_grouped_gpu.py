"""Grouped CTA-pair GEMM (``csrc/gemm_grouped.cu``) against plain PyTorch fp32 on ragged groups:
forward-type launches (live rows only, per-group bias, GELU epilogues), the weight-gradient form
(contraction over each group's live rows), arrival counters and the scattering epilogue (GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _gelu(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def _setup(G, cap, K, N, rows, seed=0):
    torch.manual_seed(seed)
    dev = "cuda"
    a = (torch.randn(G * cap, K, device=dev) * 0.5).bfloat16()
    rows_t = torch.tensor(rows, dtype=torch.int32, device=dev)
    return a, rows_t


@pytest.mark.parametrize("b_mn", [True, False])
def test_forward_type_live_rows_bias_and_gelu(b_mn):
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm_grouped

    G, cap, K, N = 3, 512, 128, 384
    rows = [300, 0, 512]
    a, rows_t = _setup(G, cap, K, N, rows)
    w = (torch.randn(G, K, N, device="cuda") * 0.1).bfloat16()
    b = w if b_mn else w.transpose(1, 2).contiguous()
    bias = torch.randn(G, N, device="cuda")
    out = torch.full((G * cap, N), 7.0, device="cuda", dtype=torch.bfloat16)
    pre = torch.full((G * cap, N), 7.0, device="cuda", dtype=torch.bfloat16)
    gemm_grouped(a, b, rows_t, cap, mode=1, b_mn=b_mn, out=out, bias=bias, act=1, aux=pre)
    torch.cuda.synchronize()
    _lib.check_status()
    for g in range(G):
        r = rows[g]
        ref_pre = a[g * cap:g * cap + r].float() @ w[g].float() + bias[g]
        got_pre = pre[g * cap:g * cap + r].float()
        assert (got_pre - ref_pre).abs().max().item() < 0.05 if r else True
        assert (out[g * cap:g * cap + r].float() - _gelu(ref_pre)).abs().max().item() < 0.05 if r else True
        # rows past the next multiple of 128 of a group's live rows are never touched
        pad = (r + 127) // 128 * 128
        assert (out[g * cap + pad:(g + 1) * cap].float() == 7.0).all()
    # GELU' epilogue (backward of the up projection): v * gelu'(pre)
    dy = (torch.randn(G * cap, K, device="cuda") * 0.5).bfloat16()
    dpre = torch.zeros(G * cap, N, device="cuda", dtype=torch.bfloat16)
    gemm_grouped(dy, b, rows_t, cap, mode=1, b_mn=b_mn, out=dpre, act=2, aux=pre)
    torch.cuda.synchronize()
    _lib.check_status()
    for g in range(G):
        r = rows[g]
        if not r:
            continue
        x = pre[g * cap:g * cap + r].float().requires_grad_(True)
        _gelu(x).sum().backward()
        ref = (dy[g * cap:g * cap + r].float() @ w[g].float()) * x.grad
        assert (dpre[g * cap:g * cap + r].float() - ref).abs().max().item() < 0.06


def test_weight_gradient_form_contracts_over_live_rows():
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm_grouped

    G, cap, Mo, N = 3, 512, 128, 320
    rows = [200, 0, 512]
    torch.manual_seed(1)
    a = (torch.randn(G * cap, Mo, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(G * cap, N, device="cuda") * 0.5).bfloat16()
    for g in range(G):      # rows between the live ones and the next multiple of 128 must be zero in one operand
        pad = (rows[g] + 127) // 128 * 128
        b[g * cap + rows[g]:g * cap + pad] = 0
    rows_t = torch.tensor(rows, dtype=torch.int32, device="cuda")
    out = torch.ones(G, Mo, N, device="cuda")
    gemm_grouped(a, b, rows_t, cap, mode=2, out=out)
    torch.cuda.synchronize()
    _lib.check_status()
    for g in range(G):
        r = rows[g]
        ref = 1.0 + a[g * cap:g * cap + r].float().t() @ b[g * cap:g * cap + r].float()
        assert (out[g] - ref).abs().max().item() < 0.02 * max(1.0, ref.abs().max().item())


def test_arrival_counters_and_scattering_epilogue_on_one_rank():
    """With the rank as its own only peer: counters already at their targets let the launch run,
    every live result row lands at its return address, and the release flag carries the epoch."""
    from allie_b200.ops import _lib
    from allie_b200.ops.gemm import gemm_grouped

    G, cap, K, N = 2, 256, 256, 128
    rows = [130, 256]
    a, rows_t = _setup(G, cap, K, N, rows, seed=2)
    w = (torch.randn(G, K, N, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(G, N, device="cuda")
    ready = torch.zeros(G * cap // 128, dtype=torch.int32, device="cuda")
    for g in range(G):
        for blk in range(cap // 128):
            ready[g * (cap // 128) + blk] = max(0, min(128, rows[g] - blk * 128))
    n_live = sum(rows)
    perm = torch.randperm(n_live, device="cuda").to(torch.int32)          # return addresses
    ret = torch.full((G * cap,), -1, dtype=torch.int32, device="cuda")
    k = 0
    for g in range(G):
        ret[g * cap:g * cap + rows[g]] = perm[k:k + rows[g]]
        k += rows[g]
    dst = torch.zeros(n_live, N, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(6 * 32, dtype=torch.int32, device="cuda")
    ticket = torch.zeros(4, dtype=torch.int32, device="cuda")
    peers = [dst.data_ptr()] + [None] * 7
    fl = [flags.data_ptr()] + [None] * 7
    gemm_grouped(a, w, rows_t, cap, mode=1, b_mn=True, bias=bias, tile_ready=ready,
                 scatter=dict(ret=ret, peers=peers, flags=fl, phase=2, epoch=5, rank=0, world=1, ticket=ticket.data_ptr()))
    torch.cuda.synchronize()
    _lib.check_status()
    assert int(flags[2 * 32]) == 5 and int(ticket[0]) == 0
    k = 0
    for g in range(G):
        r = rows[g]
        ref = a[g * cap:g * cap + r].float() @ w[g].float() + bias[g]
        got = dst[perm[k:k + r].long()].float()
        assert (got - ref).abs().max().item() < 0.05
        k += r
