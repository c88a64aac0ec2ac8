"""MoE layers on the engine (routing, dispatch/combine kernels, device-sized expert GEMMs) against
the dense fp32 oracle: losses and every gradient, single GPU (the rank is its own only peer)."""
import copy

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_moe_engine_matches_oracle():
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.models.engine import B200Engine
    from allie_b200.ops import _lib

    torch.manual_seed(0)
    T, B = 128, 8
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    kw = dict(n_layer=3, n_embd=256, n_head=4, n_positions=T, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
              num_experts=8, moe_top_k=2, moe_ffn=512, moe_layer_freq=3, aux_loss_coef=0.05, capacity_factor=8.0)
    m = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **kw)
    with torch.no_grad():       # spread the router so that top-2 choices are not razor-edge ties
        for n, p in m.named_parameters():
            if "router" in n:
                p.mul_(20.0)
    ref = copy.deepcopy(m).float()
    rng = np.random.default_rng(0)
    words = rng.integers(0, 1968, size=(B, T)).astype(np.uint32) | ((rng.integers(0, 30, size=(B, T)).astype(np.uint32) + 1) << 16)
    words[:, 0] = len(tok) + 1500
    words[:, 1] = len(tok) + 2100
    batch = tok.pad_and_collate(list(words))
    out = ref(**batch)
    out["loss"].backward()
    eng = B200Engine(m, "cuda")
    loss = eng.micro_step(torch.from_numpy(words.astype(np.int32)).cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    got = loss.tolist()
    assert abs(got[0] - out["loss"].item()) < 3e-2, (got, out["loss"].item())
    assert abs(got[1] - out["lm_loss"].item()) < 2e-2
    ctx = next(iter(eng._moe_ctx.values()))
    assert int(ctx.overflow.item()) == 0
    assert abs(float(ctx.aux_total) - float(out["aux_loss"])) < 2e-2 * max(1.0, float(out["aux_loss"]))
    stats = eng.moe_stats()
    assert stats is not None and not stats["overflow"] and abs(stats["aux_loss"] - float(ctx.aux_total)) < 1e-6
    assert list(stats["expert_tokens"]) == [2] and sum(stats["expert_tokens"][2]) == B * T * 2
    assert stats["max_over_mean_load"] >= 1.0
    refp = dict(ref.named_parameters())
    worst = {}
    for n, p in m.named_parameters():
        g, gr = p.grad.float().cpu(), refp[n].grad
        rel = ((g - gr).norm() / (gr.norm() + 1e-9)).item()
        worst[n] = rel
    bad = {n: r for n, r in worst.items() if r > 6e-2}
    assert not bad, bad
    # an optimizer step over all four arena regions runs
    eng.optimizer_step(1e-3, (0.9, 0.95), 1e-8, 0.01, 1.0)
    torch.cuda.synchronize()
    _lib.check_status()
