"""The kernel engine against the fp32 PyTorch oracle model on the same weights and batch:
losses, every parameter gradient, the evaluation outputs and one clipped AdamW step."""
import copy

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _windows(tok, B, T, seed=0):
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, 1968, size=(B, T)).astype(np.uint32)
    secs = rng.integers(0, 30, size=(B, T)).astype(np.uint32)
    words = ids | ((secs + 1) << 16) | (rng.integers(0, 3, size=(B, 1)).astype(np.uint32) << 14)
    words[:, 0] = (len(tok) + 1500) | (words[:, 0] & 0xC000)      # two ELO control tokens
    words[:, 1] = (len(tok) + 2100) | (words[:, 1] & 0xC000)
    words[:, 2] = 1970 | (words[:, 2] & 0xFFFFC000)
    return words


@pytest.mark.parametrize("n_embd,n_head", [(256, 4), (512, 4), (1280, 20), (2048, 16)])   # head sizes 64, 128; the large-ablation and MoE widths
def test_dense_engine_matches_oracle(n_embd, n_head):
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.models.engine import B200Engine
    from allie_b200.ops import _lib

    torch.manual_seed(0)
    B, T = 8, 256
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    kw = dict(n_layer=3, n_embd=n_embd, n_head=n_head, n_positions=T, resid_pdrop=0.0, embd_pdrop=0.0,
              attn_pdrop=0.0)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **kw)
    oracle = copy.deepcopy(model).float()
    words = _windows(tok, B, T)
    batch = tok.pad_and_collate(list(words))
    out = oracle(**batch)
    out["loss"].backward()

    eng = B200Engine(model, "cuda")
    w = torch.from_numpy(words.astype(np.int32)).cuda()
    loss = eng.micro_step(w)
    torch.cuda.synchronize()
    _lib.check_status()
    got = loss.tolist()
    for i, k in enumerate(("loss", "lm_loss", "value_loss", "time_loss")):
        assert abs(got[i] - out[k].item()) < 2e-2 * max(1.0, abs(out[k].item())), (k, got[i], out[k].item())

    ref_params = dict(oracle.named_parameters())
    for n, p in model.named_parameters():
        g, gr = p.grad.float().cpu(), ref_params[n].grad
        scale = gr.abs().max().item() + 1e-12
        assert (g - gr).abs().max().item() / scale < 0.08, n

    # the collated-batch entry computes the same losses as the raw-window entry
    eng.zero_grad()
    loss2 = eng.micro_step_batch(batch).tolist()
    assert all(abs(a - b) < 1e-3 * max(1.0, abs(a)) for a, b in zip(got, loss2))

    ev = eng.evaluate_batch(batch)
    assert abs(ev["loss"].item() - out["loss"].item()) < 2e-2 * max(1.0, out["loss"].item())
    assert (ev["logits"].float().cpu() - out["logits"]).abs().max().item() < 0.15
    assert (ev["value_logits"].float().cpu() - out["value_logits"]).abs().max().item() < 0.05

    # one clipped AdamW step against torch.optim.AdamW with the same decay / no-decay split
    arena = eng.arena
    decay = [n for n in arena.names if n in arena.decay_names]
    no_decay = [n for n in arena.names if n not in arena.decay_names]
    opt = torch.optim.AdamW([{"params": [ref_params[n] for n in decay], "weight_decay": 0.01},
                             {"params": [ref_params[n] for n in no_decay], "weight_decay": 0.0}],
                            lr=1e-3, betas=(0.9, 0.95))
    torch.nn.utils.clip_grad_norm_(oracle.parameters(), 1.0)
    opt.step()
    eng.zero_grad()
    eng.micro_step(w)
    eng.optimizer_step(1e-3, (0.9, 0.95), 1e-8, 0.01, 1.0)
    torch.cuda.synchronize()
    _lib.check_status()
    worst, total, count = 0.0, 0.0, 0
    for n, p in model.named_parameters():
        d = (p.data.float().cpu() - ref_params[n].data).abs()
        worst = max(worst, d.max().item()); total += d.sum().item(); count += d.numel()
    # the first Adam step moves every weight by about lr; a sign flip on a near-zero gradient costs 2 lr
    assert worst < 2.5e-3 and total / count < 1e-4, (worst, total / count)
