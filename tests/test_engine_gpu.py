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


def test_dense_engine_with_dropout_matches_oracle_under_the_same_masks(monkeypatch):
    """The configuration the benchmarks run (dropout 0.1 on embeddings, attention probabilities and
    both residual branches), end to end: every mask the kernels apply is rebuilt on the host from
    the same counter-based generator (attention: read back from the keep bits the forward kernel
    stores) and handed to the fp32 oracle in call order, then losses and every parameter gradient
    are compared.  A backward kernel that regenerated a different mask than its forward twin
    (LayerNorm backward re-deriving the mask of the projection below it, attention backward
    reading the stored bits) would show up here."""
    import ctypes

    import torch.nn.functional as F

    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.models.engine import B200Engine
    from allie_b200.ops import _lib

    torch.manual_seed(0)
    B, T, d, H, L, p = 4, 256, 256, 4, 3, 0.1
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=L, n_embd=d,
                             n_head=H, n_positions=T, resid_pdrop=p, embd_pdrop=p, attn_pdrop=p)
    oracle = copy.deepcopy(model).float().train()
    words = _windows(tok, B, T, seed=3)
    batch = tok.pad_and_collate(list(words))

    eng = B200Engine(model, "cuda")
    w = torch.from_numpy(words.astype(np.int32)).cuda()
    eng.load_window(w)
    seed = eng._next_seed()
    buf = eng.forward(B, T, True, seed, True, True)
    eng.backward(B, T, seed)
    torch.cuda.synchronize()
    _lib.check_status()
    got = eng.loss_out.tolist()

    thr = _lib.dropout_thr16(p)
    scale = 65536.0 / (65536 - thr)
    lib = _lib.cuda()

    def host_mask(stream, n):
        out = np.empty(n, dtype=np.uint8)
        assert lib.ab_dropout_mask_host(ctypes.c_ulonglong(seed), ctypes.c_uint(stream), ctypes.c_longlong(n),
                                        ctypes.c_uint(thr), out.ctypes.data_as(ctypes.c_void_p)) == 0
        return torch.from_numpy(out).float()

    def attn_mask(l):
        words_ = buf["dmask"][l].cpu().numpy().view(np.uint32)              # [B, H, T, T/32], bit = key % 32
        bits = ((words_[..., None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(B, H, T, T)
        keep = torch.from_numpy(bits.astype(np.float32))
        return torch.tril(keep)            # keys past the query were never generated (and carry zero weight)

    # masks in the order the oracle's forward asks for them: embeddings, then per block
    # attention probabilities, attention projection branch, MLP branch
    masks = [host_mask(0, B * T * d).view(B, T, d)]
    for l in range(L):
        masks += [attn_mask(l), host_mask(1 + 3 * l, B * T * d).view(B, T, d), host_mask(2 + 3 * l, B * T * d).view(B, T, d)]
    queue = list(masks)

    def fake_dropout(x, p_=0.5, training=True, inplace=False):
        if not training or p_ == 0.0:
            return x
        m = queue.pop(0)
        assert m.shape == x.shape, (m.shape, x.shape)
        return x * m * scale

    monkeypatch.setattr(F, "dropout", fake_dropout)
    out = oracle(**batch)
    out["loss"].backward()
    assert not queue
    frac = 1.0 - float(masks[0].mean())
    assert abs(frac - p) < 0.01                                    # the masks really drop about 10 %
    for i, k in enumerate(("loss", "lm_loss", "value_loss", "time_loss")):
        assert abs(got[i] - out[k].item()) < 2e-2 * max(1.0, abs(out[k].item())), (k, got[i], out[k].item())
    ref_params = dict(oracle.named_parameters())
    for n, prm in model.named_parameters():
        g, gr = prm.grad.float().cpu(), ref_params[n].grad
        scale_g = gr.abs().max().item() + 1e-12
        assert (g - gr).abs().max().item() / scale_g < 0.08, n


def test_graph_replayed_micro_step_matches_ordinary_launches():
    """The micro-step replayed as a CUDA graph (dropout on): every replay draws new masks (the
    device-side salt that its first node advances) and computes what the ordinary launches compute
    when they are given the captured seed and the same salt value."""
    import ctypes

    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.models.engine import B200Engine
    from allie_b200.ops import _lib
    from allie_b200.ops._lib import ptr

    torch.manual_seed(0)
    B, T = 4, 256
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    kw = dict(n_layer=2, n_embd=256, n_head=4, n_positions=T, resid_pdrop=0.1, embd_pdrop=0.1, attn_pdrop=0.1)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **kw)
    eng = B200Engine(model, "cuda")
    assert eng.enable_step_graph(True)
    w = torch.from_numpy(_windows(tok, B, T).astype(np.int32)).cuda()
    params = dict(model.named_parameters())

    def grads():
        torch.cuda.synchronize()
        _lib.check_status()
        return {n: p.grad.float().clone() for n, p in params.items()}

    eng.micro_step(w)                       # ordinary launches (first use of the shape)
    assert not eng._step_graphs[next(iter(eng._step_graphs))]
    eng.zero_grad()
    launches0 = _lib.LAUNCHES
    loss1 = eng.micro_step(w).clone()       # captured here, replay 1
    entry = next(iter(eng._step_graphs.values()))
    assert entry["graph"] is not None and _lib.LAUNCHES - launches0 == entry["launches"] > 50   # one replay
    g1 = grads()
    salt1 = int(eng._salt.item())
    eng.zero_grad()
    loss2 = eng.micro_step(w).clone()       # replay 2: same data, other masks
    g2 = grads()
    salt2 = int(eng._salt.item())
    assert salt1 != salt2
    assert abs(loss1[0].item() - loss2[0].item()) > 1e-6
    assert all(torch.isfinite(v).all() for v in g2.values())

    # ordinary launches with the captured seed and each replay's salt value reproduce the replays
    lib = _lib.cuda()
    salt = torch.zeros(1, dtype=torch.int64, device="cuda")
    for want_loss, want_g, s in ((loss1, g1, salt1), (loss2, g2, salt2)):
        eng.zero_grad()
        salt.fill_(s)
        assert lib.ab_set_seed_salt(ptr(salt)) == 0
        try:
            Bt, Tt = eng.load_window(w)
            eng.forward(Bt, Tt, True, entry["seed"], True, True)
            eng.backward(Bt, Tt, entry["seed"])
        finally:
            lib.ab_set_seed_salt(None)
        got = grads()
        assert abs(eng.loss_out[0].item() - want_loss[0].item()) < 1e-4 * max(1.0, abs(want_loss[0].item()))
        for n in want_g:
            scale = want_g[n].abs().max().item() + 1e-12
            assert (got[n] - want_g[n]).abs().max().item() / scale < 1e-3, n

    # a micro-step with a bucket hook keeps the ordinary launches
    eng.zero_grad()
    seen = []
    eng.micro_step(w, bucket_hook=seen.append)
    torch.cuda.synchronize()
    assert seen == list(range(len(eng.arena.buckets)))       # called once per bucket, in order
