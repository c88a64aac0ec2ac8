"""Interchange with the unmodified reference package (skipped when it is not installed under
``baseline/_ref``): a checkpoint written by this framework's trainer loads strictly into the
reference's model and optimizer, both tokenizers decode raw windows identically, and both models
return the same logits and losses from the same weights (CPU)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "modeling")),
                                reason="reference package not installed under baseline/_ref")


def test_checkpoint_tokenizer_and_forward_match_the_reference(tmp_path):
    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.train.trainer import Trainer

    os.environ["ALLIE_NO_WANDB"] = "1"
    shape = dict(n_layer=2, n_embd=64, n_head=2, n_positions=64, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    tok_kw = dict(max_length=48, vocab_size_multiple_of=128)
    tok = UCITokenizer(**tok_kw)
    rng = np.random.default_rng(3)
    stream = (rng.integers(0, 1968, size=4096).astype(np.uint32)
              | (rng.integers(0, 40, size=4096).astype(np.uint32) << 16)
              | (rng.integers(0, 3, size=4096).astype(np.uint32) << 14))
    tr = Trainer(Config({"trainer_config": {}}), output_dir=str(tmp_path / "run"), device="cpu", batch_size=4,
                 max_iters=2, decay_iters=2, warmup_iters=0, eval_interval=0, log_interval=-1, save_interval=0,
                 lr=1e-3, min_lr=1e-4, weight_decay=0.01, use_wandb=False)
    torch.manual_seed(0)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **shape)
    tr.setup_dataloaders(tok, stream, [], [])
    tr.setup_model(model)
    tr.train()                                            # three AdamW steps: the optimizer has state
    tr.save_ckpt("last")
    ck = torch.load(tmp_path / "run" / "last.pt", weights_only=False)
    windows = np.stack([stream[i:i + 48] for i in (0, 100, 200)])
    windows[:, 0] = len(tok) + 1500                       # ELO pseudo-tokens in front, as in real windows
    windows[:, 1] = len(tok) + 2250
    windows[2, 40:] = tok.pad_token_id                    # one padded row
    from allie_b200.data import Game

    games = [Game("180+0", 1520, 2410, "1-0", True, "e2e4 e7e5 g1f3 b8c6".split(), [0, 3, 70, 12]),
             Game("600+5", 900, 1100, "1/2-1/2", False, "d2d4 d7d5 c2c4".split(), [1, 1, 2]),
             Game("60+0", 2000, 1990, None, False, ["g1f3"] * 1 + ["g8f6"], [5, 6]),
             Game("180+2", 1500, 1500, "0-1", True, ["e2e4", "c7c5"] + ["g1f3", "b8c6", "f3g1", "c6b8"] * 15, [2] * 62)]
    flags = [{}, {"add_elo": False}, {"add_time_control": False}, {"add_termination": False, "add_value": False}]
    torch.save({"model": ck["model"], "optimizer": ck["optimizer"], "tokenizer": tok_kw, "shape": shape,
                "windows": windows.astype(np.int64), "games": [g.to_dict() for g in games],
                "tokenize_flags": flags}, tmp_path / "ours.pt")
    res = subprocess.run([sys.executable, os.path.join(HERE, "reference_worker.py"), str(tmp_path)],
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    ref = torch.load(tmp_path / "ref_out.pt", weights_only=False)

    from allie_b200.serve import SYSTEMS

    assert {a: (s.port, s.elo, s.algorithm, dict(s.algorithm_config)) for a, s in SYSTEMS.items()} == ref["systems"]
    assert ref["vocab"] == len(tok) and ref["ids"] == {"bos": tok.bos_token_id, "pad": tok.pad_token_id}
    batch = tok.pad_and_collate(list(windows.astype(np.uint32)))
    assert set(batch) == set(ref["batch"])
    for k, v in batch.items():
        assert torch.equal(v.to(ref["batch"][k].dtype), ref["batch"][k]), k
    # Game objects: the packed words (every flag combination) and the collated, truncated, padded batch
    ours_words = [tok.tokenize(g, **f).astype(np.int64) for g in games for f in flags]
    assert len(ours_words) == len(ref["words"])
    for a, b_ in zip(ours_words, ref["words"]):
        assert np.array_equal(a, b_)
    collated = tok.pad_and_collate(list(games))
    for k, v in collated.items():
        assert torch.equal(v.to(ref["collated_games"][k].dtype), ref["collated_games"][k]), k
    model.eval()
    with torch.no_grad():
        out = model(**batch)
    for k, want in ref["out"].items():
        assert torch.allclose(out[k].float(), want, atol=2e-4, rtol=1e-4), (k, (out[k].float() - want).abs().max())
    # the optimizer entry: same two groups, same numbering, moments arrive where the reference expects them
    groups = ck["optimizer"]["param_groups"]
    assert [len(g["params"]) for g in groups] == [ref["n_decay"], ref["n_no_decay"]]
    assert ref["opt_step"] == float(ck["optimizer"]["state"][0]["step"]) > 0
    assert abs(ref["opt_exp_avg_norm"] - float(ck["optimizer"]["state"][0]["exp_avg"].norm())) < 1e-6


def test_decode_strategies_and_prompts_match_the_reference(tmp_path):
    """The unmodified reference ``policy`` / ``mcts`` / ``adaptive-mcts`` strategies (python-chess
    replaced by a stand-in over this repository's move generator) against this framework's
    sequential and batched strategies, same weights, fp32 on the CPU: same move distributions,
    think times, resign flags and chosen moves; and the same PGN prompts for the completion baseline."""
    import random

    from allie_b200.chess import Board
    from allie_b200.data import Game, UCITokenizer
    from allie_b200.evaluation.chess_llm import ChessLLM
    from allie_b200.models import initialize_model
    from allie_b200.search import DECODE_STRATEGIES

    shape = dict(n_layer=2, n_embd=64, n_head=2, n_positions=128, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    tok_kw = dict(max_length=128, vocab_size_multiple_of=128)
    tok = UCITokenizer(**tok_kw)
    torch.manual_seed(4)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **shape).eval()
    with torch.no_grad():                  # livelier heads than a fresh init: values and times that matter
        for n, p in model.named_parameters():
            if "head" in n or "wte" in n:
                p.mul_(8.0)
    rng = random.Random(5)
    lines = [[], "f2f3 e7e5 g2g4".split(), "e2e4 e7e5 g1f3 b8c6 f1b5 a7a6".split()]
    b = Board()
    for _ in range(47):
        b.push_uci(rng.choice(b.legal_moves_uci()))
    lines.append(list(b.move_stack))       # long enough for the prompt's movetext to wrap
    games = [Game("180+0", 1500 + 300 * i, 2300, None, False, mv, [3] * len(mv)) for i, mv in enumerate(lines)]
    strategies = [("policy", {}), ("mcts", {"n_sims": 24}), ("mcts", {"n_sims": 9, "kl_reg_solution": False}),
                  ("adaptive-mcts", {"mean_n_sims": 12}), ("action-value", {"batch_size": 7})]
    from test_trainer_cpu import _random_games, _row

    rows = [_row(g) for g in _random_games(4, seed=8)]
    rows[1]["termination"] = "Time forfeit"                # not a resignation
    torch.save({"model": model.state_dict(), "tokenizer": tok_kw, "shape": shape,
                "games": [g.to_dict() for g in games], "strategies": strategies, "rows": rows},
               tmp_path / "ours.pt")
    res = subprocess.run([sys.executable, os.path.join(HERE, "reference_worker.py"), str(tmp_path), "decode"],
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    ref = torch.load(tmp_path / "ref_decode.pt", weights_only=False)

    for name, kwargs in strategies:
        want = ref["decode"][f"{name}:{sorted(kwargs.items())}"]
        for variant in (name, name + "-batched"):
            if variant not in DECODE_STRATEGIES:
                continue
            extra = {"n_trees": 3, "anc_max": 64} if variant.endswith("mcts-batched") else {}
            strat = DECODE_STRATEGIES[variant](model, tok, sample=False, device="cpu", **kwargs, **extra)
            for g, row in zip(games, want["rows"]):
                assert g.legal_moves == row["legal"]
                s = strat.score_full(g, g.legal_moves)
                assert torch.allclose(s.legal_move_probabilities, row["probs"], atol=2e-4), (variant, kwargs, g.moves)
                assert abs(s.think_time - row["think_time"]) < 1e-3 and bool(s.resigned) == bool(row["resigned"])
                assert strat.decode_full(g).move == row["move"], (variant, kwargs, g.moves)
            if "total_rollouts" in want["stats"]:
                assert strat.run_stats()["total_rollouts"] == want["stats"]["total_rollouts"]
    # rating-based sampling: arg-max for a 2200+ side after more than 8 plies, else a draw from the
    # distribution - the same draw as the reference's when the generator starts from the same seed
    for variant in ("policy", "policy-batched"):
        strat = DECODE_STRATEGIES[variant](model, tok, sample="rating-based", device="cpu")
        for i, g in enumerate(games):
            torch.manual_seed(100 + i)
            move = strat.decode_batch([g])[0].move if variant.endswith("batched") else strat.decode_full(g).move
            assert move == ref["sampled"][i], (variant, i)
    llm = ChessLLM(None)
    for g, prompt in zip(games, ref["prompts"]):
        assert llm.get_query_pgn(g.board) == prompt
    assert "\n" in ref["prompts"][3].split("\n\n")[1]     # the long game's movetext did wrap
    # the evaluation CLI's quick mode: the same per-game records as the reference's evaluate_quick
    from allie_b200.evaluation.evaluate import evaluate_quick

    for variant in ("policy", "policy-batched"):
        strat = DECODE_STRATEGIES[variant](model, tok, sample=False, device="cpu")
        mine = evaluate_quick(strat, rows, batch_size=5)["games"]
        assert len(mine) == len(ref["quick"]) == 4
        for a, b_ in zip(mine, ref["quick"]):
            for key in ("model-move", "human-move", "top-move-legal", "human-resigned", "model-resigned"):
                assert list(a[key]) == list(b_[key]), (variant, key)
            for key in ("sampled-move-legal", "model-think-time", "model-white-advantage"):
                assert np.allclose(a[key], b_[key], atol=2e-4), (variant, key)
    assert ref["quick"][0]["human-resigned"][-1] is True and ref["quick"][1]["human-resigned"][-1] is False


def test_training_steps_match_the_reference_trainer(tmp_path):
    """Four optimizer steps (two micro-batches each, warm-up then cosine decay, clipping, two AdamW
    groups) of the reference's own ``Trainer.train()`` and of this trainer's CPU path, from the same
    weights over the same windows: same learning rates, same parameters afterwards."""
    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.train.trainer import Trainer

    os.environ["ALLIE_NO_WANDB"] = "1"
    shape = dict(n_layer=2, n_embd=64, n_head=2, n_positions=64, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    tok_kw = dict(max_length=32, vocab_size_multiple_of=128)
    hyper = dict(batch_size=3, gradient_accumulation_steps=2, lr=2e-3, min_lr=2e-4, weight_decay=0.05, beta1=0.9,
                 beta2=0.95, grad_clip=0.5, warmup_iters=2, decay_iters=5, max_iters=3)
    tok = UCITokenizer(**tok_kw)
    rng = np.random.default_rng(9)
    n_batches = 2 * 4 + 1                                  # the reference draws one batch ahead
    windows = (rng.integers(0, 1968, size=(n_batches, 3, 32)).astype(np.uint32)
               | (rng.integers(0, 40, size=(n_batches, 3, 32)).astype(np.uint32) << 16)
               | (rng.integers(0, 3, size=(n_batches, 3, 1)).astype(np.uint32) << 14))
    windows[:, :, 0] = len(tok) + 1400
    windows[:, :, 1] = len(tok) + 1900
    torch.manual_seed(2)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **shape)
    from test_trainer_cpu import _random_games, _row

    val = [_row(g) for g in _random_games(7, seed=3)]      # 7 games, batch size 3: a ragged last batch
    torch.save({"model": model.state_dict(), "tokenizer": tok_kw, "shape": shape, "trainer": hyper,
                "windows": windows.astype(np.int64), "val": val}, tmp_path / "ours.pt")
    res = subprocess.run([sys.executable, os.path.join(HERE, "reference_worker.py"), str(tmp_path), "train"],
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    ref = torch.load(tmp_path / "ref_train.pt", weights_only=False)

    tr = Trainer(Config({"trainer_config": {}}), output_dir=str(tmp_path / "run"), device="cpu", eval_interval=0,
                 log_interval=-1, save_interval=0, use_wandb=False, **hyper)
    tr.setup_dataloaders(tok, np.zeros(4 * 32, dtype=np.uint32), val, [])
    tr.setup_model(model)
    lrs = []
    for step in range(4):
        lrs.append(tr.get_lr())
        wins = [torch.from_numpy(windows[2 * step + ms].view(np.int32).copy()) for ms in range(2)]
        tr.train_step(wins)
        tr.iter_num += 1
    assert len(ref["lrs"]) == 4 and np.allclose(lrs, ref["lrs"], rtol=1e-12, atol=0)
    assert lrs[0] == 0.0 and lrs[2] == 2e-3 and lrs[3] < lrs[2]
    ours = model.state_dict()
    assert set(ours) == set(ref["params"])
    worst = max((ours[k].float() - v.float()).abs().max().item() for k, v in ref["params"].items())
    assert worst < 2e-5, worst
    got_val = tr.validate()                                # mean over batches of the per-batch losses
    assert set(got_val) == set(ref["val"]) == {"val/lm_loss", "val/value_loss", "val/time_loss", "val/loss"}
    for k, v in ref["val"].items():
        assert abs(got_val[k] - v) < 1e-4 * max(1.0, abs(v)), (k, got_val[k], v)
    # the reverse direction: the checkpoint the reference trainer wrote resumes this trainer
    torch.manual_seed(99)
    fresh = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, **shape)
    tr2 = Trainer(Config({"trainer_config": {}}), output_dir=str(tmp_path / "ref_run"), device="cpu", eval_interval=0,
                  log_interval=-1, save_interval=0, use_wandb=False, **hyper)
    tr2.setup_dataloaders(tok, np.zeros(4 * 32, dtype=np.uint32), [], [])
    tr2.setup_model(fresh)                                 # picks up ref_run/last.pt
    ref_ck = torch.load(tmp_path / "ref_run" / "last.pt", weights_only=False)
    assert tr2.iter_num == ref_ck["iter_num"] == 4
    for k, v in fresh.state_dict().items():
        assert torch.equal(v, ref_ck["model"][k]), k
    st = tr2.optimizer.state_dict()["state"]
    assert len(st) == len(ref_ck["optimizer"]["state"]) > 0
    assert torch.equal(st[0]["exp_avg"], ref_ck["optimizer"]["state"][0]["exp_avg"])
    moved = (ours["model.model.transformer.h.0.mlp.c_fc.weight"] - torch.load(tmp_path / "ours.pt", weights_only=False)["model"]["model.model.transformer.h.0.mlp.c_fc.weight"]).abs().max().item()
    assert moved > 1e-4                                    # the steps did change the weights
