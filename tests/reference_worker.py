"""Runs the unmodified reference package (installed under ``baseline/_ref``, third-party imports it
lacks satisfied from ``baseline/shims``) in a process of its own: loads a state dict written by this
framework into the reference's model with ``strict=True``, collates the given raw windows with the
reference's tokenizer, runs its forward pass, builds its optimizer and loads this framework's
optimizer state into it.  Results go to ``<dir>/ref_out.pt``.

With ``decode`` as second argument it instead runs the reference's decode strategies (policy, MCTS,
adaptive MCTS) on the given games with the given weights and writes their move distributions, think
times and resign flags to ``<dir>/ref_decode.pt``, plus the prompts its PGN prompter builds.

With ``train`` it runs the reference's own ``Trainer.train()`` on the CPU (fp32, no compile) from the
given initial weights over the given sequence of raw windows (its random window iterator is replaced
from outside by a fixed one) and writes the final parameters and the per-step learning rates to
``<dir>/ref_train.pt``.

usage: reference_worker.py <dir> [decode|train]      (reads <dir>/ours.pt)
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

import numpy as np  # noqa: E402
import torch  # noqa: E402


def main():
    from modeling.data import UCITokenizer
    from modeling.model import initialize_model
    from modeling.utils import partition_model_parameters

    d = sys.argv[1]
    blob = torch.load(os.path.join(d, "ours.pt"), weights_only=False)
    tok = UCITokenizer(**blob["tokenizer"])
    torch.manual_seed(0)
    model = initialize_model(tok, os.path.join(ROOT, "baseline", "gpt2-medium"), use_control_token=True,
                             use_regression_head=True, use_pretrained=False, **blob["shape"])
    model.load_state_dict(blob["model"], strict=True)
    model.eval()
    batch = tok.pad_and_collate(list(blob["windows"].astype(np.uint32)))
    with torch.no_grad():
        out = model(**batch)
    from modeling.data import Game

    words, collated = [], []
    for g in blob.get("games", []):
        game = Game(**g)
        for flags in blob["tokenize_flags"]:
            words.append(tok.tokenize(game, **flags).astype(np.int64))
    if blob.get("games"):
        collated = tok.pad_and_collate([Game(**g) for g in blob["games"]])
    decay, no_decay = partition_model_parameters(model)
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=1e-3, betas=(0.9, 0.95))
    opt.load_state_dict(blob["optimizer"])
    first = opt.state_dict()["state"][0]
    from server.utils import SYSTEMS

    systems = {a: (s.port, s.elo, s.algorithm, dict(s.algorithm_config)) for a, s in SYSTEMS.items()}
    torch.save({"batch": {k: v for k, v in batch.items()}, "systems": systems,
                "out": {k: out[k].float() for k in ("logits", "loss", "lm_loss", "value_loss", "time_loss",
                                                    "value_logits", "time_logits")},
                "words": words, "collated_games": collated,
                "vocab": len(tok), "ids": {"bos": tok.bos_token_id, "pad": tok.pad_token_id},
                "n_decay": len(decay), "n_no_decay": len(no_decay),
                "opt_step": float(first["step"]), "opt_exp_avg_norm": float(first["exp_avg"].norm())},
               os.path.join(d, "ref_out.pt"))


def decode():
    import chess
    from evaluation.carlini import ChessLLM
    from evaluation.decode import DECODE_STRATEGIES, ActionValue
    from modeling.data import Game, UCITokenizer
    from modeling.model import initialize_model

    d = sys.argv[1]
    blob = torch.load(os.path.join(d, "ours.pt"), weights_only=False)
    tok = UCITokenizer(**blob["tokenizer"])
    model = initialize_model(tok, os.path.join(ROOT, "baseline", "gpt2-medium"), use_control_token=True,
                             use_regression_head=True, use_pretrained=False, **blob["shape"])
    model.load_state_dict(blob["model"], strict=True)
    model.eval()
    games = [Game(**g) for g in blob["games"]]
    out = {}
    classes = {**DECODE_STRATEGIES, "action-value": ActionValue}      # the reference leaves this one unregistered
    with torch.inference_mode():
        for name, kwargs in blob["strategies"]:
            strat = classes[name](model, tok, sample=False, device="cpu", precision="float32", **kwargs)
            rows = []
            for g in games:
                s = strat.score_full(g, g.legal_moves)
                rows.append({"legal": g.legal_moves, "probs": s.legal_move_probabilities.float().clone(),
                             "think_time": s.think_time, "resigned": s.resigned,
                             "move": strat.decode_full(g).move})
            out[f"{name}:{sorted(kwargs.items())}"] = {"rows": rows, "stats": strat.run_stats()}
    sampled = []
    with torch.inference_mode():
        strat = DECODE_STRATEGIES["policy"](model, tok, sample="rating-based", device="cpu", precision="float32")
        for i, g in enumerate(games):
            torch.manual_seed(100 + i)
            sampled.append(strat.decode_full(g).move)
    quick = None
    if blob.get("rows"):
        import pandas as pd
        from evaluation.evaluate import evaluate_quick

        with torch.inference_mode():
            strat = DECODE_STRATEGIES["policy"](model, tok, sample=False, device="cpu", precision="float32")
            quick = evaluate_quick(strat, pd.DataFrame(blob["rows"]))["games"]
    llm = ChessLLM(None, {"num_lookahead_tokens": 10})
    prompts = []
    for g in games:
        board = chess.Board()
        for mv in g.moves:
            board.push_uci(mv)
        prompts.append(llm.get_query_pgn(board))
    torch.save({"decode": out, "prompts": prompts, "quick": quick, "sampled": sampled}, os.path.join(d, "ref_decode.pt"))


def train():
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("WANDB_SILENT", "true")
    from modeling.data import UCITokenizer
    from modeling.model import initialize_model
    from modeling.trainer import Trainer
    from omegaconf import OmegaConf

    d = sys.argv[1]
    blob = torch.load(os.path.join(d, "ours.pt"), weights_only=False)
    tok = UCITokenizer(**blob["tokenizer"])
    cfg = OmegaConf.create({"trainer_config": {}, "data_config": {}, "model_config": {}})
    trainer = Trainer(cfg, output_dir=os.path.join(d, "ref_run"), device="cpu", dtype="float32", torch_compile=False,
                      eval_interval=0, log_interval=10 ** 9, save_interval=0, **blob["trainer"])
    model = initialize_model(tok, os.path.join(ROOT, "baseline", "gpt2-medium"), use_control_token=True,
                             use_regression_head=True, use_pretrained=False, **blob["shape"])
    model.load_state_dict(blob["model"], strict=True)
    stream = np.zeros(4 * tok.max_length, dtype=np.uint32)
    trainer.setup_dataloaders(tok, stream, blob.get("val", []), [])
    trainer.setup_model(model)
    batches = [tok.pad_and_collate(list(w.astype(np.uint32))) for w in blob["windows"]]
    trainer.train_dataiter = iter(batches)
    lrs = []
    trainer.optimizer.register_step_post_hook(lambda opt, a, k: lrs.append(opt.param_groups[0]["lr"]))
    trainer.train()
    val = trainer.validate() if blob.get("val") else {}
    trainer.save_ckpt("last")                      # the reference's own checkpoint file, for the reverse direction
    torch.save({"params": {k: v.detach().clone() for k, v in trainer.model.state_dict().items()}, "lrs": lrs,
                "val": val},
               os.path.join(d, "ref_train.pt"))


if __name__ == "__main__":
    {"decode": decode, "train": train}.get(sys.argv[2] if len(sys.argv) > 2 else "", main)()
