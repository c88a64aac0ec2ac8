"""Runs the unmodified reference package (installed under ``baseline/_ref``, third-party imports it
lacks satisfied from ``baseline/shims``) in a process of its own: loads a state dict written by this
framework into the reference's model with ``strict=True``, collates the given raw windows with the
reference's tokenizer, runs its forward pass, builds its optimizer and loads this framework's
optimizer state into it.  Results go to ``<dir>/ref_out.pt``.

usage: reference_worker.py <dir>      (reads <dir>/ours.pt)
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
    decay, no_decay = partition_model_parameters(model)
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.01}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=1e-3, betas=(0.9, 0.95))
    opt.load_state_dict(blob["optimizer"])
    first = opt.state_dict()["state"][0]
    torch.save({"batch": {k: v for k, v in batch.items()},
                "out": {k: out[k].float() for k in ("logits", "loss", "lm_loss", "value_loss", "time_loss",
                                                    "value_logits", "time_logits")},
                "vocab": len(tok), "ids": {"bos": tok.bos_token_id, "pad": tok.pad_token_id},
                "n_decay": len(decay), "n_no_decay": len(no_decay),
                "opt_step": float(first["step"]), "opt_exp_avg_norm": float(first["exp_avg"].norm())},
               os.path.join(d, "ref_out.pt"))


if __name__ == "__main__":
    main()
