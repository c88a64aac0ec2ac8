"""The trainer loop on the sm_100a engine: train, validate, log throughput, checkpoint in the
reference layout, resume (GPU)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_train_loop_checkpoint_and_resume_on_engine(tmp_path):
    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.ops import _lib
    from allie_b200.train.trainer import Trainer
    from test_trainer_cpu import _random_games, _row

    os.environ["ALLIE_NO_WANDB"] = "1"
    tok = UCITokenizer(max_length=128, vocab_size_multiple_of=128)
    stream = np.concatenate([tok.tokenize(g) for g in _random_games(60)]).astype(np.uint32)
    val = [_row(g) for g in _random_games(6, seed=1)]

    def make():
        tr = Trainer(Config({"trainer_config": {}}), output_dir=str(tmp_path / "run"), device="cuda", batch_size=4,
                     max_iters=4, decay_iters=4, warmup_iters=1, eval_interval=2, log_interval=1, save_interval=2,
                     lr=1e-3, min_lr=1e-4, use_wandb=False)
        torch.manual_seed(0)
        model = initialize_model(tok, base_model="gpt2", use_control_token=True, use_regression_head=True,
                                 n_layer=2, n_embd=128, n_head=2, n_positions=128)
        tr.setup_dataloaders(tok, stream, val, val)
        tr.setup_model(model)
        return tr

    tr = make()
    assert tr.engine is not None
    tr.train()
    torch.cuda.synchronize()
    _lib.check_status()
    log = (tmp_path / "run" / "log.txt").read_text()
    assert "train - iter 0: loss" in log and "val - iter 0:" in log
    assert "throughput - " in log and "MFU" in log
    ck = torch.load(tmp_path / "run" / "last.pt", weights_only=False)
    assert {"iter_num", "best_val_loss", "model", "optimizer"} <= set(ck)
    assert ck["model"]["model.model.transformer.h.0.attn.c_attn.weight"].shape == (128, 384)
    assert all(torch.isfinite(v.float()).all() for v in ck["model"].values())
    tr2 = make()
    assert tr2.iter_num == ck["iter_num"]
    got = dict(tr2.model.named_parameters())["model.model.transformer.wte.weight"].detach().cpu()
    assert torch.equal(got, ck["model"]["model.model.transformer.wte.weight"])
    tr2.test()
    torch.cuda.synchronize()
    _lib.check_status()
