"""Phase tracer: counts and times on the CPU path, and the trainer brackets its step phases."""
import time

import numpy as np

from allie_b200.utils.trace import PhaseTracer


def test_tracer_accumulates_and_resets():
    tr = PhaseTracer(enabled=True, device="cpu")
    for _ in range(3):
        with tr.phase("a"):
            time.sleep(0.002)
    with tr.phase("b"):
        pass
    out = tr.summary()
    assert out["a"]["count"] == 3 and out["a"]["ms"] >= 5.0
    assert out["b"]["count"] == 1
    assert tr.summary() == {}


def test_disabled_tracer_records_nothing():
    tr = PhaseTracer(enabled=False, device="cpu")
    with tr.phase("a"):
        pass
    assert tr.summary() == {}


def test_trainer_step_reports_its_phases(tmp_path, monkeypatch):
    monkeypatch.setenv("ALLIE_TRACE", "1")
    monkeypatch.setenv("ALLIE_NO_WANDB", "1")
    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.train.trainer import Trainer

    T = 32
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    tr = Trainer(Config({}), output_dir=str(tmp_path), device="cpu", batch_size=2, gradient_accumulation_steps=2,
                 lr=1e-3, min_lr=1e-4, warmup_iters=0, decay_iters=10, max_iters=2, eval_interval=0,
                 log_interval=-1, save_interval=0, use_wandb=False)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=2, n_positions=T)
    rng = np.random.default_rng(0)
    stream = (rng.integers(0, 1968, size=4096).astype(np.uint32) | (rng.integers(1, 20, size=4096).astype(np.uint32) << 16))
    tr.setup_dataloaders(tok, stream, [], [])
    tr.setup_model(model)
    assert tr.tracer.enabled
    tr.train_step()
    out = tr.tracer.summary()
    assert out["data"]["count"] == 2 and out["forward_backward"]["count"] == 2
    assert out["grad_sync_optimizer"]["count"] == 1 and out["forward_backward"]["ms"] > 0
