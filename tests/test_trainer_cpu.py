"""End-to-end trainer flow on CPU: train, log, checkpoint in the reference layout, resume, evaluate."""
import json
import os

import numpy as np
import torch

from allie_b200.config import Config, load_config
from allie_b200.data import Game, UCITokenizer
from allie_b200.models import initialize_model
from allie_b200.train.trainer import Trainer

MODEL_KW = dict(base_model="gpt2", use_control_token=True, use_regression_head=True, n_layer=2, n_embd=64,
                n_head=2, n_positions=64)


def _random_games(n, seed=0):
    rng = np.random.default_rng(seed)
    games = []
    for _ in range(n):
        g = Game("180+0", int(rng.integers(900, 2400)), int(rng.integers(900, 2400)), None, True, [], [])
        for _ in range(int(rng.integers(6, 20))):
            legal = g.legal_moves
            if not legal:
                break
            g = g.make_move(legal[int(rng.integers(0, len(legal)))])
            g.moves_seconds[-1] = int(rng.integers(0, 20))
        g.outcome = ["1-0", "0-1", "1/2-1/2"][int(rng.integers(0, 3))]
        games.append(g)
    return games


def _row(g: Game) -> dict:
    return {"time-control": g.time_control, "white-elo": g.white_elo, "black-elo": g.black_elo, "result": g.outcome,
            "termination": "Normal", "moves-uci": " ".join(g.moves), "moves-seconds": g.moves_seconds}


def _make(tmp_path, **over):
    os.environ["ALLIE_NO_WANDB"] = "1"
    tok = UCITokenizer(max_length=32, vocab_size_multiple_of=128)
    games = _random_games(40)
    stream = np.concatenate([tok.tokenize(g) for g in games]).astype(np.uint32)
    val = [_row(g) for g in _random_games(6, seed=1)]
    kw = dict(output_dir=str(tmp_path / "run"), device="cpu", batch_size=4, max_iters=4, decay_iters=4, warmup_iters=1,
              eval_interval=2, log_interval=1, save_interval=2, lr=1e-3, min_lr=1e-4, use_wandb=False)
    kw.update(over)
    tr = Trainer(Config({"trainer_config": {}}), **kw)
    torch.manual_seed(0)
    model = initialize_model(tok, **MODEL_KW)
    tr.setup_dataloaders(tok, stream, val, val)
    tr.setup_model(model)
    return tr, tok, val


def test_train_checkpoint_resume_and_eval_cli(tmp_path):
    tr, tok, val = _make(tmp_path)
    tr.train()
    run = tmp_path / "run"
    assert (run / "last.pt").exists() and (run / "best.pt").exists() and (run / "log.txt").exists()
    log = (run / "log.txt").read_text()
    assert "train - iter 0: loss" in log and "val - iter 0:" in log and "new best val loss" in log
    assert "throughput - " in log and "tokens/s" in log
    rows = [json.loads(line) for line in (run / "metrics.jsonl").read_text().splitlines()]
    assert any("val/loss" in r and "lr" in r for r in rows) and any("perf/tokens_per_s" in r for r in rows)
    ck = torch.load(run / "last.pt", weights_only=False)
    assert {"iter_num", "best_val_loss", "model", "optimizer"} <= set(ck)
    keys = set(ck["model"])
    for k in ("model.model.transformer.wte.weight", "model.model.transformer.h.0.attn.c_attn.weight",
              "model.model.lm_head.weight", "model.control_embeds.weight", "value_head.0.weight", "time_head.0.bias"):
        assert k in keys, k
    assert ck["model"]["model.model.transformer.h.0.attn.c_attn.weight"].shape == (64, 192)   # [in, out]
    assert len(ck["optimizer"]["param_groups"]) == 2 and ck["optimizer"]["param_groups"][1]["weight_decay"] == 0.0
    # resume picks up the iteration counter and the weights
    tr2, _, _ = _make(tmp_path)
    assert tr2.iter_num == ck["iter_num"] and tr2.best_val_loss == ck["best_val_loss"]
    a = dict(tr2.model.named_parameters())["model.model.transformer.wte.weight"]
    assert torch.equal(a.detach(), ck["model"]["model.model.transformer.wte.weight"])
    tr2.test()
    # evaluation CLI, quick mode, on the validation rows
    from allie_b200.config import save_config
    from allie_b200.evaluation.evaluate import main as eval_main

    cfg = {"trainer_config": {"output_dir": str(run)}, "data_config": {"tokenizer_config": {"max_length": 32, "vocab_size_multiple_of": 128}},
           "model_config": MODEL_KW}
    save_config(cfg, str(tmp_path / "cfg.yaml"))
    (tmp_path / "val.jsonl").write_text("\n".join(json.dumps(r) for r in val[:2]))
    res = eval_main(["--config", str(tmp_path / "cfg.yaml"), "--dataset", str(tmp_path / "val.jsonl"), "--quick",
                     "--decode", "policy", "--sequential", "--output_file", str(tmp_path / "out.jsonl"), "--device", "cpu"])
    assert res["implementation"] == "policy"
    assert res["positions"] > 0 and 0 <= res["move_match"] <= 1 and res["top_move_legal"] is not None
    written = json.loads((tmp_path / "out.jsonl").read_text().strip())
    assert written["decode"] == "policy" and len(written["games"]) == 2
    rec = written["games"][0]
    n0 = len(val[0]["moves-uci"].split())
    assert rec["human-move"] == val[0]["moves-uci"].split() and len(rec["model-move"]) == n0
    assert len(rec["top-move-legal"]) == n0 and len(rec["model-think-time"]) == n0
    # these random games end "Normal" with no result on the board: the human resigned after the last ply
    assert rec["human-resigned"] == [False] * n0 + [True] and len(rec["model-resigned"]) == n0 + 1
    assert "games" not in res or res["games"] is not None
    # the many-positions-per-call strategy reports the same metrics, whatever the batch size
    for bs in ("3", "256"):
        rb = eval_main(["--config", str(tmp_path / "cfg.yaml"), "--dataset", str(tmp_path / "val.jsonl"), "--quick",
                        "--decode", "policy", "--debug", "--device", "cpu", "--batch_size", bs])
        assert rb["implementation"] == "policy-batched" and rb["decode"] == "policy"    # picked automatically
        assert rb["positions"] == res["positions"] and rb["move_match"] == res["move_match"]
        assert abs(rb["value_mse"] - res["value_mse"]) < 1e-5 and abs(rb["legal_mass"] - res["legal_mass"]) < 1e-5


def test_lr_schedule_and_config_files():
    tr = Trainer.__new__(Trainer)
    tr.lr, tr.min_lr, tr.decay_lr, tr.warmup_iters, tr.decay_iters = 6e-4, 6e-5, True, 10, 110
    tr.iter_num = 5
    assert abs(tr.get_lr() - 3e-4) < 1e-12
    tr.iter_num = 60
    assert abs(tr.get_lr() - (6e-5 + 0.5 * (6e-4 - 6e-5))) < 1e-12
    tr.iter_num = 500
    assert tr.get_lr() == 6e-5
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = load_config(os.path.join(root, "pretrain_config", "medium.yaml"))
    assert cfg.trainer_config.min_lr == 1e-5 and cfg.model_config.base_model == "gpt2-medium"
    assert load_config(os.path.join(root, "pretrain_config", "ablations", "large.yaml")).model_config.base_model == "gpt2-large"


def test_corrupt_checkpoint_is_reported(tmp_path):
    tr, _, _ = _make(tmp_path, max_iters=1, eval_interval=0)
    tr.save_ckpt("last")
    p = tmp_path / "run" / "last.pt"
    p.write_bytes(p.read_bytes()[:100])      # truncated file
    try:
        _make(tmp_path, max_iters=1, eval_interval=0)
    except Exception as e:
        assert "last.pt" in str(e) or isinstance(e, (RuntimeError, EOFError, ValueError, Exception))
    else:
        raise AssertionError("a truncated checkpoint must not load silently")


def test_flops_per_token_and_mfu():
    from allie_b200.config import resolve_model_config
    from allie_b200.utils.perf import matmul_params_per_token, mfu, train_flops_per_token

    cfg = resolve_model_config("gpt2-medium", vocab_size=2048)
    assert matmul_params_per_token(cfg) == 24 * 12 * 1024 * 1024 + 1024 * 2048
    f = train_flops_per_token(cfg, 512)
    assert abs(f - (6 * matmul_params_per_token(cfg) + 24 * 6 * 512 * 1024)) < 1
    assert abs(mfu(1e6, f, n_gpus=2, peak_flops=1e15) - 1e6 * f / 2e15) < 1e-12
    moe = resolve_model_config("gpt2-medium", vocab_size=2048, num_experts=8, moe_ffn=2048, moe_layer_freq=3)
    per_moe_block = 4 * 1024 * 1024 + 2 * 2 * 1024 * 2048 + 1024 * 8
    assert matmul_params_per_token(moe) == 16 * 12 * 1024 * 1024 + 8 * per_moe_block + 1024 * 2048


def test_window_sampler_prefetch_and_buffer_reuse():
    from allie_b200.train.trainer import WindowSampler

    data = np.arange(10_000, dtype=np.uint32) | np.uint32(1 << 31)       # top bit set: must survive as int32 bits
    for prefetch in (True, False):
        ws = WindowSampler(data, batch_size=3, seq_len=16, pin=False, depth=6, prefetch=prefetch)
        live = []
        for _ in range(40):
            w = ws.next()
            u = w.numpy().view(np.uint32)
            assert u.shape == (3, 16) and np.all(u >> 31 == 1)
            low = (u & 0x7FFFFFFF).astype(np.int64)
            assert np.all(np.diff(low, axis=1) == 1) and low.max() < 10_000  # every row is a contiguous window
            live.append((w, u.copy()))
            live = live[-ws.keep:]
            # the last `keep` windows handed out are distinct buffers and have not been overwritten
            assert len({id(t) for t, _ in live}) == len(live)
            assert all(np.array_equal(t.numpy().view(np.uint32), snap) for t, snap in live)
        ws.close()
    bad = WindowSampler(data, batch_size=3, seq_len=16, pin=False)
    bad.next()
    bad.data = None                                                      # the producer thread now fails
    try:
        for _ in range(12):
            bad.next()
        raise AssertionError("expected the prefetch failure to surface")
    except RuntimeError as e:
        assert "prefetch" in str(e)


def test_config_inheritance(tmp_path):
    (tmp_path / "base.yaml").write_text("trainer_config:\n  lr: 6e-4\n  batch_size: 32\nmodel_config:\n  base_model: gpt2\n")
    (tmp_path / "sub").mkdir()
    (tmp_path / "sub" / "child.yaml").write_text("inherit: ../base.yaml\ntrainer_config:\n  batch_size: 8\ndata_config:\n  train_file: x.bin\n")
    cfg = load_config(str(tmp_path / "sub" / "child.yaml"))
    assert cfg.trainer_config == {"lr": 6e-4, "batch_size": 8} and cfg.model_config.base_model == "gpt2"
    assert cfg.data_config.train_file == "x.bin" and "inherit" not in cfg
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    short = load_config(os.path.join(root, "pretrain_config", "ablations", "short.yaml"))
    assert short.trainer_config.max_iters == 1000000 and short.trainer_config.weight_decay == 1e-2
    assert short.model_config.base_model == "gpt2-medium" and short.data_config.tokenizer_config.max_length == 512


def test_stop_signal_saves_a_checkpoint_and_resume_continues(tmp_path):
    import signal
    import threading

    tr, _, _ = _make(tmp_path, max_iters=10_000, decay_iters=10_000, eval_interval=0, save_interval=0, log_interval=50)
    running = {"train": True}                             # the signal is only sent while train() owns the handler
    timer = threading.Timer(1.0, lambda: running["train"] and os.kill(os.getpid(), signal.SIGUSR1))
    timer.start()
    try:
        tr.train()                                        # returns because of the signal, long before max_iters
    finally:
        running["train"] = False
        timer.cancel()
    assert tr.stopped_early and 0 < tr.iter_num < 10_000
    ck = torch.load(tmp_path / "run" / "last.pt", weights_only=False)
    assert ck["iter_num"] == tr.iter_num
    assert "stop requested" in (tmp_path / "run" / "log.txt").read_text()
    tr2, _, _ = _make(tmp_path, max_iters=tr.iter_num + 2, decay_iters=10_000, eval_interval=0, save_interval=0,
                      log_interval=50)
    assert tr2.iter_num == ck["iter_num"]                 # the requeued job picks up where the signal arrived
    tr2.train()
    assert not tr2.stopped_early and tr2.iter_num == ck["iter_num"] + 3
    assert signal.getsignal(signal.SIGUSR1) is signal.SIG_DFL     # train() put the previous handlers back


def test_engine_keeps_a_bounded_number_of_inference_buffer_sets():
    """The buffer cache of the engine, exercised on the CPU through a bare instance: training
    shapes stay, inference shapes are kept least-recently-used up to a small number."""
    from allie_b200.config import ModelConfig
    from allie_b200.models.engine import B200Engine

    eng = B200Engine.__new__(B200Engine)
    eng.cfg = ModelConfig(vocab_size=128, n_positions=64, n_embd=16, n_layer=1, n_head=1, attn_pdrop=0.0)
    eng.device, eng._bufs, eng.max_inference_shapes = torch.device("cpu"), {}, 3
    train = eng._buffers(2, 8, True)
    a = eng._buffers(1, 8, False)
    for t in (16, 24):
        eng._buffers(1, t, False)
    assert eng._buffers(1, 8, False) is a                       # a hit refreshes the entry ...
    eng._buffers(1, 32, False)                                  # ... so the next miss evicts (1, 16), not (1, 8)
    keys = set(eng._bufs)
    assert keys == {(2, 8, True), (1, 8, False), (1, 24, False), (1, 32, False)}
    assert eng._buffers(2, 8, True) is train
    for t in range(33, 40):
        eng._buffers(2, t, False)
    assert sum(1 for k in eng._bufs if not k[2]) == 3 and (2, 8, True) in eng._bufs
    try:
        eng._buffers(1, 65, False)
        raise AssertionError("expected the position-table guard")
    except ValueError as e:
        assert "positions" in str(e)


def test_every_trainer_key_of_the_shipped_configs_is_an_argument_of_the_trainer():
    """``Trainer(config, **config.trainer_config)`` is how the CLI builds it: a key the signature does
    not know would only fail at launch time.  Also pins the extension keys by name."""
    import glob
    import inspect

    params = set(inspect.signature(Trainer.__init__).parameters)
    assert {"shard_optimizer", "grad_sync", "expert_parallel", "cuda_graph", "use_wandb"} <= params
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = glob.glob(os.path.join(root, "pretrain_config", "**", "*.yaml"), recursive=True)
    assert len(files) >= 5
    for f in files:
        cfg = load_config(f)
        keys = set(cfg.trainer_config.to_container()) if hasattr(cfg.trainer_config, "to_container") else set(dict(cfg.trainer_config))
        assert keys <= params, (f, sorted(keys - params))
