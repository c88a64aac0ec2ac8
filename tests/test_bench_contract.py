"""Host-side pieces of the benchmark scripts: the synthetic token stream has the packed layout of
real data, the clock sampler degrades cleanly without nvidia-smi, the model table is consistent (CPU)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402


def test_synthetic_stream_layout():
    from allie_b200.data import UCITokenizer

    tok = UCITokenizer(max_length=512, vocab_size_multiple_of=128)
    w = bench.synthetic_stream(8 * 512, len(tok), 512, seed=1)
    assert w.dtype == np.uint32 and w.shape == (8 * 512,)
    rows = w.reshape(8, 512)
    ids = rows & 0x3FFF
    assert np.all(ids[:, :2] >= len(tok)) and np.all(ids[:, :2] < len(tok) + 3000)        # two ELO pseudo-tokens
    assert np.all((ids[:, 2] >= 1968) & (ids[:, 2] < 1992))                               # a time-control token
    assert np.all(ids[:, 3:] < 1968)                                                      # moves
    assert np.all((rows[:, 3:] >> 16) >= 1)                                               # every move carries seconds + 1
    outcome = (rows >> 14) & 3
    assert np.all(outcome == outcome[:, :1]) and outcome.max() <= 2                       # one outcome per window
    batch = tok.pad_and_collate(list(rows[:2]))
    assert batch["input_ids"].shape == (2, 512) and float(batch["attention_mask"].min()) == 1.0
    assert not np.array_equal(w, bench.synthetic_stream(8 * 512, len(tok), 512, seed=2))


def test_clock_sampler_without_nvidia_smi(monkeypatch):
    monkeypatch.setenv("PATH", "")
    s = bench.ClockSampler(0)
    s.start()
    s.mark()
    out = s.stop()
    assert out["sm_mhz"] is None and out["reasons"]
    s.rows = [["0", "1500", "1965", "900", "0x4", "Not Active", "Not Active", "Not Active", "Active"],
              ["0", "1700", "1965", "950", "0x4", "Not Active", "Not Active", "Not Active", "Active"],
              ["0", "1600", "1965", "950", "0x0", "Not Active", "Not Active", "Not Active", "Not Active"]]

    class Done:
        def terminate(self): ...
        def wait(self, timeout=None): ...

    s.proc, s.first = Done(), 0
    out = s.stop()
    assert out == {"sm_mhz": 1600.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}


def test_model_table():
    assert bench.MODELS["medium"] is bench.MODEL and bench.MODEL["n_embd"] // bench.MODEL["n_head"] == 64
    large = bench.MODELS["large"]
    assert (large["n_layer"], large["n_embd"], large["n_head"]) == (32, 1280, 20) and large["n_embd"] % 128 == 0
    assert bench.GLOBAL_BATCH % bench.MICRO_BATCH == 0 and bench.GLOBAL_BATCH // bench.MICRO_BATCH == 8


def test_both_arms_share_one_config_dictionary():
    """The two arms of the headline benchmark describe their workload with the same ``config``
    (arm-specific detail goes elsewhere), for every model shape and rank count."""
    for name in bench.MODELS:
        for world in (1, 2, 4, 8):
            ga = bench.GLOBAL_BATCH // (bench.MICRO_BATCH * world)
            cfg = bench.common_config(name, ga, world)
            assert cfg["global_batch"] == 512 and cfg["seq_len"] == 512 and cfg["grad_accum"] * world * 64 == 512
            assert cfg["parallelism"] == f"dp{world}" and "dropout 0.1" in cfg["model"]
    src = open(bench.__file__).read()
    assert src.count('"config": common_config(args.model, ga, world)') == 2


def test_command_dispatcher(capsys, tmp_path):
    from allie_b200.__main__ import COMMANDS, main
    import importlib

    for module, func, _ in COMMANDS.values():
        assert callable(getattr(importlib.import_module(module), func))      # every command resolves
    try:
        main(["--help"])
    except SystemExit as e:
        assert e.code == 0
    assert "stress-test" in capsys.readouterr().out
    try:
        main(["no-such-command"])
    except SystemExit as e:
        assert e.code == 2
    main(["dataset", "random-games", str(tmp_path / "g.jsonl"), "--n", "3"])
    assert len((tmp_path / "g.jsonl").read_text().splitlines()) == 3
