"""Data-parallel trainer: CPU gloo ranks (host logic) and, on a multi-GPU box, the fused NVLink
gradient path against the all_reduce path."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(nproc, out_dir, mode, device, port, extra_env=None, extra_args=()):
    env = dict(os.environ, ALLIE_NO_WANDB="1", **(extra_env or {}))
    env.pop("RANK", None)
    if nproc == 1:
        cmd = [sys.executable, os.path.join(HERE, "ddp_worker.py"), str(out_dir), mode, device, *extra_args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port),
               os.path.join(HERE, "ddp_worker.py"), str(out_dir), mode, device, *extra_args]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


def test_cpu_gloo_two_ranks_match_single(tmp_path):
    """2 gloo ranks, each with half of every micro-batch, must land on the single-process parameters
    of a run whose gradients are averaged the same way."""
    _launch(2, tmp_path, "collective", "cpu", 29611)
    a = torch.load(tmp_path / "params_collective_0.pt")
    b = torch.load(tmp_path / "params_collective_1.pt")
    assert torch.equal(a["params"], b["params"]), "ranks diverged"
    assert all(l == l for l in a["losses"])
    log = (tmp_path / "run_collective" / "log.txt").read_text()
    assert "throughput - 500 tokens/s, 2000.0 ms/step (max over 2 rank(s))" in log


def test_cpu_gloo_two_ranks_with_moe_layers_stay_in_step(tmp_path):
    """The MoE model (all experts on every rank on the CPU path) under 2 gloo ranks: router, expert
    and dense gradients are all averaged, so the ranks end on identical parameters."""
    _launch(2, tmp_path, "collective", "cpu", 29612, extra_args=("moe",))
    a = torch.load(tmp_path / "params_collective_0.pt")
    b = torch.load(tmp_path / "params_collective_1.pt")
    assert torch.equal(a["params"], b["params"]), "ranks diverged"
    assert all(l == l for l in a["losses"])


@pytest.mark.gpu
def test_fused_nvlink_path_matches_all_reduce(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    n = 2
    _launch(n, tmp_path, "collective", "cuda", 29621)
    _launch(n, tmp_path, "fused", "cuda", 29622, {"ALLIE_NVL_MULTIMEM": "0"})
    ref = torch.load(tmp_path / "params_collective_0.pt")
    for r in range(n):
        got = torch.load(tmp_path / f"params_fused_{r}.pt")
        assert got["fused"] and not got["multimem"]
        d = (got["params"] - ref["params"]).abs()
        # a differently ordered gradient sum can flip the sign of a near-zero Adam step (2*lr)
        assert d.max().item() < 3 * 2e-3 and d.mean().item() < 2e-5, (d.max().item(), d.mean().item())
    os.rename(tmp_path / "params_fused_0.pt", tmp_path / "params_p2p_0.pt")
    _launch(n, tmp_path, "fused", "cuda", 29623, {"ALLIE_NVL_MULTIMEM": "1"})
    got = torch.load(tmp_path / "params_fused_0.pt")
    p2p = torch.load(tmp_path / "params_p2p_0.pt")
    d = (got["params"] - p2p["params"]).abs()
    assert d.max().item() < 3 * 2e-3 and d.mean().item() < 2e-5, (d.max().item(), d.mean().item(), got["multimem"])


@pytest.mark.gpu
def test_expert_parallel_two_ranks_match_single_rank(tmp_path):
    """MoE model: 2 ranks (each owning half of the experts, tokens exchanged through the peer-memory
    dispatch/combine kernels, dense gradients through the fused NVLink path) must land on the
    parameters of a single-rank run over the same global batch."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    one, two = tmp_path / "one", tmp_path / "two"
    one.mkdir(); two.mkdir()
    _launch(1, one, "collective", "cuda", 29631, extra_args=("moe",))
    _launch(2, two, "fused", "cuda", 29632, {"ALLIE_NVL_MULTIMEM": "0"}, extra_args=("moe",))
    ref = torch.load(one / "params_collective_0.pt")["named"]
    for r in range(2):
        got = torch.load(two / f"params_fused_{r}.pt")
        assert got["fused"]
        for name, p in got["named"].items():
            want = ref[name]
            if p.shape != want.shape:          # rank-local expert shard
                El = p.shape[0]
                want = want[r * El:(r + 1) * El]
            d = (p - want).abs()
            assert d.max().item() < 3 * 2e-3 and d.mean().item() < 2e-4, (name, r, d.max().item(), d.mean().item())
        assert got["reload_ok"] is True
    # the two-rank checkpoint stores whole expert banks, laid out like the single-rank file
    ck1 = torch.load(one / "run_collective" / "last.pt", weights_only=False)
    ck2 = torch.load(two / "run_fused" / "last.pt", weights_only=False)
    assert ck1["model"].keys() == ck2["model"].keys()
    for k, v in ck1["model"].items():
        assert ck2["model"][k].shape == v.shape, k
        d = (ck2["model"][k].float() - v.float()).abs()
        assert d.max().item() < 3 * 2e-3, (k, d.max().item())
    for i, st in ck1["optimizer"]["state"].items():
        assert ck2["optimizer"]["state"][i]["exp_avg"].shape == st["exp_avg"].shape, i


@pytest.mark.gpu
def test_fused_path_survives_a_slow_rank_zero_in_validate_and_save(tmp_path):
    """Trainer.train() on 2 GPUs with validation and checkpoints every other iteration, rank 0's
    evaluation slowed down on the host by more than the gradient kernels' wait limit: no device
    wait runs out (the status word stays clean), the ranks end on identical parameters, and the
    checkpoint rank 0 wrote holds complete fp32 weights and Adam moments."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _launch(2, tmp_path, "fused", "cuda", 29641, {"ALLIE_NVL_MULTIMEM": "0"}, extra_args=("loop",))
    a = torch.load(tmp_path / "params_fused_0.pt")
    b = torch.load(tmp_path / "params_fused_1.pt")
    assert a["fused"] and b["fused"] and a["buckets"] == 3
    assert torch.equal(a["params"], b["params"]), (a["params"] - b["params"]).abs().max()
    ck = torch.load(tmp_path / "run_fused" / "last.pt", weights_only=False)
    assert ck["iter_num"] == 4
    st = ck["optimizer"]["state"]
    assert len(st) == len(ck["optimizer"]["param_groups"][0]["params"]) + len(ck["optimizer"]["param_groups"][1]["params"])
    # every weight matrix is cut between the two ranks somewhere: its gathered moments must be
    # alive over its whole extent, not only in the part rank 0 owns
    decayed = ck["optimizer"]["param_groups"][0]["params"]
    big = [st[i]["exp_avg_sq"] for i in decayed if st[i]["exp_avg_sq"].numel() >= 128 * 128]
    assert len(big) >= 12
    assert all(float((v > 0).float().mean()) > 0.9 for v in big)
    assert (tmp_path / "run_fused" / "best.pt").exists()


def test_trainer_loop_with_eval_and_save_under_two_gloo_ranks(tmp_path):
    """The same loop on CPU gloo ranks (host logic of the collective validate / save path)."""
    _launch(2, tmp_path, "collective", "cpu", 29642, extra_args=("loop",))
    a = torch.load(tmp_path / "params_collective_0.pt")
    b = torch.load(tmp_path / "params_collective_1.pt")
    assert torch.equal(a["params"], b["params"]) and a["iter_num"] == b["iter_num"] == 6
    assert (tmp_path / "run_collective" / "last.pt").exists() and (tmp_path / "run_collective" / "best.pt").exists()


def test_shard_bounds_tile_the_arena():
    from allie_b200.parallel.nvl import shard_bounds

    for n in (0, 1, 63, 64, 65, 1000, 4096, 354_871_296, 354_871_297):
        for world in (1, 2, 3, 4, 8):
            end = 0
            for rank in range(world):
                off, length = shard_bounds(n, world, rank)
                assert off == end and off % 64 == 0 or length == 0, (n, world, rank, off, length)
                assert length >= 0
                end = off + length if length else end
            assert end == n, (n, world, end)
            sizes = [shard_bounds(n, world, r)[1] for r in range(world)]
            assert max(sizes) <= -(-n // world) + 63                    # nobody owns much more than 1/world


def test_evaluation_cli_under_two_ranks_matches_one_process(tmp_path):
    """The evaluation CLI under torchrun splits the games over the ranks and rank 0 merges the
    records: the written line equals the single-process one."""
    import json

    from allie_b200.config import save_config
    from allie_b200.etl.dataset import random_games

    cfg = {"trainer_config": {"output_dir": str(tmp_path / "run")},
           "data_config": {"tokenizer_config": {"max_length": 64, "vocab_size_multiple_of": 128}},
           "model_config": dict(base_model="gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                                n_embd=32, n_head=1, n_positions=64)}
    save_config(cfg, str(tmp_path / "cfg.yaml"))
    random_games(str(tmp_path / "games.jsonl"), n=5, max_plies=14, seed=4)
    # both runs need the same weights: a random-init model saved as the checkpoint they load
    import torch as _torch

    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model

    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    _torch.manual_seed(0)
    model = initialize_model(tok, **cfg["model_config"])
    _torch.save({"model": model.state_dict()}, tmp_path / "w.pt")
    common = ["-m", "allie_b200.evaluation.evaluate", "--config", str(tmp_path / "cfg.yaml"), "--dataset",
              str(tmp_path / "games.jsonl"), "--quick", "--decode", "policy-batched", "--device", "cpu",
              "--checkpoint", str(tmp_path / "w.pt")]
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE))
    env.pop("RANK", None)
    one = subprocess.run([sys.executable, *common, "--output_file", str(tmp_path / "one.jsonl")], env=env,
                         capture_output=True, text=True, timeout=600)
    assert one.returncode == 0, one.stderr[-3000:]
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29631", *common, "--output_file",
                          str(tmp_path / "two.jsonl")], env=env, capture_output=True, text=True, timeout=600)
    assert two.returncode == 0, two.stderr[-3000:]
    a = json.loads((tmp_path / "one.jsonl").read_text())
    lines = (tmp_path / "two.jsonl").read_text().splitlines()
    assert len(lines) == 1                                   # only rank 0 writes
    b = json.loads(lines[0])
    assert len(a["games"]) == len(b["games"]) == 5
    for ga, gb in zip(a["games"], b["games"]):               # same games in the same order
        for k in ("moves-uci", "model-move", "human-move", "top-move-legal", "human-resigned", "model-resigned"):
            assert ga[k] == gb[k], k
        for k in ("model-think-time", "model-white-advantage", "sampled-move-legal"):
            # the two runs batch the positions differently: the last bits of a float may differ
            assert len(ga[k]) == len(gb[k]) and all(abs(x - y) < 1e-4 for x, y in zip(ga[k], gb[k])), k
    for k in ("positions", "move_match", "top_move_legal", "resign_rate"):
        assert a[k] == b[k], k
    assert abs(a["value_mse"] - b["value_mse"]) < 1e-6
