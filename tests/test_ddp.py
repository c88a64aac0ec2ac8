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
