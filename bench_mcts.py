"""MCTS leaf-evaluation throughput (positions per second) of the medium model.

Workload: `--trees` concurrent search trees (default 256) with `--sims` simulations each (default
400) on one GPU, random-init GPT-2-medium-shaped Allie model in bf16, root positions = random legal
games whose prompts are 1-300 tokens long.  Every leaf evaluation is one KV-cached decode step
(softmax policy over the leaf's legal moves, value, think time).

    python bench_mcts.py                       # batched C++ search + KV-cached sm_100a evaluator
    python bench_mcts.py --impl sequential     # the reference algorithm: one tree at a time, every
                                               # leaf re-encodes its whole game at batch 1
    python bench_mcts.py --impl reference      # the unmodified reference package (baseline/_ref): its own
                                               # model and MCTS strategy, python-chess replaced by a stand-in
    torchrun --nproc-per-node 8 bench_mcts.py --gpus 8   # one independent 256-tree search per GPU
    python bench_mcts.py --ablate              # where the time of one evaluation step goes
    ALLIE_DECODE_PDL=0 python bench_mcts.py --ablate     # the same with ordinary kernel launches
Prints one JSON line (rank 0; with several GPUs the value is the sum of positions over the ranks
divided by the slowest rank's time, and the p50 per-move latency is the median over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def random_games(n, tok, rng, max_tokens=300):
    from allie_b200.data import Game

    games = []
    for i in range(n):
        target = int(rng.integers(0, max_tokens - 3))
        g = Game("180+0", int(rng.integers(800, 2600)), int(rng.integers(800, 2600)), None, False, [], [])
        while len(g.moves) < target:
            legal = g.legal_moves
            if not legal or g.board.is_game_over():
                break
            nxt = g.make_move(legal[int(rng.integers(0, len(legal)))])
            if nxt.board.is_game_over():
                break
            g = nxt
        games.append(g)
    return games


def run_reference(sims: int, positions: int, small: bool, seed: int = 0) -> dict:
    """The reference package as installed under ``baseline/_ref``: its ``initialize_model`` (Hugging
    Face GPT-2 inside its two wrappers, random init), its tokenizer and its ``MCTS`` strategy at
    ``precision="float32"`` as its evaluation CLI runs it (``src/evaluation/decode.py:309-470``,
    ``evaluate.py:249``).  A position = one forward pass of its model."""
    import numpy as np
    import torch

    from allie_b200.data import UCITokenizer as OurTok

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "modeling")):
        return {"unavailable": "baseline/_ref is missing (pip install --target was not run)"}
    for p_ in (os.path.join(ROOT, "baseline", "shims"), ref_dir):
        if p_ not in sys.path:
            sys.path.insert(0, p_)
    try:
        from evaluation.decode import MCTS
        from modeling.data import Game, UCITokenizer
        from modeling.model import initialize_model
    except Exception as e:
        return {"unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    games = random_games(positions, OurTok(max_length=512, vocab_size_multiple_of=128), np.random.default_rng(seed))
    rtok = UCITokenizer(max_length=512, vocab_size_multiple_of=128)
    shape = dict(n_layer=2, n_embd=256, n_head=4) if small else {}
    torch.manual_seed(0)
    model = initialize_model(rtok, os.path.join(ROOT, "baseline", "gpt2-medium"), use_control_token=True,
                             use_regression_head=True, use_pretrained=False, **shape).to(dev).eval()
    calls = [0]
    model.register_forward_hook(lambda *a: calls.__setitem__(0, calls[0] + 1))
    rgames = [Game(**g.to_dict()) for g in games]
    strat = MCTS(model, rtok, sample=False, device=dev, precision="float32", n_sims=sims)
    per_move = []
    with torch.inference_mode():
        strat.score_full(rgames[0], rgames[0].legal_moves)
        if dev == "cuda":
            torch.cuda.synchronize()
        calls[0] = 0
        t0 = time.perf_counter()
        for g in rgames:
            t1 = time.perf_counter()
            strat.score_full(g, g.legal_moves)
            if dev == "cuda":
                torch.cuda.synchronize()
            per_move.append(time.perf_counter() - t1)
        dt = time.perf_counter() - t0
    return {"value": calls[0] / dt, "seconds": dt, "positions": calls[0],
            "p50_move_latency_s": sorted(per_move)[len(per_move) // 2], "dtype": "fp32 (TF32 matmuls)",
            "root_positions": len(rgames),
            "note": "unmodified reference evaluation.decode.MCTS on its own model, one tree at a time, "
                    "batch-1 full re-encode per leaf"}


def build_model(small: bool):
    import torch

    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=512, vocab_size_multiple_of=128)
    shape = dict(n_layer=2, n_embd=256, n_head=4) if small else dict(n_layer=24, n_embd=1024, n_head=16)
    model = initialize_model(tok, "gpt2-medium", use_control_token=True, use_regression_head=True,
                             n_positions=1024, **shape)
    return tok, model


def run_batched(trees: int, sims: int, small: bool, seed: int = 0) -> dict:
    """``trees`` concurrent searches of ``sims`` simulations each on the current GPU: batched C++
    search + KV-cached sm_100a leaf evaluator.  One call of ``search`` plays one move in every
    tree, so its duration is the per-move latency of every game in the batch."""
    import numpy as np
    import torch

    from allie_b200.models.engine import B200Engine
    from allie_b200.ops import _lib
    from allie_b200.search.batched import BatchedMCTS, KVStepEvaluator

    tok, model = build_model(small)
    eng = B200Engine(model, "cuda")
    games = random_games(trees, tok, np.random.default_rng(seed))
    ev = KVStepEvaluator(eng, tok, trees, anc_max=128, legal_max=224, max_prefix=320, max_nodes=sims + 8)
    bm = BatchedMCTS(tok, ev, n_trees=trees, n_sims=sims)
    bm.search(games[:trees], n_sims=8)           # warm-up (graph capture, first launches)
    torch.cuda.synchronize()
    ev.positions = 0
    bm.phase_seconds = {k: 0.0 for k in bm.phase_seconds}
    l0 = _lib.LAUNCHES
    t0 = time.perf_counter()
    res = bm.search(games)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    _lib.check_status()
    return dict(value=ev.positions / dt, seconds=dt, positions=ev.positions, steps=ev.kv.steps,
                moves_per_s=len(games) / dt, p50_move_latency_s=dt, latency_per_move_batch_s=dt,
                gpu_launches=_lib.LAUNCHES - l0, sims_done=int(sum(r.n_sims for r in res)),
                phase_seconds={k: round(v, 4) for k, v in bm.phase_seconds.items()})


def run_ablation(trees: int, small: bool) -> dict:
    """Where the time of one leaf-evaluation step goes: the step's CUDA graph is captured again with
    one kind of kernel left out at a time and timed with CUDA events (50 replays each) on the
    request left behind by a short search."""
    import numpy as np
    import torch

    import allie_b200.search.evaluator as E
    from allie_b200.models.engine import B200Engine
    from allie_b200.ops import _lib, kernels as K
    from allie_b200.search.batched import BatchedMCTS, KVStepEvaluator

    tok, model = build_model(small)
    eng = B200Engine(model, "cuda")
    games = random_games(trees, tok, np.random.default_rng(0))
    ev = KVStepEvaluator(eng, tok, trees, anc_max=128, legal_max=224, max_prefix=320, max_nodes=64)
    BatchedMCTS(tok, ev, n_trees=trees, n_sims=24).search(games, n_sims=24)
    kv = ev.kv
    torch.cuda.synchronize()

    class WithoutAttention:
        def __init__(self, real):
            self.real = real

        def __getattr__(self, name):
            return (lambda *a: 0) if name == "ab_decode_attn" else getattr(self.real, name)

    def timed(patch: dict) -> float:
        saved = {key: getattr(*key) for key in patch}
        for (obj, name), fn in patch.items():
            setattr(obj, name, fn)
        try:
            kv._launch_step()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                kv._launch_step()
        finally:
            for (obj, name), fn in saved.items():
                setattr(obj, name, fn)
        for _ in range(5):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(50):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) / 50 * 1000, 1)

    noop = lambda *a, **k: None
    real_lib = _lib.cuda()
    no_attn = {(_lib, "cuda"): lambda: WithoutAttention(real_lib)}
    out = {"full_step_us": timed({}),
           "without_decode_attn_us": timed(no_attn),
           "without_layernorm_us": timed({(K, "layernorm_fwd"): noop}),
           "without_gemms_us": timed({(E, "gemm"): noop}),
           "gemms_only_us": timed({(K, "layernorm_fwd"): noop, **no_attn})}
    _lib.check_status()
    return {"metric": "leaf-evaluation step breakdown", "unit": "us per step", "trees": trees, **out}


def run_sequential(sims: int, positions: int, small: bool, seed: int = 0) -> dict:
    """The reference algorithm restated on this framework's PyTorch model (fp32): one tree at a
    time, every leaf re-encodes its whole game at batch 1 (``src/evaluation/decode.py:336-467``)."""
    import numpy as np
    import torch

    from allie_b200.search import MCTS
    from allie_b200.search.runner import TorchRunner

    tok, model = build_model(small)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model.to(dev).eval()
    runner = TorchRunner(model, tok, dev)
    games = random_games(positions, tok, np.random.default_rng(seed))
    m = MCTS(model, tok, device=dev, runner=runner, n_sims=sims)
    m.score_full(games[0], games[0].legal_moves)
    if dev == "cuda":
        torch.cuda.synchronize()
    c0 = runner.calls
    t0 = time.perf_counter()
    for g in games:
        m.score_full(g, g.legal_moves)
    if dev == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return dict(value=(runner.calls - c0) / dt, seconds=dt, positions=runner.calls - c0,
                p50_move_latency_s=dt / len(games),
                note="sequential PUCT, batch-1 full re-encode per leaf, fp32 PyTorch model")


def combine_over_ranks(out: dict, world: int) -> dict:
    """Whole-job figures of one independent search per rank: positions summed, divided by the
    slowest rank's time; the per-move latency is the median over ranks."""
    if world == 1 or "positions" not in out:
        return out
    import torch
    import torch.distributed as dist

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    stats = torch.tensor([float(out["positions"]), float(out["seconds"]), float(out.get("p50_move_latency_s", 0.0))],
                         dtype=torch.float64, device=dev)
    allv = [torch.zeros_like(stats) for _ in range(world)]
    dist.all_gather(allv, stats)
    positions = sum(float(v[0]) for v in allv)
    slowest = max(float(v[1]) for v in allv)
    out.update(value=positions / slowest, positions=int(positions), seconds=slowest,
               per_rank_seconds=[round(float(v[1]), 4) for v in allv],
               p50_move_latency_s=sorted(float(v[2]) for v in allv)[world // 2])
    return out


def main():
    import torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--trees", type=int, default=256)
    ap.add_argument("--sims", type=int, default=400)
    ap.add_argument("--impl", default="batched", choices=["batched", "sequential", "reference"])
    ap.add_argument("--small", action="store_true", help="tiny model (smoke test)")
    ap.add_argument("--seq-positions", type=int, default=8, help="root positions for --impl sequential / reference")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--ablate", action="store_true",
                    help="time the step's graph with one kind of kernel left out at a time (one GPU) and exit")
    args = ap.parse_args()
    if args.ablate:
        print(json.dumps(run_ablation(args.trees, args.small)), flush=True)
        return
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, "launch with torchrun --nproc-per-node <gpus>"
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo")
    out = {"metric": "MCTS leaf-eval positions/sec", "unit": "positions/s", "impl": args.impl,
           "dtype": "bf16" if args.impl == "batched" else "fp32", "data": "synthetic random legal games, prompts of 1-300 tokens",
           "config": {"model": "tiny" if args.small else "gpt2-medium-like 24L d1024 16H", "trees": args.trees,
                      "sims": args.sims}, "n_gpus": world}
    if args.impl == "batched":
        out.update(run_batched(args.trees, args.sims, args.small, seed=rank))      # different root positions per rank
    elif args.impl == "sequential":
        out.update(run_sequential(args.sims, args.seq_positions, args.small, seed=rank))
    else:
        out.update(run_reference(args.sims, args.seq_positions, args.small, seed=rank))
    out = combine_over_ranks(out, world)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
