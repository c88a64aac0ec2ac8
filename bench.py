"""Headline benchmark: training throughput (tokens/s) of the GPT-2-medium-shaped Allie model.

Config (default, the headline): 24 layers, d_model 1024, 16 heads, MLP 4096, context 512, vocab 2048, policy +
value + think-time losses, dropout 0.1 as the reference trains, bf16 tensor-core math with fp32
residual stream / master weights, global batch 512 sequences per optimizer step (micro-batch 64 per
GPU, gradient accumulation 8 / n_gpus: strong scaling), AdamW with global-norm clipping.
Synthetic uniform-random move tokens with two leading ELO tokens per window, random-init weights.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...             # the unmodified reference trainer
    python bench.py --model large ...                         # large-ablation shape: 32 layers, d_model 1280, 20 heads

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N``.  Rank 0 prints one
JSON line.  ``value`` is timed on the device with CUDA events around exactly K optimizer steps,
max over ranks, inputs already resident on the GPU; ``e2e`` times the same K steps through
``Trainer.train_step()`` as the training loop calls it: windows drawn by the trainer's sampler
(host gather on its prefetch thread), the per-micro-step host->device copy of the raw windows
from pinned memory, and a device->host read of the loss every step.

After the headline, rank 0 runs the two other headline workloads as jobs of their own on the same
GPUs (the training benchmark has released them by then) inside a time budget and reports their
results under ``secondary``: ``mcts`` (256 trees x 400 simulations per GPU,
positions/s and per-move latency) at any N, and ``moe`` (the 9.3 B-parameter mixture-of-experts
config, expert parallel over all ranks, tokens/s) at N = 8.  ``--impl reference`` fills the same
object with the unmodified reference ``evaluation.decode.MCTS`` and, for the MoE config the
reference does not have, a plain-PyTorch expert-parallel baseline (``all_to_all_single`` +
``torch._grouped_mm``).  At N >= 2 the line also carries ``grad_sync_check``: a tiny model stepped
through the fused NVLink gradient path and through all_reduce + replicated AdamW from the same
state, and a tiny MoE model stepped with its experts spread over the ranks and with them
replicated, with the largest parameter difference of each pair.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(n_layer=24, n_embd=1024, n_head=16, n_positions=1024)
# --model large: the large-ablation shape (about twice the medium parameter count)
MODELS = {"medium": MODEL, "large": dict(n_layer=32, n_embd=1280, n_head=20, n_positions=1024)}
SEQ_LEN, VOCAB_MULT, GLOBAL_BATCH, MICRO_BATCH = 512, 128, 512, 64
BASELINE_TOKENS_PER_S = 2.17e5   # derived from the reference README: 8x RTX A6000, ~2 weeks
START_ITER = 10                  # both arms start their steps here in the 2000-iteration warm-up


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  ``start()`` launches the sampler
    (during warm-up, so it is already producing rows), ``mark()`` is called at the start of the
    timed region and ``stop()`` summarises the rows sampled after the mark."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.idx = gpu_index
        self.first = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def mark(self):
        self.first = len(self.rows)

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows[self.first:]:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx = float(r[2])
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def synthetic_stream(n_words: int, vocab: int, seq_len: int, seed: int):
    """Uniform random move tokens with think times and outcomes packed like real data; every
    ``seq_len`` words start with two ELO pseudo-tokens and a time-control token."""
    import numpy as np

    rng = np.random.default_rng(seed)
    ids = rng.integers(0, 1968, size=n_words, dtype=np.uint32)
    secs = rng.integers(0, 30, size=n_words, dtype=np.uint32)
    words = ids | ((secs + 1) << 16)
    starts = np.arange(0, n_words - 3, seq_len)
    outcome = rng.integers(0, 3, size=len(starts), dtype=np.uint32) << 14
    words = words.reshape(-1)
    words[starts] = (vocab + rng.integers(800, 2600, size=len(starts))).astype(np.uint32)
    words[starts + 1] = (vocab + rng.integers(800, 2600, size=len(starts))).astype(np.uint32)
    words[starts + 2] = rng.integers(1968, 1992, size=len(starts)).astype(np.uint32)
    for k in range(seq_len):
        sl = starts + k
        sl = sl[sl < n_words]
        words[sl] |= outcome[: len(sl)]
    return words


def dist_info():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    import torch
    import torch.distributed as dist

    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(world: int):
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def common_config(model_name: str, ga: int, world: int) -> dict:
    """The part of ``config`` both arms print identically (same shape, batch, accumulation)."""
    shape = MODELS[model_name]
    d = shape["n_embd"]
    return {"model": f"gpt2-{model_name}-like {shape['n_layer']}L d{d} {shape['n_head']}H mlp{4 * d} ctx512 vocab2048 "
                     "+ control token + value/time heads, dropout 0.1",
            "global_batch": GLOBAL_BATCH, "seq_len": SEQ_LEN, "micro_batch": MICRO_BATCH, "grad_accum": ga,
            "parallelism": f"dp{world}",
            "l2_policy": "inputs larger than L2: each micro-step streams >1 GB of activations and 1.2 GB of "
                         "fp32 weights+grads, distinct windows per micro-step"}


def grad_sync_check(world: int) -> dict:
    """Numerical check of the multi-GPU paths on tiny models, before anything is timed.  (a) Two
    optimizer steps through the fused NVLink gradient path against the same steps through
    all_reduce + replicated AdamW, from the same weights and windows.  (b) A tiny MoE model
    stepped with its experts spread over the ranks (dispatch / combine through peer memory)
    against the same model with every expert on every rank.  Reports the largest absolute
    parameter difference of each pair (max over ranks); one Adam step moves a weight by about
    ``lr``, and a gradient sum in another order can flip the sign of a near-zero update."""
    import numpy as np
    import torch

    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.ops import _lib
    from allie_b200.train.trainer import Trainer

    rank = dist_info()[0]
    T, B, LR = 128, 4, 1e-3
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    rng = np.random.default_rng(5)
    stream = (rng.integers(0, 1968, size=1 << 16).astype(np.uint32)
              | (rng.integers(1, 20, size=1 << 16).astype(np.uint32) << 16))
    wrng = np.random.default_rng(11)
    starts = wrng.integers(0, len(stream) - T, size=(2, 2, B * world))
    steps = [[torch.from_numpy(np.stack([stream[s:s + T] for s in starts[st][ms][rank::world]]).astype(np.uint32).view(np.int32))
              for ms in range(2)] for st in range(2)]

    def run(mode: str, moe: bool, expert_parallel: bool = True) -> "torch.Tensor":
        tr = Trainer(Config({}), output_dir=tempfile.mkdtemp(prefix="allie_chk_"), batch_size=B,
                     gradient_accumulation_steps=2, lr=LR, min_lr=1e-4, warmup_iters=0, decay_iters=100, max_iters=3,
                     eval_interval=0, log_interval=-1, save_interval=0, weight_decay=0.01, grad_clip=1.0,
                     grad_sync=mode, use_wandb=False, expert_parallel=expert_parallel)
        torch.manual_seed(0)
        extra = dict(num_experts=8, moe_ffn=256, moe_layer_freq=2, capacity_factor=8.0, aux_loss_coef=0.0) if moe else {}
        model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=4 if not moe else 2,
                                 n_embd=128, n_head=2, n_positions=T, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0,
                                 **extra)
        if moe:
            with torch.no_grad():
                for n_, p_ in model.named_parameters():
                    if "router" in n_:
                        p_.mul_(20.0)      # decisive routing: no token sits on a tie between two experts
        tr.setup_dataloaders(tok, stream, [], [])
        tr.setup_model(model)
        for ws in steps:
            tr.train_step(ws)
            tr.iter_num += 1
        tr.sync_parameters()
        torch.cuda.synchronize()
        _lib.check_status()
        named = {n: p.detach().float().clone() for n, p in model.named_parameters()}
        tr.sampler.close()
        return named

    def worst(a: dict, b: dict, world: int) -> float:
        d = 0.0
        for n, p in a.items():
            q = b[n]
            if p.shape != q.shape:                     # expert bank: this rank's slice of the replicated bank
                El = p.shape[0]
                q = q[rank * El:(rank + 1) * El]
            d = max(d, float((p - q).abs().max()))
        return max_over_ranks(d, world)

    fused, coll = run("fused", False), run("collective", False)
    ep, rep = run("fused", True, True), run("fused", True, False)
    return {"fused_vs_all_reduce_max_abs_diff": worst(fused, coll, world),
            "expert_parallel_vs_replicated_max_abs_diff": worst(ep, rep, world), "lr": LR, "steps": 2,
            "note": "tiny models (4 blocks d128 / 2 blocks with 8 experts), dropout off, same windows"}


def _run_child(script_args: list[str], world: int, timeout_s: float, port: int) -> dict:
    """Runs one of the other benchmark scripts as its own job (``torchrun`` with ``world`` ranks, or a
    plain process) and returns the JSON line it prints.  A process of its own means a failure
    there (an exception, a device-side wait that ran out, a crash) cannot take the headline number
    of this process with it."""
    import signal

    drop = ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK",
            "ROLE_WORLD_SIZE", "ROLE_NAME", "MASTER_ADDR", "MASTER_PORT")
    env = {k: v for k, v in os.environ.items() if k not in drop and not k.startswith("TORCHELASTIC_")}
    if world > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), *script_args]
    else:
        cmd = [sys.executable, *script_args]
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, cwd=ROOT,
                            start_new_session=True)
    try:
        out, err = proc.communicate(timeout=timeout_s)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)       # the process group this call started, nothing else
        proc.communicate()
        return {"failed": f"no result within {timeout_s:.0f} s"}
    for line in reversed(out.splitlines()):
        line = line.strip()
        if line.startswith("{"):
            try:
                return json.loads(line)
            except json.JSONDecodeError:
                continue
    return {"failed": f"exit code {proc.returncode}: " + " | ".join(err.strip().splitlines()[-3:])[-300:]}


def run_secondary(args, world: int, reference: bool, t_start: float) -> dict:
    """The other two headline workloads, each as a job of its own on the same GPUs, started by rank
    0 after the training benchmark has released them, inside what is left of ``--secondary-budget``
    seconds: MCTS leaf evaluation at every N (one independent 256-tree x 400-simulation search
    per GPU; the reference arm: its own sequential MCTS on 8 root positions per GPU), the MoE
    config at N = 8 (``--secondary all``: a reduced MoE shape at smaller N)."""
    if args.secondary == "none":
        return {"skipped": "--secondary none"}
    base_port = int(os.environ.get("MASTER_PORT", "29500"))
    mcts = [os.path.join(ROOT, "bench_mcts.py"), "--gpus", str(world)]
    mcts += ["--impl", "reference", "--seq-positions", "8"] if reference else ["--impl", "batched"]
    moe = [os.path.join(ROOT, "bench_moe.py"), "--gpus", str(world), "--impl", "torch" if reference else "ours"]
    if world != 8:
        moe += ["--layers", "6", "--experts", "16", "--steps", "5"]      # reduced shape: the full one needs 8 GPUs
    jobs = [("mcts", mcts, 60.0)]
    if world == 8 or args.secondary == "all":
        jobs.append(("moe", moe, 120.0))
    out = {} if len(jobs) > 1 else {"moe": {"skipped": "the 9.3 B-parameter MoE config needs its experts spread over 8 GPUs"}}
    for i, (name, cmd, least) in enumerate(jobs):
        left = args.secondary_budget - (time.perf_counter() - t_start)
        if left < least:
            out[name] = {"skipped": f"time budget exhausted ({left:.0f} s left)"}
            continue
        t0 = time.perf_counter()
        out[name] = _run_child(cmd, world, left, base_port + 17 + i)
        out[name]["wall_s"] = round(time.perf_counter() - t0, 1)
    return out


def run_ours(args) -> dict:
    import numpy as np
    import torch

    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.ops import _lib
    from allie_b200.train.trainer import Trainer

    t_start = time.perf_counter()
    rank, world, local = dist_info()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert 8 % world == 0
    ga = GLOBAL_BATCH // (MICRO_BATCH * world)
    os.environ.setdefault("ALLIE_NO_WANDB", "1")
    out_dir = tempfile.mkdtemp(prefix="allie_bench_")
    cfg = Config({"trainer_config": {}, "data_config": {}, "model_config": {}})
    trainer = Trainer(cfg, output_dir=out_dir, batch_size=MICRO_BATCH, gradient_accumulation_steps=ga,
                      lr=6e-4, min_lr=1e-5, weight_decay=1e-2, grad_clip=1.0, warmup_iters=2000,
                      decay_iters=2_000_000, max_iters=2_000_000, eval_interval=0, log_interval=-1,
                      save_interval=0, use_wandb=False, cuda_graph=False if args.no_cuda_graph else None)
    tok = UCITokenizer(max_length=SEQ_LEN, vocab_size_multiple_of=VOCAB_MULT)
    torch.manual_seed(1234)
    model = initialize_model(tok, "gpt2-medium", use_control_token=True, use_regression_head=True,
                             use_pretrained=False, **MODELS[args.model])
    stream = synthetic_stream(64 * 1024 * SEQ_LEN // 8, len(tok), SEQ_LEN, seed=7 + rank)
    trainer.setup_dataloaders(tok, stream, [], [])
    trainer.setup_model(model)
    # the first iterations of the warm-up schedule (lr = 6e-4 * iter / 2000), as a run from random
    # init sees them; fresh Adam moments stepped at a mid-schedule rate overshoot the think-time
    # loss a hundredfold for two steps, which would make final_loss meaningless
    trainer.iter_num = START_ITER
    dev = trainer.engine.device
    sync_check = grad_sync_check(world) if world > 1 else None

    # windows larger than L2 in aggregate: K*ga distinct [64, 512] windows per rank, pre-staged
    n_win = (args.steps + args.warmup) * ga
    host_windows = [trainer.sampler.next().clone().pin_memory() for _ in range(min(n_win, 64))]
    dev_windows = [w.to(dev) for w in host_windows]

    def step_device(i):
        ws = [dev_windows[(i * ga + m) % len(dev_windows)] for m in range(ga)]
        return trainer.train_step(ws)

    def step_e2e(i, sink):
        # the call the training loop makes: the trainer draws its own windows (sampler thread,
        # pinned staging buffers), copies them to the device and steps
        loss = trainer.train_step()
        sink.copy_(loss, non_blocking=True)

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    _lib.check_status()

    barrier_sync(world)
    sampler.mark()
    launches0 = _lib.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step_device(args.warmup + i)
    e1.record()
    barrier_sync(world)
    launches = _lib.LAUNCHES - launches0
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    final_loss = float(loss)
    _lib.check_status()

    # end-to-end: pinned host windows -> H2D every micro-step, loss -> host every step
    sink = torch.zeros((), dtype=torch.float32, pin_memory=True)
    step_e2e(0, sink)
    barrier_sync(world)
    t0 = time.perf_counter()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for i in range(args.steps):
        step_e2e(i, sink)
        torch.cuda.current_stream().synchronize()   # the loss value is on the host here
        _ = float(sink)
    g1.record()
    barrier_sync(world)
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(g0.elapsed_time(g1), wall_ms), world)

    # phase breakdown (outside both timed regions): device time of data / forward+backward /
    # gradient synchronisation + optimizer per step, from the trainer's CUDA-event phase timers
    trainer.tracer.enabled = True
    trainer.tracer.summary()
    for i in range(2):
        step_device(i)
    phases = {k: round(v["ms"] / 2, 3) for k, v in trainer.tracer.summary().items()}
    phases = {k: max_over_ranks(v, world) for k, v in phases.items()}
    trainer.tracer.enabled = False

    tokens_per_step = GLOBAL_BATCH * SEQ_LEN
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    n_params = sum(p.numel() for p in model.parameters())
    shape = MODELS[args.model]
    L, d, V = shape["n_layer"], shape["n_embd"], len(tok)
    flops_per_token = 6 * (n_params - V * d - shape["n_positions"] * d) + 6 * V * d + 12 * L * d * SEQ_LEN
    result = {
        "metric": f"train tokens/sec ({args.model} config)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": value / BASELINE_TOKENS_PER_S, "dtype": "bf16", "data": "synthetic",
        "impl": "allie_b200",
        "config": common_config(args.model, ga, world),
        "arm": {"grad_sync": ("fused-nvlink-multimem" if trainer.grad_sync.nvl.multimem else
                              "fused-nvlink-multimem-reduce" if trainer.grad_sync.nvl.mc_grad else "fused-nvlink-p2p")
                             if (trainer.grad_sync and trainer.grad_sync.fused)
                             else ("all_reduce" if world > 1 else "none"),
                "grad_buckets": len(trainer.engine.arena.buckets),
                "micro_step_cuda_graph": bool(trainer.engine.step_graph),
                "e2e_path": "Trainer.train_step(): sampler thread -> pinned windows -> H2D -> step -> loss D2H"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": ga * MICRO_BATCH * SEQ_LEN * 4, "d2h_bytes_per_step": 4},
        "gpu_launches": launches,
        "phase_ms_per_step": phases,
        "final_loss": final_loss,
        "model_tflops_per_gpu": value * flops_per_token / world / 1e12,
    }
    if sync_check is not None:
        result["grad_sync_check"] = sync_check
    # release the GPUs (and the process group) before the secondary workloads run as their own jobs
    trainer.cleanup()
    trainer.engine = trainer.grad_sync = trainer.model = None
    del dev_windows, host_windows, model
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    if rank == 0:
        result["secondary"] = run_secondary(args, world, False, t_start)
    return result


def run_reference(args) -> dict:
    """The unmodified reference package (installed with ``pip --target baseline/_ref --no-deps``),
    driven through its own ``Trainer`` / ``initialize_model`` / ``UCITokenizer`` and its stock
    ``train()`` loop (bf16 autocast, ``torch.compile``, DDP, fused AdamW).  Third-party modules that are
    not installed here (omegaconf, python-chess, optimum) are satisfied by import stand-ins in
    ``baseline/shims``; the GPT-2-medium shape comes from a local ``config.json`` instead of the hub.
    Timing hooks are attached from outside through ``optimizer.register_step_post_hook``."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "modeling")):
        return {"impl": "reference", "unavailable": "baseline/_ref is missing (pip install --target was not run)"}
    sys.path.insert(0, os.path.join(ROOT, "baseline", "shims"))
    sys.path.insert(0, ref_dir)
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("WANDB_SILENT", "true")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    try:
        import numpy as np
        import torch
        import torch.distributed as dist
        from modeling.data import UCITokenizer
        from modeling.model import initialize_model
        from modeling.trainer import Trainer
        from omegaconf import OmegaConf
    except Exception as e:
        return {"impl": "reference", "unavailable": f"reference import failed: {type(e).__name__}: {e}"[:300]}

    t_start = time.perf_counter()
    rank, world, local = dist_info()
    assert world == args.gpus
    ga = GLOBAL_BATCH // (MICRO_BATCH * world)
    W, K = args.warmup, args.steps
    out_dir = tempfile.mkdtemp(prefix="allie_ref_")
    cfg = OmegaConf.create({"trainer_config": {}, "data_config": {}, "model_config": {}})
    trainer = Trainer(cfg, output_dir=out_dir, dtype="bfloat16", torch_compile=True, batch_size=MICRO_BATCH,
                      gradient_accumulation_steps=ga, lr=6e-4, min_lr=1e-5, weight_decay=1e-2,
                      warmup_iters=2000, decay_iters=2_000_000, max_iters=W + K - 1, eval_interval=0,
                      log_interval=10**9, save_interval=0)
    tok = UCITokenizer(max_length=SEQ_LEN, vocab_size_multiple_of=VOCAB_MULT)
    torch.manual_seed(1234)
    shape = {k: v for k, v in MODELS[args.model].items() if args.model != "medium"}   # HF config overrides
    model = initialize_model(tok, os.path.join(ROOT, "baseline", "gpt2-medium"), use_control_token=True,
                             use_regression_head=True, use_pretrained=False, **shape)
    stream = synthetic_stream(64 * 1024 * SEQ_LEN // 8, len(tok), SEQ_LEN, seed=7 + rank)
    trainer.setup_dataloaders(tok, stream, [], [])
    trainer.setup_model(model)
    trainer.iter_num = START_ITER
    trainer.max_iters = START_ITER + W + K - 1

    state = {"n": 0, "ms": None, "clocks": None, "wall0": None}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)

    def hook(optimizer, a, kw):
        state["n"] += 1
        if state["n"] == 1:
            sampler.start()
        if state["n"] == W:
            barrier_sync(world)
            sampler.mark()
            state["wall0"] = time.perf_counter()
            e0.record()
        elif state["n"] == W + K:
            e1.record()
            barrier_sync(world)
            state["wall_ms"] = (time.perf_counter() - state["wall0"]) * 1e3
            state["clocks"] = sampler.stop()
            state["ms"] = e0.elapsed_time(e1)

    trainer.optimizer.register_step_post_hook(hook)
    trainer.train()
    if state["ms"] is None:
        return {"impl": "reference", "unavailable": "reference train() ended before the timed steps completed"}
    ms = max_over_ranks(state["ms"], world)
    tokens_per_step = GLOBAL_BATCH * SEQ_LEN
    value = tokens_per_step * K / (ms / 1e3)
    result = {
        "metric": f"train tokens/sec ({args.model} config)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": value / BASELINE_TOKENS_PER_S, "dtype": "bf16",
        "data": "synthetic", "impl": "reference",
        "config": common_config(args.model, ga, world),
        "arm": {"stack": "reference Trainer.train(): autocast bf16 + torch.compile + DDP + fused AdamW",
                "note": "the reference loop times its own host data pipeline, H2D copies and "
                        "loss.item() every step, so value == e2e for this arm"},
        "clocks": state["clocks"],
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": ga * MICRO_BATCH * SEQ_LEN * (8 * 3 + 4 * 3),
                "d2h_bytes_per_step": 4},
        "gpu_launches": 0,
    }
    trainer.cleanup()
    for attr in ("model", "optimizer", "model_fn"):
        if hasattr(trainer, attr):
            setattr(trainer, attr, None)
    del model
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    if rank == 0:
        result["secondary"] = run_secondary(args, world, True, t_start)
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="medium", choices=sorted(MODELS),
                    help="medium = the headline config; large = the large-ablation shape (32L, d1280, 20H)")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="launch the kernels of every micro-step one by one instead of replaying a CUDA graph "
                         "(for per-kernel profiles)")
    ap.add_argument("--secondary", default="auto", choices=["auto", "none", "all"],
                    help="auto: MCTS at every N, MoE at N = 8; all: also a reduced MoE shape at N < 8; none: headline only")
    ap.add_argument("--secondary-budget", type=float, default=600.0,
                    help="seconds (from process start) after which no further secondary benchmark is started")
    args = ap.parse_args()
    rank, world, _ = dist_info()
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun when started as a plain process
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"),
               os.path.abspath(__file__), *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        try:
            res = run_reference(args)
        except Exception as e:  # the reference arm must never take the bench down
            import traceback

            traceback.print_exc(file=sys.stderr)
            res = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}
    else:
        res = run_ours(args)
    if rank == 0:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
