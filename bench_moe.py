"""Training throughput of the mixture-of-experts configuration (tokens/s).

Config: 24 layers, d_model 2048, 16 heads of 128, every third block routes top-2 over 64 experts
of FFN 4096 (dense FFN 4096 elsewhere; about 9.3 B parameters), context 512, vocab 2048, softmax
router with load-balance loss, expert parallelism over all ranks, global batch 512 sequences
(micro-batch 32 per GPU: 512 routed token slots per expert and micro-step), dropout 0.1, bf16 tensor-core math.  Synthetic tokens, random init.

    torchrun --nproc-per-node 8 bench_moe.py --gpus 8              # this framework
    torchrun --nproc-per-node 8 bench_moe.py --gpus 8 --impl torch # plain-PyTorch EP baseline
``--layers`` / ``--experts`` shrink the model for smoke runs on fewer GPUs (the full model only
fits when its experts are spread over 8 GPUs).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from bench import ClockSampler, barrier_sync, dist_info, max_over_ranks, synthetic_stream  # noqa: E402

SEQ_LEN, GLOBAL_BATCH, MICRO_BATCH = 512, 512, 32


def run_moe(impl: str = "ours", steps: int = 10, warmup: int = 3, layers: int = 24, experts: int = 64,
            global_batch: int = GLOBAL_BATCH, micro_batch: int = MICRO_BATCH) -> dict:
    """One MoE training benchmark on the ranks of the current torchrun job (or one process).
    ``impl``: ``ours`` (this framework) or ``torch`` (plain-PyTorch expert-parallel baseline).
    May run after another trainer in the same process: the process group is reused."""
    import numpy as np
    import torch

    rank, world, local = dist_info()
    os.environ.setdefault("ALLIE_NO_WANDB", "1")
    from allie_b200.config import Config
    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model

    ga = max(1, global_batch // (micro_batch * world))
    tok = UCITokenizer(max_length=SEQ_LEN, vocab_size_multiple_of=128)
    shape = dict(n_layer=layers, n_embd=2048, n_head=16, n_inner=4096, n_positions=1024,
                 num_experts=experts, moe_top_k=2, moe_ffn=4096, moe_layer_freq=3, aux_loss_coef=0.01,
                 capacity_factor=2.0, ep_world=world, ep_rank=rank)
    torch.manual_seed(1234)
    stream = synthetic_stream(1 << 22, len(tok), SEQ_LEN, seed=7 + rank)
    tokens_per_step = ga * micro_batch * world * SEQ_LEN
    # both arms step at the learning rate of the first warm-up iterations (3e-4 * 10 / 2000): fresh
    # Adam moments stepped at a mid-schedule rate overshoot the think-time loss a hundredfold for
    # two steps (every parameter moves by lr along the sign of its gradient), dense model or not
    LR, WARM, ITER = 3e-4, 2000, 10
    stats = lambda: {}
    if impl == "ours":
        from allie_b200.ops import _lib
        from allie_b200.train.trainer import Trainer

        trainer = Trainer(Config({}), output_dir=tempfile.mkdtemp(prefix="allie_moe_"), batch_size=micro_batch,
                          gradient_accumulation_steps=ga, lr=LR, min_lr=1e-5, weight_decay=1e-2, grad_clip=1.0,
                          warmup_iters=WARM, decay_iters=2_000_000, max_iters=2_000_000, eval_interval=0,
                          log_interval=-1, save_interval=0, use_wandb=False)
        model = initialize_model(tok, "gpt2-medium", use_control_token=True, use_regression_head=True, **shape)
        trainer.setup_dataloaders(tok, stream, [], [])
        trainer.setup_model(model)
        trainer.iter_num = ITER
        dev = trainer.engine.device
        wins = [trainer.sampler.next().clone().to(dev) for _ in range(max(ga, 4))]
        step = lambda i: trainer.train_step([wins[(i * ga + m) % len(wins)] for m in range(ga)])
        counter = lambda: _lib.LAUNCHES
        check = _lib.check_status

        def stats():
            eng = trainer.engine
            st = eng.moe_stats() or {}
            # share of (token, choice) pairs beyond an expert's capacity, estimated from this rank's
            # routing (every rank draws tokens from the same distribution): those rows are dropped
            # (their tokens keep the residual only), so they are work the step did not do
            sent = kept = 0.0
            caps = {l: m.ctx.cap_e for (l, key), m in eng._moe_layers.items() if key[1]}
            for l, counts in (st.get("expert_tokens") or {}).items():
                for c in counts:
                    sent += world * c
                    kept += min(world * c, caps.get(l, world * c))
            return {"expert_load_max_over_mean": round(st.get("max_over_mean_load", 0.0), 3),
                    "capacity_overflow": bool(st.get("overflow", False)), "aux_loss": round(st.get("aux_loss", 0.0), 4),
                    "pairs_dropped_fraction_est": round(1.0 - kept / sent, 4) if sent else 0.0}
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import torch.distributed as dist
        from moe_torch import GROUPED, patch_model_for_baseline

        if world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl")
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        model = initialize_model(tok, "gpt2-medium", use_control_token=True, use_regression_head=True, **shape)
        patch_model_for_baseline(model)
        model.to(dev).train()
        local_params = {id(p) for m in model.modules() if type(m).__name__ == "ExpertBank" for p in m.parameters()}
        dense = [p for p in model.parameters() if id(p) not in local_params]
        lr = LR * ITER / WARM
        opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=1e-2, fused=True)
        wins = []
        for _ in range(max(ga, 4)):
            s = np.random.default_rng(len(wins) + rank).integers(0, len(stream) - SEQ_LEN, size=micro_batch)
            w = np.stack([stream[i:i + SEQ_LEN] for i in s]).astype(np.int64)
            wins.append({k: v.to(dev) for k, v in tok.pad_and_collate(list(w.astype(np.uint32))).items()})

        def step(i):
            for m in range(ga):
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = model(**wins[(i * ga + m) % len(wins)])["loss"]
                loss.backward()
            if world > 1:
                flat = torch.cat([p.grad.reshape(-1) for p in dense])
                dist.all_reduce(flat)
                flat /= world
                o = 0
                for p in dense:
                    p.grad.copy_(flat[o:o + p.numel()].view_as(p)); o += p.numel()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step(); opt.zero_grad(set_to_none=True)
            return loss.detach()
        counter = lambda: 0
        check = lambda: None
    trace = []                       # device-side loss of every step, read back after the timed region
    sampler = ClockSampler(local)
    sampler.start()
    for i in range(warmup):
        trace.append(step(i).clone())
    torch.cuda.synchronize()
    check()
    barrier_sync(world)
    sampler.mark()
    l0 = counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(warmup + i)
        trace.append(loss.clone())
    e1.record()
    barrier_sync(world)
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    check()
    n_params = sum(p.numel() for p in model.parameters())
    if impl == "ours":
        name = "allie_b200"
    else:
        name = "plain-pytorch-ep (all_to_all_single + " + ("torch._grouped_mm)" if GROUPED else "per-expert cuBLAS loop)")
    res = {"metric": "train tokens/sec (MoE config)", "value": tokens_per_step * steps / (ms / 1e3),
           "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup,
           "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "dtype": "bf16",
           "data": "synthetic", "impl": name,
           "config": {"model": f"{layers}L d2048 16H hd128, MoE every 3rd layer: {experts} experts x FFN 4096, top-2",
                      "global_batch": ga * micro_batch * world, "seq_len": SEQ_LEN, "micro_batch": micro_batch,
                      "grad_accum": ga, "parallelism": f"dp{world}+ep{world}", "params_per_rank": n_params,
                      "lr": LR * ITER / WARM},
           "clocks": clocks, "gpu_launches": counter() - l0, "final_loss": float(loss if loss.dim() == 0 else loss[0]),
           "loss_per_step": [round(float(t if t.dim() == 0 else t[0]), 3) for t in trace], **stats()}
    if impl == "ours":
        del trainer
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    ap.add_argument("--micro-batch", type=int, default=MICRO_BATCH)
    args = ap.parse_args()
    rank, world, _ = dist_info()
    assert world == args.gpus
    res = run_moe(args.impl, args.steps, args.warmup, args.layers, args.experts, args.global_batch, args.micro_batch)
    if rank == 0:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
