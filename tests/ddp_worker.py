"""Worker for the multi-rank trainer tests (run under torch.distributed.run).

usage: ddp_worker.py <out_dir> <mode> <device> [moe|loop]   mode: fused | collective | auto
Trains a tiny model for 3 optimizer steps on a fixed synthetic stream (dropout off) and writes
the final flat parameters of every rank to <out_dir>/params_<mode>_<rank>.pt .
With ``loop`` the steps run inside ``Trainer.train()`` with validation and checkpoints every other
iteration, and rank 0's evaluation is slowed down on the host by more than the device-side wait
limit of the gradient kernels.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch

from allie_b200.config import Config
from allie_b200.data import UCITokenizer
from allie_b200.models import initialize_model
from allie_b200.train.trainer import Trainer


def run_loop(out_dir, mode, device):
    """Trainer.train() with eval / save intervals on; rank 0 is slow in validate()."""
    import json
    import time

    from allie_b200.etl.dataset import random_games

    rank = int(os.environ.get("RANK", 0))
    T, B = 128, 4
    tr = Trainer(Config({}), output_dir=os.path.join(out_dir, f"run_{mode}"), device=device, batch_size=B,
                 gradient_accumulation_steps=2, lr=1e-3, min_lr=1e-4, warmup_iters=0, decay_iters=100,
                 max_iters=5, eval_interval=2, log_interval=1, save_interval=2, weight_decay=0.01,
                 grad_clip=1.0, grad_sync=mode, use_wandb=False)
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    torch.manual_seed(0)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=3,
                             n_embd=128, n_head=2, n_positions=T)
    rng = np.random.default_rng(5)
    stream = (rng.integers(0, 1968, size=1 << 16).astype(np.uint32)
              | (rng.integers(1, 20, size=1 << 16).astype(np.uint32) << 16))
    games = os.path.join(out_dir, f"val_{rank}.jsonl")
    random_games(games, n=6, max_plies=30, seed=9)
    val = [json.loads(l) for l in open(games)]
    tr.setup_dataloaders(tok, stream, val, val)
    tr.setup_model(model)
    if rank == 0:
        slow = tr.evaluate

        def evaluate(dataset):
            time.sleep(2.5)
            return slow(dataset)

        tr.evaluate = evaluate
    tr.train()
    if device.startswith("cuda"):
        from allie_b200.ops import _lib

        torch.cuda.synchronize()
        _lib.check_status()
    flat = torch.cat([p.detach().float().reshape(-1).cpu() for _, p in sorted(model.named_parameters())])
    fused = bool(tr.grad_sync is not None and tr.grad_sync.fused)
    buckets = len(tr.engine.arena.buckets) if tr.engine is not None else 0
    torch.save({"params": flat, "rank": rank, "fused": fused, "buckets": buckets, "iter_num": tr.iter_num},
               os.path.join(out_dir, f"params_{mode}_{rank}.pt"))
    tr.cleanup()


def main():
    out_dir, mode, device = sys.argv[1], sys.argv[2], sys.argv[3]
    moe = len(sys.argv) > 4 and sys.argv[4] == "moe"
    if len(sys.argv) > 4 and sys.argv[4] == "loop":
        os.environ["ALLIE_NO_WANDB"] = "1"
        return run_loop(out_dir, mode, device)
    os.environ["ALLIE_NO_WANDB"] = "1"
    rank = int(os.environ.get("RANK", 0))
    T, B = 128, 4
    tr = Trainer(Config({}), output_dir=os.path.join(out_dir, f"run_{mode}"), device=device, batch_size=B,
                 gradient_accumulation_steps=2, lr=1e-3, min_lr=1e-4, warmup_iters=0, decay_iters=100,
                 max_iters=3, eval_interval=0, log_interval=-1, save_interval=0, weight_decay=0.01,
                 grad_clip=1.0, grad_sync=mode, use_wandb=False)
    tok = UCITokenizer(max_length=T, vocab_size_multiple_of=128)
    torch.manual_seed(0)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=2,
                             n_embd=128, n_head=2, n_positions=T, resid_pdrop=0.0, embd_pdrop=0.0,
                             attn_pdrop=0.0, **(dict(num_experts=8, moe_ffn=256, moe_layer_freq=2, capacity_factor=8.0,
                                                      aux_loss_coef=0.0) if moe else {}))
    if moe:
        with torch.no_grad():
            for n_, p_ in model.named_parameters():
                if "router" in n_:
                    p_.mul_(20.0)
    rng = np.random.default_rng(5)
    stream = (rng.integers(0, 1968, size=1 << 16).astype(np.uint32)
              | (rng.integers(1, 20, size=1 << 16).astype(np.uint32) << 16))
    tr.setup_dataloaders(tok, stream, [], [])
    tr.setup_model(model)
    world = tr.ddp_world_size
    wrng = np.random.default_rng(11)
    losses = []
    for step in range(3):
        # the same global batch regardless of world size: rank r takes every world-th window
        starts = wrng.integers(0, len(stream) - T, size=(2, 8))     # 8 windows per micro-step in total
        wins = []
        for ms in range(2):
            mine = starts[ms][rank::world]
            w = np.stack([stream[s:s + T] for s in mine]).astype(np.uint32).view(np.int32)
            wins.append(torch.from_numpy(w))
        losses.append(float(tr.train_step(wins)))
        tr.iter_num += 1
    if device == "cpu":
        # the log line's window time is the maximum over ranks: rank r reports (r + 1) seconds
        tr._log_throughput(float(rank + 1), 1, 1000)
    reload_ok = None
    if moe and device.startswith("cuda"):
        # checkpoint round trip: the file holds whole expert banks whatever the rank count, and
        # loading it gives every rank back exactly its own slice of weights and Adam moments
        import torch.distributed as dist

        tr._gather_optimizer_state()
        tr.save_ckpt("last")
        if dist.is_initialized():
            dist.barrier()
        arena = tr.engine.arena
        before = {n: p.detach().clone() for n, p in model.named_parameters()}
        m_before, v_before = arena.exp_avg.clone(), arena.exp_avg_sq.clone()
        arena.master.zero_(); arena.exp_avg.zero_(); arena.exp_avg_sq.zero_()
        tr.load_ckpt("last")
        reload_ok = (all(torch.equal(before[n], p.detach()) for n, p in model.named_parameters())
                     and torch.equal(m_before[arena.sync_end:], arena.exp_avg[arena.sync_end:])
                     and torch.equal(v_before[arena.sync_end:], arena.exp_avg_sq[arena.sync_end:])
                     # the moments of the replicated parameters are gathered on rank 0 only (it writes the file)
                     and (rank != 0 or torch.equal(m_before[:arena.sync_end], arena.exp_avg[:arena.sync_end])))
    tr.sync_parameters()      # the fp32 masters of weight matrices are current only on their owner rank
    flat = torch.cat([p.detach().float().reshape(-1).cpu() for _, p in sorted(model.named_parameters())])
    fused = bool(tr.grad_sync is not None and tr.grad_sync.fused)
    named = {n: p.detach().float().cpu() for n, p in model.named_parameters()}
    torch.save({"params": flat, "named": named, "rank": rank, "world": world, "losses": losses, "fused": fused,
                "reload_ok": reload_ok, "multimem": bool(fused and tr.grad_sync.nvl.multimem)},
               os.path.join(out_dir, f"params_{mode}_{rank}.pt"))
    if device.startswith("cuda"):
        from allie_b200.ops import _lib

        torch.cuda.synchronize()
        _lib.check_status()
    tr.cleanup()


if __name__ == "__main__":
    main()
