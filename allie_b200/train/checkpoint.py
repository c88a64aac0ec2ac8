"""Checkpoints in the reference's format (``src/modeling/trainer.py:382-409``):
``{output_dir}/{last|best}.pt`` = ``torch.save({"iter_num", "best_val_loss", "model": state_dict,
"optimizer": torch-AdamW-style state_dict})``.  The model state dict carries the reference's keys
(including the tied ``lm_head.weight`` duplicate); the optimizer entry uses two parameter groups
(decay / no-decay) whose parameters are numbered in *sorted name* order, so files written here load
into the reference trainer and vice versa.  The engine keeps its Adam moments in flat arenas; they
are scattered to / gathered from per-parameter tensors here.  Extra keys (``rng``, ``engine``) are
ignored by the reference.

Expert parallelism: every rank holds a slice (along the expert dimension) of each expert bank and
of its Adam moments.  The file always stores whole banks, so a checkpoint written by N ranks loads
into any other rank count: ``save_checkpoint`` is then a collective (every rank calls it, rank 0
writes) and ``load_checkpoint`` cuts this rank's slice out of the whole bank.
"""
from __future__ import annotations

import os

import torch


def _ordered_names(engine) -> tuple[list[str], int]:
    """Parameter names in the reference optimizer's numbering (decay group then no-decay group,
    each sorted by name) and the size of the first group."""
    from ..models.engine import partition_parameter_names

    decay, no_decay = partition_parameter_names(engine.model)
    return decay + no_decay, len(decay)


def _local_names(engine) -> list[str]:
    """Names of the rank-local (expert-parallel) parameters of this engine."""
    a = engine.arena
    return [n for n in a.names if a.offsets[n] >= a.sync_end]


def _ep_world() -> tuple[int, int]:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def gather_expert_banks(engine) -> dict[str, dict[str, torch.Tensor]]:
    """Collective over all ranks.  For every rank-local parameter returns the whole bank on the
    CPU (slices of all ranks concatenated in rank order): ``{name: {"param", "exp_avg",
    "exp_avg_sq"}}``; the moment entries are missing before the first optimizer step."""
    import torch.distributed as dist

    rank, world = _ep_world()
    local = _local_names(engine)
    if world == 1 or not local:
        return {}
    a = engine.arena
    out: dict[str, dict[str, torch.Tensor]] = {}
    for n in local:
        srcs = {"param": a.view(a.master, n)}
        if a.exp_avg is not None:
            srcs["exp_avg"] = a.view(a.exp_avg, n)
            srcs["exp_avg_sq"] = a.view(a.exp_avg_sq, n)
        out[n] = {}
        for key, t in srcs.items():
            t = t.detach().contiguous()
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            if rank == 0:
                out[n][key] = torch.cat([p.cpu() for p in parts], 0)
    return out


def _my_slice(full: torch.Tensor, local_shape) -> torch.Tensor:
    """This rank's slice of a whole expert bank (no-op when the shapes already agree)."""
    if tuple(full.shape) == tuple(local_shape):
        return full
    rank, world = _ep_world()
    n_local = local_shape[0]
    assert full.shape[0] == n_local * world and tuple(full.shape[1:]) == tuple(local_shape[1:]), \
        f"expert bank of shape {tuple(full.shape)} does not split into {world} x {tuple(local_shape)}"
    return full[rank * n_local:(rank + 1) * n_local]


def _optimizer_state_from_engine(engine, lr, betas, weight_decay, banks=None) -> dict:
    a = engine.arena
    names, n_decay = _ordered_names(engine)
    banks = banks or {}
    state = {}
    if a.exp_avg is not None:
        step = torch.tensor(float(engine.step_count))
        for i, n in enumerate(names):
            if n in banks and "exp_avg" in banks[n]:
                state[i] = {"step": step.clone(), "exp_avg": banks[n]["exp_avg"],
                            "exp_avg_sq": banks[n]["exp_avg_sq"]}
                continue
            state[i] = {"step": step.clone(), "exp_avg": a.view(a.exp_avg, n).detach().cpu().clone(),
                        "exp_avg_sq": a.view(a.exp_avg_sq, n).detach().cpu().clone()}
    common = dict(lr=lr, betas=tuple(betas), eps=1e-8, amsgrad=False, foreach=None, maximize=False,
                  capturable=False, differentiable=False, fused=True, decoupled_weight_decay=True)
    groups = [dict(common, weight_decay=weight_decay, params=list(range(n_decay))),
              dict(common, weight_decay=0.0, params=list(range(n_decay, len(names))))]
    return {"state": state, "param_groups": groups}


def _optimizer_state_into_engine(engine, opt_sd: dict) -> None:
    a = engine.arena
    state = opt_sd.get("state", {})
    if not state:
        return
    a.ensure_state()
    names, _ = _ordered_names(engine)
    order = [i for g in opt_sd["param_groups"] for i in g["params"]]
    assert len(order) == len(names), "optimizer state does not match the model"
    step = 0
    for idx, n in zip(order, names):
        st = state.get(idx, state.get(str(idx)))
        if st is None:
            continue
        a.view(a.exp_avg, n).copy_(_my_slice(st["exp_avg"], a.shapes[n]).to(a.exp_avg.device).view(a.shapes[n]))
        a.view(a.exp_avg_sq, n).copy_(_my_slice(st["exp_avg_sq"], a.shapes[n]).to(a.exp_avg.device).view(a.shapes[n]))
        step = max(step, int(float(st["step"])))
    engine.step_count = step


def save_checkpoint(path: str, model, engine, optimizer, iter_num: int, best_val_loss: float, *,
                    lr: float, betas, weight_decay: float) -> None:
    """Writes the checkpoint.  With expert parallelism (rank-local parameters and more than one
    rank) every rank must call this: the banks are gathered collectively and rank 0 writes."""
    banks = gather_expert_banks(engine) if engine is not None else {}
    rank, world = _ep_world()
    if engine is not None and world > 1 and _local_names(engine) and rank != 0:
        return
    model_sd = {k: (banks[k]["param"].to(v.dtype) if k in banks else v.detach().cpu().clone())
                for k, v in model.state_dict().items()}
    if engine is not None:
        opt_sd = _optimizer_state_from_engine(engine, lr, betas, weight_decay, banks)
        extra = {"engine": {"fwd_count": engine.fwd_count, "seed": engine.seed}}
    else:
        opt_sd = optimizer.state_dict()
        extra = {}
    tmp = path + ".tmp"
    torch.save({"iter_num": iter_num, "best_val_loss": best_val_loss, "model": model_sd,
                "optimizer": opt_sd, "rng": torch.get_rng_state(), **extra}, tmp)
    os.replace(tmp, path)  # a crash mid-write never leaves a truncated checkpoint behind


def load_checkpoint(path: str, model, engine, optimizer, device) -> dict:
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    for key in ("iter_num", "best_val_loss", "model", "optimizer"):
        if key not in ckpt:
            raise ValueError(f"{path}: not a trainer checkpoint (missing {key!r})")
    # parameters are views into the engine's arena: load_state_dict copies in place
    model_sd = ckpt["model"]
    if engine is not None and _local_names(engine):
        shapes = engine.arena.shapes
        model_sd = {k: (_my_slice(v, shapes[k]) if k in shapes else v) for k, v in model_sd.items()}
    from ..models import load_model_state

    load_model_state(model, model_sd)
    if engine is not None:
        engine.arena.refresh_shadow()
        _optimizer_state_into_engine(engine, ckpt["optimizer"])
        if "engine" in ckpt:
            engine.fwd_count = ckpt["engine"].get("fwd_count", engine.fwd_count)
    elif optimizer is not None:
        optimizer.load_state_dict(ckpt["optimizer"])
    return {"iter_num": ckpt["iter_num"], "best_val_loss": ckpt["best_val_loss"]}
