"""Checkpoints in the reference's format (``src/modeling/trainer.py:382-409``):
``{output_dir}/{last|best}.pt`` = ``torch.save({"iter_num", "best_val_loss", "model": state_dict,
"optimizer": torch-AdamW-style state_dict})``.  The model state dict carries the reference's keys
(including the tied ``lm_head.weight`` duplicate); the optimizer entry uses two parameter groups
(decay / no-decay) whose parameters are numbered in *sorted name* order, so files written here load
into the reference trainer and vice versa.  The engine keeps its Adam moments in flat arenas; they
are scattered to / gathered from per-parameter tensors here.  Extra keys (``rng``, ``engine``) are
ignored by the reference.
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


def _optimizer_state_from_engine(engine, lr, betas, weight_decay) -> dict:
    a = engine.arena
    names, n_decay = _ordered_names(engine)
    state = {}
    if a.exp_avg is not None:
        step = torch.tensor(float(engine.step_count))
        for i, n in enumerate(names):
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
        a.view(a.exp_avg, n).copy_(st["exp_avg"].to(a.exp_avg.device).view(a.shapes[n]))
        a.view(a.exp_avg_sq, n).copy_(st["exp_avg_sq"].to(a.exp_avg.device).view(a.shapes[n]))
        step = max(step, int(float(st["step"])))
    engine.step_count = step


def save_checkpoint(path: str, model, engine, optimizer, iter_num: int, best_val_loss: float, *,
                    lr: float, betas, weight_decay: float) -> None:
    model_sd = {k: v.detach().cpu().clone() for k, v in model.state_dict().items()}
    if engine is not None:
        opt_sd = _optimizer_state_from_engine(engine, lr, betas, weight_decay)
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
    model.load_state_dict(ckpt["model"])
    if engine is not None:
        engine.arena.refresh_shadow()
        _optimizer_state_into_engine(engine, ckpt["optimizer"])
        if "engine" in ckpt:
            engine.fwd_count = ckpt["engine"].get("fwd_count", engine.fwd_count)
    elif optimizer is not None:
        optimizer.load_state_dict(ckpt["optimizer"])
    return {"iter_num": ckpt["iter_num"], "best_val_loss": ckpt["best_val_loss"]}
