"""Batched MCTS: the C++ tree search (``csrc/mcts.cpp``) driven against a batch evaluator.

``BatchedMCTS.search(games)`` runs one independent search per game, all trees advancing in
lock-step: select a leaf per tree on the CPU, evaluate all leaves in one GPU step, expand and back
up.  Two evaluators exist: :class:`KVStepEvaluator` (the KV-cached sm_100a evaluator, one token of
compute per leaf) and :class:`RunnerStepEvaluator` (re-encodes each leaf's game through a
:class:`~allie_b200.search.runner.ModelRunner`; the CPU path and the bridge to the sequential
oracle in the tests).  Results carry what the strategies of the reference return: visit counts,
the KL-regularised policy, think time, resign flag.
"""
from __future__ import annotations

from time import perf_counter
from ctypes import POINTER, c_float, c_int, c_void_p
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

from ..data import Game, UCITokenizer, undo_time_normalization
from ..moves import CHESS_MOVES
from ..ops import _lib
from .strategies import kl_regularized_policy_np

_cfg_done = False


def _lib_mcts():
    global _cfg_done
    lib = _lib.host()
    if not _cfg_done:
        lib.mcts_create.restype = c_void_p
        lib.mcts_create.argtypes = [c_int, c_float, c_float, c_int, c_int]
        lib.mcts_destroy.argtypes = [c_void_p]
        ip, fp = POINTER(c_int), POINTER(c_float)
        lib.mcts_set_root.argtypes = [c_void_p, c_int, ip, c_int, c_int, c_int, ip, c_int]
        lib.mcts_root_turn.argtypes = [c_void_p, c_int]
        lib.mcts_expand_root.argtypes = [c_void_p, c_int, ip, fp, c_int]
        lib.mcts_set_budget.argtypes = [c_void_p, c_int, c_int]
        lib.mcts_sims_done.argtypes = [c_void_p, c_int]
        lib.mcts_select.argtypes = [c_void_p, fp, ip, ip, ip, ip, ip, c_int, ip, ip, c_int, ip]
        lib.mcts_backup.argtypes = [c_void_p, fp, c_int, fp, c_int]
        lib.mcts_root_stats.argtypes = [c_void_p, c_int, ip, ip, fp, fp, c_int]
        lib.mcts_node_count.argtypes = [c_void_p, c_int]
        _cfg_done = True
    return lib


def _ip(a: np.ndarray):
    return a.ctypes.data_as(POINTER(c_int))


def _fp(a: np.ndarray):
    return a.ctypes.data_as(POINTER(c_float))


@dataclass
class SearchResult:
    legal_moves: list[str]
    visits: np.ndarray
    priors: np.ndarray
    values: np.ndarray
    policy: torch.Tensor            # final move distribution over legal_moves
    think_time: float | None
    resigned: bool
    root_value: float
    n_sims: int


class RunnerStepEvaluator:
    """Evaluates leaves by re-encoding their whole games (any ModelRunner; CPU capable)."""

    def __init__(self, runner, tokenizer: UCITokenizer, n_trees: int, anc_max: int, legal_max: int):
        self.runner, self.tok, self.n = runner, tokenizer, n_trees
        self.anc_max, self.legal_max = anc_max, legal_max
        self.games: list[Game | None] = [None] * n_trees
        self.slot_tok: list[dict[int, int]] = [dict() for _ in range(n_trees)]
        self.positions = 0

    def prefill(self, games: list[Game | None]):
        self.games = list(games)
        self.slot_tok = [dict() for _ in range(self.n)]
        live = [g for g in games if g is not None]
        ev = self.runner.evaluate(live)
        V = ev.logits.size(1)
        logits, value, time = torch.zeros(self.n, V), torch.zeros(self.n), torch.zeros(self.n)
        j = 0
        for i, g in enumerate(games):
            if g is not None:
                logits[i], value[i], time[i] = ev.logits[j], ev.value[j], ev.time[j]
                j += 1
        return logits, value, time

    def step(self, req: dict) -> tuple[np.ndarray, np.ndarray]:
        need = np.nonzero(req["need_eval"])[0]
        priors = np.zeros((self.n, self.legal_max), dtype=np.float32)
        value = np.zeros(self.n, dtype=np.float32)
        games = []
        for t in need:
            na = int(req["n_anc"][t])
            slots = req["anc"][t, :na]
            self.slot_tok[t][int(req["slot"][t])] = int(req["tok"][t])
            g = self.games[t]
            for s in slots:
                g = g.make_move(CHESS_MOVES[self.slot_tok[t][int(s)]])
            games.append(g)
        if games:
            ev = self.runner.evaluate(games)
            self.positions += len(games)
            for j, t in enumerate(need):
                nl = int(req["n_legal"][t])
                ids = torch.from_numpy(req["legal"][t, :nl].astype(np.int64))
                priors[t, :nl] = F.softmax(ev.logits[j][ids], 0).numpy()
                value[t] = float(ev.value[j])
        return priors, value


class KVStepEvaluator:
    """Adapter of :class:`~allie_b200.search.evaluator.KVLeafEvaluator` to the search loop."""

    def __init__(self, engine, tokenizer: UCITokenizer, n_trees: int, anc_max: int, legal_max: int,
                 max_prefix: int = 320, max_nodes: int = 512, use_graph: bool = True):
        from .evaluator import KVLeafEvaluator

        self.kv = KVLeafEvaluator(engine, n_trees, max_prefix, max_nodes, anc_max, legal_max, use_graph)
        self.tok, self.n = tokenizer, n_trees
        self.anc_max, self.legal_max = anc_max, legal_max
        self.max_slots = self.kv.S
        self.max_positions = int(engine.cfg.n_positions)
        self.positions = 0

    def prefill(self, games: list[Game | None]):
        rows = []
        for g in games:
            if g is None:
                rows.append(np.array([self.tok.bos_token_id], dtype=np.int64))
            else:
                rows.append((self.tok.tokenize(g)[: self.tok.max_length] & 0x3FFF).astype(np.int64))
        return self.kv.prefill(rows)

    def step(self, req: dict) -> tuple[np.ndarray, np.ndarray]:
        kv = self.kv
        h = kv.req_host
        for name, key in (("active", "need_eval"), ("tok", "tok"), ("pos", "pos"), ("slot", "slot"),
                          ("n_anc", "n_anc"), ("n_legal", "n_legal"), ("anc", "anc"), ("legal", "legal")):
            kv.view(h, name).numpy()[...] = req[key]
        out = kv.step()
        self.positions += int(req["need_eval"].sum())
        return out[:, : self.legal_max], out[:, self.legal_max]


class BatchedMCTS:
    def __init__(self, tokenizer: UCITokenizer, evaluator, n_trees: int, n_sims: int = 50,
                 c_puct: float = 1.25, c_base: float = 19652.0, depth_limit: int = 100,
                 kl_reg_solution: bool = True, dummy_value_function: bool = False,
                 anc_max: int = 128, legal_max: int = 224, max_slots: int | None = None):
        self.tok, self.ev, self.n = tokenizer, evaluator, n_trees
        self.n_sims, self.c_puct, self.c_base = n_sims, c_puct, c_base
        self.depth_limit = min(depth_limit, anc_max - 1)
        self.kl, self.dummy = kl_reg_solution, dummy_value_function
        self.anc_max, self.legal_max = anc_max, legal_max
        self.max_slots = max_slots if max_slots is not None else getattr(evaluator, "max_slots", 1 << 30)
        self.lib = _lib_mcts()
        self.h = self.lib.mcts_create(n_trees, c_puct, c_base, self.depth_limit, self.max_slots)
        n = n_trees
        i32 = np.int32
        self.req = dict(need_eval=np.zeros(n, i32), tok=np.zeros(n, i32), pos=np.zeros(n, i32),
                        slot=np.zeros(n, i32), n_anc=np.zeros(n, i32), n_legal=np.zeros(n, i32),
                        anc=np.zeros((n, anc_max), i32), legal=np.zeros((n, legal_max), i32))
        self.total_rollouts = 0
        # host wall-clock seconds spent in the three phases of the search loop (select on the CPU,
        # leaf evaluation on the GPU including its copies, backup on the CPU)
        self.phase_seconds = {"select": 0.0, "evaluate": 0.0, "backup": 0.0}

    def __del__(self):
        try:
            self.lib.mcts_destroy(self.h)
        except Exception:
            pass

    def search(self, games: list[Game], n_sims=None, c_puct_per_tree=None) -> list[SearchResult]:
        """``n_sims``: an int, or a callable mapping the root's normalised think-time prediction to
        a budget (adaptive search)."""
        assert len(games) <= self.n
        n = self.n
        padded: list[Game | None] = list(games) + [None] * (n - len(games))
        legal_buf = np.zeros(self.legal_max, np.int32)
        root_legal: list[np.ndarray] = []
        for t, g in enumerate(padded):
            if g is None:
                self.lib.mcts_set_root(self.h, t, _ip(legal_buf), 0, 1, 0, _ip(legal_buf), self.legal_max)
                root_legal.append(np.zeros(0, np.int32))
                continue
            ids = np.array([self.tok.token_to_id[m] for m in g.moves], dtype=np.int32)
            prefix_len = min(len(self.tok.tokenize(g)), self.tok.max_length)
            nl = self.lib.mcts_set_root(self.h, t, _ip(ids), len(ids), prefix_len, 0, _ip(legal_buf), self.legal_max)
            if nl < 0:
                raise ValueError(f"illegal move in game {t}")
            root_legal.append(legal_buf[:nl].copy())
            # a leaf at depth k sits at position prefix_len + k - 1 of the learned position table
            limit = getattr(self.ev, "max_positions", None)
            if limit is not None and prefix_len + self.depth_limit > limit:
                raise ValueError(f"game {t}: {prefix_len} tokens plus a search depth of {self.depth_limit} exceed "
                                 f"the model's {limit} positions; lower depth_limit or the tokenizer's max_length")
        logits, value, time = self.ev.prefill(padded)
        budgets = np.zeros(n, np.int32)
        cp = np.full(n, self.c_puct, np.float32)
        for t, g in enumerate(padded):
            if g is None or len(root_legal[t]) == 0:
                continue
            ids = torch.from_numpy(root_legal[t].astype(np.int64))
            pri = F.softmax(logits[t][ids], 0).numpy().astype(np.float32)
            self.lib.mcts_expand_root(self.h, t, _ip(root_legal[t]), _fp(pri), len(pri))
            b = n_sims(float(time[t]), g) if callable(n_sims) else (self.n_sims if n_sims is None else int(n_sims))
            budgets[t] = b
            if c_puct_per_tree is not None:
                cp[t] = c_puct_per_tree(b)
            self.lib.mcts_set_budget(self.h, t, int(b))
        r = self.req
        ph = self.phase_seconds
        clock = perf_counter
        while True:
            t0 = clock()
            nreq = self.lib.mcts_select(self.h, _fp(cp), _ip(r["need_eval"]), _ip(r["tok"]), _ip(r["pos"]),
                                        _ip(r["slot"]), _ip(r["anc"]), self.anc_max, _ip(r["n_anc"]),
                                        _ip(r["legal"]), self.legal_max, _ip(r["n_legal"]))
            t1 = clock()
            ph["select"] += t1 - t0
            if nreq == 0:
                break
            pri, val = self.ev.step(r)
            pri = np.ascontiguousarray(pri, dtype=np.float32)
            val = np.ascontiguousarray(val, dtype=np.float32)
            t2 = clock()
            ph["evaluate"] += t2 - t1
            self.lib.mcts_backup(self.h, _fp(pri), pri.shape[1], _fp(val), int(self.dummy))
            ph["backup"] += clock() - t2
        results = []
        mv = np.zeros(self.legal_max, np.int32); vis = np.zeros(self.legal_max, np.int32)
        pr = np.zeros(self.legal_max, np.float32); va = np.zeros(self.legal_max, np.float32)
        for t, g in enumerate(games):
            nc = self.lib.mcts_root_stats(self.h, t, _ip(mv), _ip(vis), _fp(pr), _fp(va), self.legal_max)
            legal = [CHESS_MOVES[i] for i in mv[:nc]]
            visits, priors, values = vis[:nc].copy(), pr[:nc].copy(), va[:nc].copy()
            done = int(budgets[t])
            self.total_rollouts += done
            lg = logits[t]
            ids = torch.from_numpy(root_legal[t].astype(np.int64))
            raw_value = float(value[t])
            pov = 1 if self.lib.mcts_root_turn(self.h, t) else -1     # the search already replayed the game
            resigned = bool(nc > 0 and float(lg[self.tok.resigned_token_id]) > float(lg[ids].max())
                            and pov * raw_value < -0.9)
            if nc == 0:
                policy = torch.zeros(0)
            elif done == 0 or visits.sum() == 0:
                policy = torch.from_numpy(priors.copy())
            elif not self.kl:
                policy = torch.from_numpy(visits.astype(np.float32) / visits.sum())
            else:
                policy = torch.from_numpy(kl_regularized_policy_np(priors, values, visits, float(cp[t])))
            results.append(SearchResult(legal, visits, priors, values, policy,
                                        undo_time_normalization(float(time[t])), resigned, raw_value, done))
        return results
