"""Game records, the UCI-move tokenizer and dataset loading.

Behavioural contract (reference ``src/modeling/data.py``):

* vocabulary = 1968 UCI moves + 24 blitz time controls + the resign/checkmate marker + BOS, EOS,
  UNK, PAD, optionally padded with ``<UNUSED-i`` entries up to a multiple
  (``data.py:175-213``); ids: moves 0..1967, time controls 1968..1991, resign 1992, BOS 1993,
  EOS 1994, UNK 1995, PAD 1996.
* a tokenised game is a ``uint32`` array; each word packs the token id (low 14 bits; the two
  leading ELO pseudo-tokens are ``elo + len(tokenizer)``), the game outcome (bits 14-15) and
  ``seconds + 1`` of the *next* move in the high 16 bits, 0 meaning "what follows is not a move"
  (``data.py:217-270``).
* ``pad_and_collate`` undoes the packing into ``input_ids / attention_mask / position_ids / labels /
  value_labels / time_labels`` (``data.py:281-337``).

The training path of this package does not run ``pad_and_collate`` on the host at all: the raw
``uint32`` window is shipped to the GPU and unpacked there (``csrc/embed.cu``); this module is the
CPU statement of the same arithmetic and what evaluation and serving use.
"""
from __future__ import annotations

import glob
import json
import logging
import os
from dataclasses import dataclass
from functools import cached_property
from typing import Any, Sequence

import numpy as np
import torch

from .moves import CHESS_MOVES

Batch = dict[str, torch.Tensor]
logger = logging.getLogger(__name__)

BLITZ_TIME_CONTROLS_TOKENS = [
    f"{base}+{inc}" for base, inc in (
        (180, 0), (300, 0), (180, 2), (300, 3), (300, 2), (420, 0), (240, 0), (180, 1), (180, 3),
        (300, 1), (360, 0), (300, 4), (420, 1), (240, 2), (180, 5), (120, 2), (120, 3), (240, 3),
        (240, 1), (360, 2), (60, 3), (60, 5), (240, 4), (240, 5))
]
NORMAL_TERMINATION_TOKEN = "<RESIGNED-OR-CHECKMATED>"

WHITE_WIN_MASK = 0x0000
DRAW_MASK = 0x4000
BLACK_WIN_MASK = 0x8000
OUTCOME_MASKS = {"1-0": WHITE_WIN_MASK, "1/2-1/2": DRAW_MASK, "0-1": BLACK_WIN_MASK}

# statistics of per-move seconds on the training set (reference data.py:156-157)
TIME_MEAN = 4.64001
TIME_STDEV = 6.16533

IGNORE = -100


def apply_time_normalization(t):
    """Clamp seconds to [0, 60] and standardise."""
    if isinstance(t, torch.Tensor):
        t = t.clamp(0, 60)
    else:
        t = min(max(t, 0), 60)
    return (t - TIME_MEAN) / TIME_STDEV


def undo_time_normalization(t_normed):
    return t_normed * TIME_STDEV + TIME_MEAN


@dataclass
class Game:
    """One (possibly partial) game.  ``to_dict`` is also the server wire format."""

    time_control: str | None
    white_elo: int | None
    black_elo: int | None
    outcome: str | None
    normal_termination: bool
    moves: list[str]
    moves_seconds: list[int]
    next_move_seconds: int | None = None

    @cached_property
    def board(self):
        from .chess import Board

        b = Board()
        for mv in self.moves:
            b.push_uci(mv)
        return b

    @cached_property
    def legal_moves(self) -> list[str]:
        return self.board.legal_moves_uci()

    def make_move(self, move: str) -> "Game":
        return Game(self.time_control, self.white_elo, self.black_elo, self.outcome,
                    self.normal_termination, self.moves + [move], self.moves_seconds + [0], None)

    def to_dict(self) -> dict:
        keys = ("time_control", "white_elo", "black_elo", "outcome", "normal_termination", "moves",
                "moves_seconds", "next_move_seconds")
        return {k: getattr(self, k) for k in keys}

    @classmethod
    def from_dict(cls, data: dict) -> "Game":
        return cls(**data)


@dataclass(frozen=True)
class PlayResult:
    move: str
    move_time: float | None


def json_to_game(d: dict) -> Game:
    """JSONL row -> Game; unknown results count as draws (reference data.py:89-99)."""
    result = d["result"]
    return Game(
        time_control=d["time-control"],
        white_elo=int(d["white-elo"]),
        black_elo=int(d["black-elo"]),
        outcome=result if result in OUTCOME_MASKS else "1/2-1/2",
        normal_termination=d["termination"] == "Normal",
        moves=d["moves-uci"].split(),
        moves_seconds=list(d["moves-seconds"]),
    )


def json_to_partial_game(d: dict, halfmove: int) -> Game:
    """Prefix of a game up to ``halfmove`` plies, remembering the human's next think time."""
    secs = list(d["moves-seconds"])
    return Game(
        time_control=d["time-control"],
        white_elo=int(d["white-elo"]),
        black_elo=int(d["black-elo"]),
        outcome=None,
        normal_termination=False,
        moves=d["moves-uci"].split()[:halfmove],
        moves_seconds=secs[:halfmove],
        next_move_seconds=secs[halfmove] if halfmove < len(secs) else None,
    )


class UCITokenizer:
    def __init__(self, max_length: int = 128, vocab_size_multiple_of: int = 1,
                 bos_token: str = "<BOS>", eos_token: str = "<EOS>", unk_token: str = "<UNK>",
                 pad_token: str = "<PAD>", **kwargs: Any):
        if kwargs:
            logger.warning(f"tokenizer got unrecognized arguments {kwargs}")
        self.max_length = max_length
        self.bos_token, self.eos_token = bos_token, eos_token
        self.unk_token, self.pad_token = unk_token, pad_token
        self.resigned_token = NORMAL_TERMINATION_TOKEN
        self.special_tokens = [bos_token, eos_token, unk_token, pad_token]
        self.tokens = list(CHESS_MOVES) + list(BLITZ_TIME_CONTROLS_TOKENS) + [self.resigned_token]
        self.tokens += self.special_tokens
        n_unused = (-len(self.tokens)) % vocab_size_multiple_of
        self.tokens += [f"<UNUSED-{i}" for i in range(n_unused)]
        self.token_to_id = {tok: i for i, tok in enumerate(self.tokens)}
        self.special_token_ids = [self.token_to_id[t] for t in self.special_tokens]
        self.bos_token_id = self.token_to_id[bos_token]
        self.eos_token_id = self.token_to_id[eos_token]
        self.unk_token_id = self.token_to_id[unk_token]
        self.pad_token_id = self.token_to_id[pad_token]
        self.resigned_token_id = self.token_to_id[self.resigned_token]

    def __len__(self) -> int:
        return len(self.tokens)

    # ------------------------------------------------------------------ encode
    def tokenize(self, game: Game, add_elo: bool = True, add_time_control: bool = True,
                 add_termination: bool = True, add_value: bool = True) -> np.ndarray:
        if add_elo:
            assert isinstance(game.white_elo, int) and isinstance(game.black_elo, int)
            words = [game.white_elo + len(self), game.black_elo + len(self)]
        else:
            words = [self.bos_token_id]
        assert isinstance(game.moves, list)
        secs = game.moves_seconds
        assert isinstance(secs, list) and len(secs) == len(game.moves)
        if add_time_control:
            assert isinstance(game.time_control, str)
            head = game.time_control
        else:
            head = self.unk_token
        # the word of token i carries the think time of the move that FOLLOWS it
        following = list(secs) + [-1]
        for tok, t in zip([head] + game.moves, following):
            t = -1 if t < 0 else t
            assert t < 0xFFFF, f"move time {t}s overflows 16-bit repr"
            words.append(self.token_to_id.get(tok, self.unk_token_id) + ((t + 1) << 16))
        if add_termination and game.normal_termination:
            words.append(self.resigned_token_id)
        if game.outcome is not None:
            words.append(self.eos_token_id)
        arr = np.array(words, dtype=np.uint32)
        if add_value and game.outcome is not None:
            assert game.outcome in OUTCOME_MASKS
            arr = arr | np.uint32(OUTCOME_MASKS[game.outcome])
        return arr

    def pad(self, seq: list[int]) -> list[int]:
        out = seq + [self.pad_token_id] * (self.max_length - len(seq))
        assert len(out) == self.max_length
        return out

    # ------------------------------------------------------------------ decode
    def unpack(self, data: torch.Tensor, return_labels: bool = True) -> Batch:
        """Packed int64 words [B, T] -> model inputs and labels."""
        enc = data >> 16
        seconds = apply_time_normalization(enc - 1)
        time_labels = torch.where(enc == 0, torch.full_like(seconds, IGNORE), seconds)
        outcomes = (data & 0xFFFF) >> 14
        assert int(outcomes.max()) < 3
        input_ids = data & 0x3FFF
        real = input_ids != self.pad_token_id
        labels = torch.where(real, input_ids, torch.full_like(input_ids, IGNORE))
        labels[labels >= len(self)] = IGNORE
        value_labels = torch.where(real, 1.0 - outcomes.to(torch.float32),
                                   torch.full(outcomes.shape, float(IGNORE)))
        out = {
            "input_ids": input_ids,
            "attention_mask": real.to(torch.float),
            "position_ids": (real.long().cumsum(-1) - 1).clamp(0),
            "value_labels": value_labels,
            "time_labels": time_labels,
        }
        if return_labels:
            out["labels"] = labels
        return out

    def pad_and_collate(self, games: Sequence[Game | np.ndarray], return_labels: bool = True) -> Batch:
        if isinstance(games[0], np.ndarray):
            data = torch.from_numpy(np.asarray(games).astype(np.int64))
        else:
            seqs = [self.tokenize(g)[: self.max_length].astype(np.int64) for g in games]
            width = max(len(s) for s in seqs)
            buf = np.full((len(seqs), width), self.pad_token_id, dtype=np.int64)
            for i, s in enumerate(seqs):
                buf[i, : len(s)] = s
            data = torch.from_numpy(buf)
        return self.unpack(data, return_labels)


class JsonlDataset:
    """Minimal stand-in for a HF ``datasets.Dataset`` over JSONL rows (list-like of dicts)."""

    def __init__(self, rows: list[dict]):
        self.rows = rows

    def __len__(self) -> int:
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]

    def __iter__(self):
        return iter(self.rows)

    @classmethod
    def from_glob(cls, pattern: str) -> "JsonlDataset":
        rows: list[dict] = []
        for path in sorted(glob.glob(pattern)):
            with open(path) as f:
                rows.extend(json.loads(line) for line in f if line.strip())
        return cls(rows)


def load_data(tokenizer_config: dict, train_file: str = "data/lichess-2022-blitz-train/2022.bin",
              eval_dir: str = "data/lichess-2022-blitz-sampled"):
    """``data_config`` entry point (reference data.py:340-362): a flat ``uint32`` memmap for
    training and JSONL validation / test splits found as ``*val.jsonl`` / ``*test.jsonl``."""
    tokenizer = UCITokenizer(**dict(tokenizer_config))
    train = np.memmap(train_file, dtype=np.uint32, mode="r")
    val = JsonlDataset.from_glob(os.path.join(eval_dir, "*val.jsonl"))
    test = JsonlDataset.from_glob(os.path.join(eval_dir, "*test.jsonl"))
    return tokenizer, (train, val, test)
