"""PGN prompting of a text-completion model (reference ``src/evaluation/carlini.py:30-159``, used by
the ``gpt-3.5-turbo`` baseline at ``src/evaluation/decode.py:661-731``).

``ChessLLM`` turns a position into the PGN prefix a completion model is asked to continue (a fixed
four-tag header naming two world champions, then the movetext, ending in the next move number when
white is to move), sends it through a *completion function* and keeps the leading SAN moves of the
answer that are legal.  The transport is a parameter: ``complete(prompt, max_tokens) -> str``.  The
default transport posts to the OpenAI completions endpoint with ``urllib`` and needs an API key and
network access; tests and offline use pass their own function.  Answers are remembered per position
(FEN -> SAN) in memory and, when ``cache_path`` is given, in a JSON file.
"""
from __future__ import annotations

import json
import os
import urllib.request
from typing import Callable

from ..chess import Board

HEADER = ('[White "Magnus Carlsen"]\n[Black "Garry Kasparov"]\n'
          '[WhiteElo "2900"]\n[BlackElo "2800"]\n\n')
Completion = Callable[[str, int], str]


def openai_completion(api_key: str, model: str = "gpt-3.5-turbo-instruct", temperature: float = 0.0,
                      url: str = "https://api.openai.com/v1/completions") -> Completion:
    """A completion function backed by the OpenAI HTTP API."""

    def complete(prompt: str, max_tokens: int) -> str:
        body = json.dumps({"model": model, "prompt": prompt, "temperature": temperature,
                           "max_tokens": max_tokens}).encode()
        req = urllib.request.Request(url, data=body, headers={
            "Content-Type": "application/json", "Authorization": f"Bearer {api_key}"})
        with urllib.request.urlopen(req, timeout=60) as resp:
            return json.load(resp)["choices"][0]["text"]

    return complete


class ChessLLM:
    def __init__(self, complete: Completion | None, config: dict | None = None,
                 cache_path: str | None = None, **override):
        self.config = {"num_lookahead_tokens": 10, **(config or {}), **override}
        if self.config["num_lookahead_tokens"] < 9:
            raise ValueError("one move can take 9 tokens (3 for the number, 6 for e.g. 'N3xg5+')")
        self.complete = complete
        self.cache_path = cache_path
        self.cache: dict[str, str] = {}
        if cache_path and os.path.exists(cache_path):
            with open(cache_path) as f:
                self.cache = json.load(f)

    def get_query_pgn(self, board: Board) -> str | None:
        """The prompt for ``board``, or None when the game is over."""
        if board.outcome() is not None:
            return None
        # The reference prints the game with python-chess (movetext wrapped at 80 columns, result
        # marker "*" at the end), cuts the marker off and, with white to move, appends the number
        # of the coming move.
        text = board.movetext(columns=80, result="*")[:-1].strip()
        if board.turn:
            text = text + f" {board.fullmove_number}." if text else "1."
        return HEADER + text

    @staticmethod
    def try_moves(board: Board, next_text: str) -> list[str]:
        """Leading SAN tokens of ``next_text`` that play legally from ``board`` (move numbers skipped)."""
        board = board.copy()
        ok: list[str] = []
        for tok in next_text.split():
            if "." in tok:
                continue
            try:
                board.push_san(tok)
            except ValueError:
                break
            ok.append(tok)
        return ok

    def make_request(self, prompt: str, num_tokens: int) -> str:
        if self.complete is None:
            raise RuntimeError("ChessLLM has no completion function")
        text = self.complete(prompt, num_tokens)
        if text[:2] == "-O":            # a castling move split from its leading "O": ask again after a space
            text = self.complete(prompt + " ", num_tokens)
        return text

    def get_best_move(self, board: Board, num_tokens: int | None = None) -> str | None:
        """SAN of the model's move for ``board`` (None if its answer starts with an illegal move)."""
        key = board.fen()
        if key in self.cache:
            return self.cache[key]
        prompt = self.get_query_pgn(board)
        if prompt is None:
            return None
        moves = self.try_moves(board, self.make_request(prompt, num_tokens or self.config["num_lookahead_tokens"]))
        if not moves:
            return None
        walk = board.copy()
        for san in moves:                # the continuation is the model's prediction for later plies too
            self.cache[walk.fen()] = san
            walk.push_san(san)
        if self.cache_path:
            tmp = self.cache_path + ".tmp"
            with open(tmp, "w") as f:
                json.dump(self.cache, f)
            os.replace(tmp, self.cache_path)
        return moves[0]
