"""External baselines of the reference registry: ``maia`` (lc0 with Maia weights over UCI) and
``gpt-3.5-turbo`` (a text-completion model prompted with PGN).  Both need things this package cannot
ship (the lc0 binary and weight files; network access and credentials), so they register themselves
and raise a clear error on construction when their dependency is missing (reference
``src/evaluation/decode.py:128-182, 661-731``).  ``GPT35Turbo`` accepts any completion function, so
the prompting, parsing and caching logic is usable (and tested) without the network."""
from __future__ import annotations

import os
import random

import torch

from ..data import Game
from ..evaluation.chess_llm import ChessLLM, Completion, openai_completion
from ..evaluation.uci import EngineUnavailable, UCIEngine
from .strategies import DECODE_STRATEGIES, DecodeStrategy, ScoreResult


class Maia(DecodeStrategy):
    """Maia networks (1100..1900) through ``lc0``, one node per move.  ``maia_elo=None`` loads every
    network found and plays the one rated closest to the side to move; with ``opening_strategy``
    the first ten plies are answered by that strategy instead (the server gives Maia the policy
    system as its opening book)."""

    def __init__(self, model=None, tokenizer=None, sample=False, device=None, precision="float32",
                 maia_elo: int | None = None, maia_weights_dir: str = "maia-weights",
                 opening_strategy: DecodeStrategy | None = None, engine_path: str = "lc0", **kwargs):
        self.model, self.tokenizer, self.sample = model, tokenizer, False
        self.opening_strategy = opening_strategy
        self.engines: dict[int, UCIEngine] = {}
        for elo in (range(1100, 2000, 100) if maia_elo is None else [maia_elo]):
            for name in (f"maia-{elo}.pb", f"maia-{elo}.pb.gz"):
                w = os.path.join(maia_weights_dir, name)
                if os.path.exists(w):
                    self.engines[elo] = UCIEngine(engine_path, {"Threads": 4, "WeightsFile": w})
                    break
        if not self.engines:
            raise EngineUnavailable(f"Maia needs the lc0 binary and maia-<elo>.pb weights in {maia_weights_dir!r}")

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        if self.opening_strategy is not None and len(game.moves) < 10:
            return self.opening_strategy.score_full(game, legal_moves)
        elo = game.white_elo if game.board.turn else game.black_elo
        assert elo is not None, game
        best = min(self.engines, key=lambda e: abs(e - elo))
        _, _, mv = self.engines[best].analyse(game.moves, nodes=1)
        probs = torch.zeros(len(legal_moves))
        probs[legal_moves.index(mv)] = 1.0
        return ScoreResult(probs)

    def cleanup(self) -> None:
        for e in self.engines.values():
            e.quit()
        if self.opening_strategy is not None:
            self.opening_strategy.cleanup()


class GPT35Turbo(DecodeStrategy):
    """Plays the first legal move of a completion model's continuation of the game's PGN; a random
    legal move when the continuation starts with an illegal one.  The completion function comes
    from ``complete=``, else from the key file named by ``api_key_file`` / ``$OPENAI_API_KEY_FILE``
    or the key in ``$OPENAI_API_KEY``.  The continuation beyond the first move is remembered as
    the answer for the positions it passes through (keyed by the move list)."""

    def __init__(self, model=None, tokenizer=None, sample=False, device=None, precision="float32",
                 complete: Completion | None = None, api_key_file: str | None = None,
                 cache_path: str | None = None, dryrun: bool = False, **kwargs):
        self.model, self.tokenizer, self.sample, self.dryrun = model, tokenizer, False, dryrun
        if complete is None:
            key = os.environ.get("OPENAI_API_KEY")
            path = api_key_file or os.environ.get("OPENAI_API_KEY_FILE")
            if path and os.path.exists(path):
                with open(path) as f:
                    key = f.read().strip()
            if not key:
                raise EngineUnavailable("the gpt-3.5-turbo baseline needs a completion function or an "
                                        "OpenAI API key (OPENAI_API_KEY / OPENAI_API_KEY_FILE) and network access")
            complete = openai_completion(key, "gpt-3.5-turbo-instruct", 0.0)
        self.requests = 0

        def counted(prompt: str, max_tokens: int) -> str:
            self.requests += 1
            return complete(prompt, max_tokens)

        self.chessllm = ChessLLM(counted, {"num_lookahead_tokens": 20}, cache_path=cache_path)
        self.cache: dict[str, str] = {}

    def make_move(self, game: Game) -> str:
        board = game.board
        state = " ".join(board.move_stack)
        if state in self.cache:
            return self.cache[state]
        prompt = self.chessllm.get_query_pgn(board)
        sans = self.chessllm.try_moves(board, self.chessllm.make_request(prompt, 20)) if prompt else []
        walk = board.copy()
        first = None
        for san in sans:
            key = " ".join(walk.move_stack)
            uci = walk.push_san(san)
            self.cache[key] = uci
            first = first or uci
        return first if first is not None else random.choice(game.legal_moves)

    def score_full(self, game: Game, legal_moves: list[str]) -> ScoreResult:
        probs = torch.zeros(len(legal_moves))
        probs[legal_moves.index(self.make_move(game))] = 1.0
        return ScoreResult(probs)

    def run_stats(self) -> dict:
        return {"completion_requests": self.requests}


DECODE_STRATEGIES.setdefault("maia", Maia)
DECODE_STRATEGIES.setdefault("gpt-3.5-turbo", GPT35Turbo)
