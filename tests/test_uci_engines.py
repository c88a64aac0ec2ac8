"""UCI client, Stockfish-based move quality and the Maia strategy against a fake engine process (CPU)."""
import os
import stat
import sys

import pytest
import torch

from allie_b200.data import Game
from allie_b200.evaluation import utils as eval_utils
from allie_b200.evaluation.uci import EngineUnavailable, UCIEngine
from allie_b200.search import DECODE_STRATEGIES
from allie_b200.search.external import Maia

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture()
def fake_engine(tmp_path):
    exe = tmp_path / "fake-engine"
    exe.write_text(f"#!/bin/sh\nexec {sys.executable} {os.path.join(HERE, 'fake_uci_engine.py')}\n")
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)
    return str(exe)


def test_client_and_move_quality(fake_engine, monkeypatch):
    eng = UCIEngine(fake_engine, {"Threads": 2})
    cp, mate, best = eng.analyse([], 1000)
    assert (cp, mate) == (0, None) and best == Board_first()
    cp, _, best = eng.analyse("e2e4 d7d5".split(), 10)
    assert cp == 0 and best == "e4d5"                       # the only capture
    cp, _, _ = eng.analyse("e2e4 d7d5 e4d5".split(), 10)
    assert cp == -100                                       # black to move, a pawn down
    eval_utils._eval_cached.cache_clear()
    monkeypatch.setattr(eval_utils, "_engine", eng)
    assert eval_utils.stockfish_eval("e2e4 d7d5 e4d5".split()) == 100          # white-relative
    loss, acc = eval_utils.move_quality("e2e4 d7d5".split(), "e4d5")
    assert loss == 0.0 and acc == 100.0
    loss, acc = eval_utils.move_quality("e2e4 d7d5 g1f3".split(), "d5e4")      # black wins a pawn
    assert loss == 0.0 and acc == 100.0
    loss, acc = eval_utils.move_quality("e2e4 d7d5 g1f3 d5e4".split(), "f3g1")  # white keeps the deficit
    assert loss == 0.0
    assert eval_utils.stockfish_eval_fen("4k3/8/8/8/8/8/8/R3K3 b - - 0 1") == 500       # white-relative at black's turn
    assert eval_utils.accuracy_from_win_percents(50.0, 60.0) == 100.0
    assert abs(eval_utils.accuracy_from_win_percents(60.0, 50.0) - (103.1668 * 2.718281828459045 ** -0.4354 - 3.1669)) < 1e-9
    assert eval_utils.accuracy_from_win_percents(100.0, 0.0) == 0.0
    eng.quit()
    with pytest.raises(EngineUnavailable):
        UCIEngine("/nonexistent/engine")


def Board_first():
    from allie_b200.chess import Board

    return Board().legal_moves_uci()[0]


class Book:
    """Opening strategy stub: always the last legal move."""

    def score_full(self, game, legal):
        from allie_b200.search import ScoreResult

        p = torch.zeros(len(legal))
        p[-1] = 1.0
        return ScoreResult(p)

    def cleanup(self):
        self.closed = True


def test_maia_picks_network_by_rating_and_uses_opening_book(fake_engine, tmp_path):
    assert DECODE_STRATEGIES["maia"] is Maia
    with pytest.raises(EngineUnavailable):
        Maia(maia_weights_dir=str(tmp_path / "none"), engine_path=fake_engine)
    wdir = tmp_path / "maia-weights"
    wdir.mkdir()
    for elo in (1100, 1500, 1900):
        (wdir / f"maia-{elo}.pb").write_bytes(b"x")
    book = Book()
    m = Maia(maia_weights_dir=str(wdir), engine_path=fake_engine, opening_strategy=book)
    assert sorted(m.engines) == [1100, 1500, 1900]
    g = Game("180+0", 1480, 1950, None, False, "e2e4 d7d5".split(), [1, 1])
    assert m.decode_full(g).move == g.legal_moves[-1]                      # ply 2 < 10: the book answers
    long = "g1f3 g8f6 f3g1 f6g8 g1f3 g8f6 f3g1 f6g8 e2e4 d7d5".split()
    g = Game("180+0", 1480, 1950, None, False, long, [1] * len(long))
    assert m.decode_full(g).move == "e4d5"                                 # the engine's capture
    one = Maia(maia_elo=1500, maia_weights_dir=str(wdir), engine_path=fake_engine)
    assert list(one.engines) == [1500] and one.decode(g) == "e4d5"
    m.cleanup(); one.cleanup()
    assert book.closed


def test_full_and_value_evaluation_with_fake_stockfish(fake_engine, monkeypatch):
    from allie_b200.evaluation.evaluate import evaluate, evaluate_value
    from allie_b200.search import ScoreResult

    class Greedy:
        """Strategy stub: all mass on the first legal move; white advantage 0.25 everywhere."""
        sample = False

        def score_full(self, game, legal):
            p = torch.zeros(len(legal))
            p[0] = 1.0
            return ScoreResult(p, white_advantage=0.25, top_move_legal=True, sampled_move_legal=0.5)

    eval_utils._eval_cached.cache_clear()
    monkeypatch.setattr(eval_utils, "_engine", UCIEngine(fake_engine))
    rows = [{"moves-uci": "e2e4 d7d5 e4d5", "moves-seconds": [1, 1, 1], "time-control": "180+0", "white-elo": 1500,
             "black-elo": 1500, "result": "1-0", "termination": "Normal"}]
    out = evaluate(Greedy(), rows, batch_size=2)
    rec = out["games"][0]
    assert out["positions"] == 3 and rec["human-move"] == ["e2e4", "d7d5", "e4d5"]
    assert rec["model-move"] == rec["top-move"] and len(rec["model-centipawn-loss"]) == 3
    # the fake engine counts material only, so a quiet move loses nothing by its measure
    assert rec["model-centipawn-loss"][2] == 0.0 and rec["model-lichess-accuracy"][2] == 100.0
    assert eval_utils._engine is None                        # the engine process is shut down at the end
    monkeypatch.setattr(eval_utils, "_engine", UCIEngine(fake_engine))
    eval_utils._eval_cached.cache_clear()
    val = evaluate_value(Greedy(), rows)
    assert val["games"][0]["stockfish-eval"] == [0, 0, 0] and val["games"][0]["model-white-advantage"] == [0.25] * 3
    assert abs(val["value_vs_stockfish_mse"] - 0.0625) < 1e-9
    eval_utils._engine.quit()
