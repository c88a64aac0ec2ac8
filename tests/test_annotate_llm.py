"""Board text helpers (FEN, SAN), JSONL annotation and the PGN-prompted completion baseline, all on
CPU with fakes standing in for Stockfish and for the completion service."""
import json

import pytest

from allie_b200.chess import Board
from allie_b200.data import Game
from allie_b200.evaluation import annotate as ann
from allie_b200.evaluation.chess_llm import HEADER, ChessLLM
from allie_b200.search.external import GPT35Turbo

RUY = "e2e4 e7e5 g1f3 b8c6 f1b5 a7a6 b5c6 d7c6 e1g1".split()


def test_san_and_fen_roundtrip():
    b = Board()
    sans = []
    for mv in RUY:
        sans.append(b.san(mv))
        b.push_uci(mv)
    assert sans == ["e4", "e5", "Nf3", "Nc6", "Bb5", "a6", "Bxc6", "dxc6", "O-O"]
    assert b.fen() == "r1bqkbnr/1pp2ppp/p1p5/4p3/4P3/5N2/PPPP1PPP/RNBQ1RK1 b kq - 1 5"
    assert b.movetext() == "1. e4 e5 2. Nf3 Nc6 3. Bb5 a6 4. Bxc6 dxc6 5. O-O"
    c = Board()
    for s in sans:
        c.push_san(s)
    assert c.move_stack == RUY
    assert Board(b.fen()).fen() == b.fen()


def test_san_disambiguation_promotion_and_mate():
    assert Board("4k3/8/8/8/8/8/8/R3K2R w KQ - 0 1").san("a1d1") == "Rd1"
    assert Board("4k3/8/8/8/8/8/8/R6R w - - 0 1").san("a1d1") == "Rad1"
    assert Board("4k3/8/8/8/R7/8/8/R3K3 w - - 0 1").san("a1a2") == "R1a2"
    assert Board("7k/P7/8/8/8/8/8/K7 w - - 0 1").san("a7a8q") == "a8=Q+"
    b = Board()
    for mv in "f2f3 e7e5 g2g4".split():
        b.push_uci(mv)
    assert b.san("d8h4") == "Qh4#"
    with pytest.raises(ValueError):
        b.parse_san("Qh5")
    start = Board()
    assert start.parse_san("Ngf3") == "g1f3" and start.parse_san("e4!?") == "e2e4"   # over-specified / annotated
    with pytest.raises(ValueError):
        start.parse_san("Nbf3")


def test_en_passant_flag_and_fen_field():
    b = Board()
    for mv in "e2e4 a7a6 e4e5 d7d5".split():
        b.push_uci(mv)
    assert b.fen().split()[3] == "d6"
    assert b.is_en_passant("e5d6") and b.is_capture("e5d6") and b.san("e5d6") == "exd6"
    b2 = Board()
    b2.push_uci("e2e4")                     # no black pawn can take on e3: field stays empty
    assert b2.fen().split()[3] == "-"


def test_annotate_rows(tmp_path, monkeypatch):
    calls = []

    def fake_quality(moves, move):
        calls.append((len(moves), move))
        return float(len(moves)), 100.0 - len(moves)

    shuffle = "g1f3 g8f6 f3g1 f6g8 g1f3 g8f6 f3g1 f6g8"
    rows = [{"moves-uci": "e2e4 d7d5 e4e5 f7f5 e5f6 g8f6 g1f3 e7e6 f1e2 f8e7 e1g1", "white-elo": 1500},
            {"moves-uci": shuffle}]
    out = ann.annotate(rows, fake_quality)
    a = out[0]
    assert a["white-elo"] == 1500 and len(a["human-centipawn-loss"]) == 11
    assert a["human-centipawn-loss"][3] == 3.0 and a["human-lichess-accuracy"][3] == 97.0
    assert [i for i, x in enumerate(a["move-is-en-passant"]) if x] == [4]
    assert [i for i, x in enumerate(a["move-is-castling"]) if x] == [10]
    assert not any(a["move-is-promotion"]) and not any(a["move-is-threefold"])
    assert out[1]["move-is-threefold"] == [False] * 7 + [True]

    src = tmp_path / "games.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    monkeypatch.setattr(ann.eval_utils, "move_quality", fake_quality)
    dst = ann.main([str(src)])
    assert dst.endswith("games-annotated.jsonl")
    back = [json.loads(line) for line in open(dst)]
    assert back[1]["move-is-threefold"][-1] is True and len(back) == 2


def test_chess_llm_prompt_parse_and_cache(tmp_path):
    seen = []

    def complete(prompt, max_tokens):
        seen.append(prompt)
        return " Nf6 6. Re1 b5 7. Zz9 Bb3"

    b = Board()
    for mv in RUY:
        b.push_uci(mv)
    llm = ChessLLM(complete, cache_path=str(tmp_path / "cache.json"))
    assert llm.get_query_pgn(Board()) == HEADER + "1."
    assert llm.get_query_pgn(b) == HEADER + "1. e4 e5 2. Nf3 Nc6 3. Bb5 a6 4. Bxc6 dxc6 5. O-O"
    assert llm.get_best_move(b) == "Nf6"
    assert len(seen) == 1
    b.push_san("Nf6")
    assert llm.get_best_move(b) == "Re1" and len(seen) == 1        # predicted continuation served from cache
    again = ChessLLM(None, cache_path=str(tmp_path / "cache.json"))
    assert again.get_best_move(b) == "Re1"                         # and from the file, with no transport
    with pytest.raises(ValueError):
        ChessLLM(complete, num_lookahead_tokens=5)


def test_gpt35_strategy_with_fake_completion():
    answers = {"1.": " e4 e5 2. Nf3", }

    def complete(prompt, max_tokens):
        tail = prompt.split("\n\n")[1]
        return answers.get(tail, " Qxz9")

    s = GPT35Turbo(complete=complete)
    g = Game.from_dict({"time_control": "180+0", "white_elo": 1500, "black_elo": 1500, "outcome": None,
                        "normal_termination": None, "moves": [], "moves_seconds": [], "next_move_seconds": None})
    r = s.decode_full(g)
    assert r.move == "e2e4" and s.requests == 1
    g1 = g.make_move("e2e4")
    assert s.decode_full(g1).move == "e7e5" and s.requests == 1    # remembered continuation
    g3 = g1.make_move("e7e5").make_move("g1f3")
    mv = s.decode_full(g3).move                                    # illegal answer -> some legal move
    assert mv in g3.legal_moves and s.requests == 2
    assert s.run_stats() == {"completion_requests": 2}


def test_san_writer_and_both_parsers_agree_on_random_games():
    """Every legal move of positions along random games: SAN text -> move must give the move back,
    through the board's own parser and through the PGN reader's resolver."""
    import random

    from allie_b200.etl.pgn import san_to_uci

    rng = random.Random(7)
    checked = 0
    for _ in range(6):
        b = Board()
        for ply in range(60):
            legal = b.legal_moves_uci()
            if not legal or b.is_game_over():
                break
            sans = {}
            for mv in legal:
                s = b.san(mv)
                assert s == b.san_reference(mv), (b.fen(), mv, s)         # C++ writer against the Python statement
                assert s not in sans, (b.fen(), s, mv, sans[s])           # SAN is unambiguous
                sans[s] = mv
                if ply % 5 == 0:
                    assert b.parse_san(s) == mv and san_to_uci(b, s) == mv, (b.fen(), s, mv)
                    checked += 1
            b.push_uci(rng.choice(legal))
        assert Board(b.fen()).legal_moves_uci() == b.legal_moves_uci()
    assert checked > 500
