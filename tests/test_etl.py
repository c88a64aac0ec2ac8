"""Data preparation: SAN resolution, PGN rows, tokenised stream (CPU)."""
import json

import numpy as np

from allie_b200.chess import Board
from allie_b200.data import UCITokenizer
from allie_b200.etl.dataset import concat, elo_stats, random_games, tokenize
from allie_b200.etl.pgn import parse_game, san_to_uci

PGN = '''[Event "Rated Blitz game"]
[White "a"]
[Black "b"]
[Result "1-0"]
[WhiteElo "1500"]
[BlackElo "1600"]
[TimeControl "180+2"]
[Termination "Normal"]

1. e4 { [%clk 0:03:00] } 1... e5 { [%clk 0:03:00] } 2. Nf3 { [%clk 0:02:58] } 2... Nc6 { [%clk 0:02:59] } 3. Bc4 { [%clk 0:02:55] } 3... Nf6 { [%clk 0:02:50] } 4. O-O { [%clk 0:02:50] } 4... Bc5 { [%clk 0:02:45] } 5. d3 { [%clk 0:02:45] } 5... d6 { [%clk 0:02:40] } 1-0
'''


def test_san_resolution():
    b = Board()
    assert san_to_uci(b, "e4") == "e2e4" and san_to_uci(b, "Nf3") == "g1f3"
    b = Board("8/P6k/8/8/8/8/8/K7 w - - 0 1")
    assert san_to_uci(b, "a8=Q+") == "a7a8q"
    b = Board("r3k2r/8/8/8/8/8/8/R3K2R w KQkq - 0 1")
    assert san_to_uci(b, "O-O-O") == "e1c1" and san_to_uci(b, "Rad1") == "a1d1"


def test_parse_game_and_stream(tmp_path):
    row = parse_game(PGN)
    assert row["moves-uci"].split()[:4] == ["e2e4", "e7e5", "g1f3", "b8c6"] and row["moves-uci"].split()[6] == "e1g1"
    assert row["moves-seconds"][0] == 2 and row["moves-seconds"][2] == 4 and len(row["moves-seconds"]) == 10
    assert parse_game(PGN.replace("Blitz", "Bullet")) is None
    random_games(str(tmp_path / "g.jsonl"), n=20, max_plies=30)
    rows = [json.loads(l) for l in open(tmp_path / "g.jsonl")]
    assert len(rows) == 20 and all(len(r["moves-uci"].split()) == len(r["moves-seconds"]) for r in rows)
    tok = UCITokenizer(max_length=64)
    n = tokenize(str(tmp_path / "g.jsonl"), str(tmp_path / "a.bin"), tokenizer=tok)
    assert n == np.memmap(tmp_path / "a.bin", dtype=np.uint32, mode="r").size
    assert concat([str(tmp_path / "a.bin"), str(tmp_path / "a.bin")], str(tmp_path / "c.bin")) == 2 * n
    st = elo_stats(str(tmp_path / "g.jsonl"), str(tmp_path / "hist.json"))
    assert st["n"] == 40 and sum(st["histogram"]) == 20 and json.load(open(tmp_path / "hist.json")) == st["histogram"]


def test_position_values_and_puzzles(tmp_path):
    from allie_b200.etl.dataset import position_values, puzzles

    src = tmp_path / "g.jsonl"
    src.write_text(json.dumps({"moves-uci": "e2e4 e7e5 g1f3"}) + "\n")
    n = position_values(str(src), evaluator=lambda moves, nodes: 100 * len(moves))   # white-relative cp
    row = json.loads(src.read_text())
    assert n == 1 and row["moves-eval"] == [100, -200, 300]
    assert abs(row["position-values"][0] - (2 / (1 + np.exp(-0.368208)) - 1)) < 1e-9
    assert row["position-values"][1] < 0 < row["position-values"][2] < 1

    csv_path = tmp_path / "p.csv"
    lines = ["PuzzleId,FEN,Moves,Rating,Themes,GameUrl"]
    for i in range(30):
        lines.append(f"p{i},8/8/8/8/8/8/8/K6k w - - 0 1,a1a2,1500,short mateIn{i % 5 + 1},https://lichess.org/game{i}/black#10")
    csv_path.write_text("\n".join(lines) + "\n")
    fetched = []
    ids = puzzles(str(csv_path), str(tmp_path / "out"), per_theme=4, download=True,
                  fetch=lambda url: fetched.append(url) or b"[Event \"x\"]\n")
    assert sorted(ids) == [f"mateIn{k}" for k in range(1, 6)] and all(len(v) == 4 for v in ids.values())
    assert len(fetched) == 20 and fetched[0].startswith("https://lichess.org/game/export/game")
    assert len((tmp_path / "out" / "mateIn3.csv").read_text().splitlines()) == 5
    assert len(list((tmp_path / "out" / "pgn").iterdir())) == 20


def test_elo_balanced_sampling(tmp_path):
    from allie_b200.etl.dataset import elo_bin, keep_probability, sample

    assert elo_bin({"white-elo": 1449, "black-elo": 1450}) == 14 and elo_bin({"white-elo": "1551", "black-elo": 1550}) == 16
    assert keep_probability(15, {15: 400}, 100) == 0.25 and keep_probability(30, {15: 400}, 100) == 1.0
    src = tmp_path / "all.jsonl"
    with open(src, "w") as f:
        for i in range(3000):                                   # 2 400 games around 1500, 600 around 2200
            elo = 1500 if i % 5 else 2200
            f.write(json.dumps({"white-elo": elo, "black-elo": elo + 10, "moves-uci": "e2e4"}) + "\n")
    written = sample(str(src), str(tmp_path / "s"), target_per_bin=600, seed=1)
    rows = [json.loads(l) for l in open(tmp_path / "s-train.jsonl")]
    assert written["train"] == len(rows) and sum(written.values()) <= 3000
    low = sum(r["white-elo"] == 1500 for r in rows)
    high = sum(r["white-elo"] == 2200 for r in rows)
    assert 500 < low < 700 and 570 < high <= 600            # both bins end near the target


def _pgn_of_random_game(rng, plies, glue_numbers=False):
    """A Lichess-style PGN of a random legal game with clock comments on every move."""
    b = Board()
    clocks, parts, ucis = [180, 180], [], []
    for ply in range(plies):
        legal = b.legal_moves_uci()
        if not legal or b.is_game_over():
            break
        mv = legal[int(rng.integers(0, len(legal)))]
        san = b.san(mv)
        side = ply % 2
        clocks[side] = max(0, clocks[side] - int(rng.integers(0, 6)) + 2)
        clk = "{ [%%clk 0:%02d:%02d] }" % (clocks[side] // 60, clocks[side] % 60)
        if side == 0:
            parts.append(f"{ply // 2 + 1}.{san}" if glue_numbers else f"{ply // 2 + 1}. {san}")
        else:
            parts.append(f"{ply // 2 + 1}... {san}")
        parts.append(clk)
        b.push_uci(mv)
        ucis.append(mv)
    head = ('[Event "Rated Blitz game"]\n[Site "https://lichess.org/abc"]\n[Result "*"]\n[WhiteElo "1500"]\n'
            '[BlackElo "1600"]\n[TimeControl "180+2"]\n[Termination "Normal"]\n[Opening "?"]\n\n')
    return head + " ".join(parts) + " *\n", ucis


def test_native_pgn_parser_matches_python_parser():
    from allie_b200.etl.pgn import parse_movetext

    rng = np.random.default_rng(11)
    for k in range(12):
        text, ucis = _pgn_of_random_game(rng, int(rng.integers(10, 120)), glue_numbers=k % 3 == 0)
        fast, slow = parse_game(text), parse_game(text, native=False)
        assert fast == slow and fast is not None
        assert fast["moves-uci"].split() == ucis and fast["game-id"] == "https://lichess.org/abc"
        assert len(fast["moves-seconds"]) == len(ucis) and min(fast["moves-seconds"]) >= 0
    assert parse_game(PGN) == parse_game(PGN, native=False)
    assert parse_movetext("1. e4 e5 2. Ke3", 180, 0) is None                 # illegal move
    assert parse_movetext("1. e4 e5 2. Nf3 Nc6 3. Bb5 a6 4. O-O 1-0", 180, 0) == (
        ["e2e4", "e7e5", "g1f3", "b8c6", "f1b5", "a7a6", "e1g1"], [])
    assert parse_movetext("1. Nf3 Nf6 2. Ng1 Ng8 3. Nc3 Nc6 4. Nf3 Nf6 5. Nd4 Nd5 6. Ndb5 Ndb4", 60, 0)[0][-2:] == ["d4b5", "d5b4"]


def test_pgn_cli_reads_files_and_splits_games(tmp_path):
    from allie_b200.etl.pgn import main as pgn_main

    rng = np.random.default_rng(3)
    games = [_pgn_of_random_game(rng, 30) for _ in range(9)]
    (tmp_path / "dump.pgn").write_text("\n".join(text for text, _ in games))
    pgn_main([str(tmp_path / "dump.pgn"), str(tmp_path / "out.jsonl"), "--workers", "2"])
    rows = [json.loads(l) for l in open(tmp_path / "out.jsonl")]
    assert [r["moves-uci"].split() for r in rows] == [ucis for _, ucis in games]
