"""C++ move generator: perft counts, vocabulary parity, move order and terminal detection (CPU)."""
import pytest

from allie_b200.chess import Board, vocab_uci
from allie_b200.data import Game
from allie_b200.moves import CHESS_MOVES

PERFT = [
    (None, [20, 400, 8902, 197281]),
    ("r3k2r/p1ppqpb1/bn2pnp1/3PN3/1p2P3/2N2Q1p/PPPBBPPP/R3K2R w KQkq - 0 1", [48, 2039, 97862]),
    ("8/2p5/3p4/KP5r/1R3p1k/8/4P1P1/8 w - - 0 1", [14, 191, 2812, 43238]),
    ("r3k2r/Pppp1ppp/1b3nbN/nP6/BBP1P3/q4N2/Pp1P2PP/R2Q1RK1 w kq - 0 1", [6, 264, 9467]),
    ("rnbq1k1r/pp1Pbppp/2p5/8/2B5/8/PPP1NnPP/RNBQK2R w KQ - 1 8", [44, 1486, 62379]),
    ("r4rk1/1pp1qppp/p1np1n2/2b1p1B1/2B1P1b1/P1NP1N2/1PP1QPPP/R4RK1 w - - 0 10", [46, 2079, 89890]),
]


@pytest.mark.parametrize("fen,counts", PERFT)
def test_perft(fen, counts):
    b = Board(fen)
    for depth, want in enumerate(counts, start=1):
        assert b.perft(depth) == want, (fen, depth)


def test_vocab_matches_python_table():
    for i in (0, 1, 20, 1455, 1456, 1791, 1792, 1800, 1967):
        assert vocab_uci(i) == CHESS_MOVES[i]
    assert all(vocab_uci(i) == CHESS_MOVES[i] for i in range(0, 1968, 37))


def test_start_position_order():
    # python-chess order: knights (g1 before b1, targets high square first), then pawn single pushes
    # from h to a, then double pushes from h to a
    want = ["g1h3", "g1f3", "b1c3", "b1a3", "h2h3", "g2g3", "f2f3", "e2e3", "d2d3", "c2c3", "b2b3", "a2a3",
            "h2h4", "g2g4", "f2f4", "e2e4", "d2d4", "c2c4", "b2b4", "a2a4"]
    assert Board().legal_moves_uci() == want


def test_castling_promotion_en_passant():
    b = Board()
    for m in "e2e4 e7e5 g1f3 b8c6 f1c4 f8c5".split():
        b.push_uci(m)
    assert "e1g1" in b.legal_moves_uci()
    b.push_uci("e1g1")
    assert b.piece_at(6) == 6 and b.piece_at(5) == 4      # king g1, rook f1
    b2 = Board()
    for m in "e2e4 a7a6 e4e5 d7d5".split():
        b2.push_uci(m)
    assert "e5d6" in b2.legal_moves_uci()
    b2.push_uci("e5d6")
    assert b2.piece_at(35) == 0                            # captured pawn on d5 is gone
    b3 = Board("8/P6k/8/8/8/8/8/K7 w - - 0 1")
    assert b3.legal_moves_uci()[-4:] == ["a7a8q", "a7a8r", "a7a8b", "a7a8n"]
    with pytest.raises(ValueError):
        Board().push_uci("e2e5")


def test_terminal_detection():
    b = Board()
    for m in "f2f3 e7e5 g2g4 d8h4".split():
        b.push_uci(m)
    assert b.is_game_over() and b.outcome().termination == "checkmate" and b.outcome().winner is False
    assert Board("7k/5Q2/6K1/8/8/8/8/8 b - - 0 1").outcome().termination == "stalemate"
    assert Board("8/8/8/8/8/2k5/8/K1B5 w - - 0 1").outcome().termination == "insufficient_material"
    assert Board("8/8/8/8/8/2k5/8/K1R5 w - - 0 1").outcome() is None
    assert Board("8/8/8/8/8/2k5/8/K1R5 w - - 150 100").outcome().termination == "seventyfive_moves"
    b = Board()
    for _ in range(4):
        for m in "g1f3 g8f6 f3g1 f6g8".split():
            assert not b.is_game_over()
            b.push_uci(m)
    assert b.outcome().termination == "fivefold_repetition" and b.outcome().winner is None


def test_game_board_and_legal_moves():
    g = Game("180+0", 1500, 1500, None, False, ["e2e4", "e7e5"], [1, 2])
    assert g.board.turn is True and len(g.board.move_stack) == 2
    assert len(g.legal_moves) == 29
    g2 = g.make_move("g1f3")
    assert g2.moves[-1] == "g1f3" and g2.moves_seconds[-1] == 0 and len(g.moves) == 2


def test_legal_move_order_follows_python_chess_generation_order():
    """Golden move orders, written down by hand from python-chess's generation algorithm (not
    produced by this repository's generator): pieces other than pawns from the highest square to the
    lowest, each with its targets from the highest square to the lowest; then castling; then pawn
    captures (promotions as q, r, b, n), single pushes, double pushes, en passant; in check, king
    moves first and then the moves that capture or block the checker.  The search takes the FIRST
    best child and indexes its priors in this order, so the order is part of the behaviour."""
    from allie_b200.chess import Board

    cases = {
        # rook and king moves, castling, a promotion push
        "4k3/P7/8/8/8/8/8/4K2R w K - 0 1":
            "h1h8 h1h7 h1h6 h1h5 h1h4 h1h3 h1h2 h1g1 h1f1 e1f2 e1e2 e1d2 e1f1 e1d1 e1g1 a7a8q a7a8r a7a8b a7a8n",
        # black to move with an en-passant capture available (generated last)
        "4k3/8/8/8/3pP3/8/8/4K3 b - e3 0 1": "e8f8 e8d8 e8f7 e8e7 e8d7 d4d3 d4e3",
        # in check from a rook on the king's file: only king moves off the file (the bishop's way to
        # the blocking square is shut by its own pawn)
        "4r1k1/8/8/8/8/8/3P4/2B1K3 w - - 0 1": "e1f2 e1f1 e1d1",
        # king steps around a knight's attacks; capture-promotions before the plain capture, then
        # push-promotions, single and double pushes
        "1r2k3/P7/8/8/8/2n5/1P6/4K3 w - - 0 1":
            "e1f2 e1d2 e1f1 a7b8q a7b8r a7b8b a7b8n b2c3 a7a8q a7a8r a7a8b a7a8n b2b3 b2b4",
    }
    for fen, want in cases.items():
        assert Board(fen).legal_moves_uci() == want.split(), fen
    # a middlegame position (Ruy Lopez after 3.Bb5, black to move)
    b = Board()
    for m in "e2e4 e7e5 g1f3 b8c6 f1b5".split():
        b.push_uci(m)
    assert b.legal_moves_uci() == (
        "g8e7 g8h6 g8f6 f8e7 f8d6 f8c5 f8b4 f8a3 e8e7 d8e7 d8f6 d8g5 d8h4 a8b8 c6b8 c6e7 c6a5 c6d4 c6b4 "
        "h7h6 g7g6 f7f6 d7d6 b7b6 a7a6 h7h5 g7g5 f7f5 d7d5 a7a5").split()
