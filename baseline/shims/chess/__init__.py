"""Stand-in for python-chess (not installed here), so that the unmodified reference package can be
imported and its decode code run.  It offers the small part of the python-chess API that the
reference touches (``src/modeling/data.py:51-61``, ``src/evaluation/decode.py``,
``src/evaluation/carlini.py``): ``Board`` with ``push_uci / push / push_san / parse_san / san /
legal_moves / move_stack / turn / is_game_over / outcome / copy / fen / fullmove_number / ply``,
``Move`` with ``uci() / from_uci() / promotion`` and the colour constants.  The rules themselves come
from this repository's C++ move generator (``allie_b200/csrc/chess.hpp``), which lists legal moves
in python-chess order.  The reference's training path only imports the module.
"""
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
if _ROOT not in sys.path:
    sys.path.append(_ROOT)

WHITE, BLACK = True, False
PAWN, KNIGHT, BISHOP, ROOK, QUEEN, KING = range(1, 7)
_PROMO = {"n": KNIGHT, "b": BISHOP, "r": ROOK, "q": QUEEN}


class Move:
    def __init__(self, text: str):
        self._uci = text
        self.promotion = _PROMO.get(text[4:5])

    @classmethod
    def from_uci(cls, text: str) -> "Move":
        return cls(text)

    def uci(self) -> str:
        return self._uci

    def __eq__(self, other) -> bool:
        return isinstance(other, Move) and other._uci == self._uci

    def __hash__(self) -> int:
        return hash(self._uci)

    def __str__(self) -> str:
        return self._uci

    def __repr__(self) -> str:
        return f"Move.from_uci({self._uci!r})"


class _LegalMoves:
    def __init__(self, core):
        self._core = core

    def __iter__(self):
        return iter([Move(m) for m in self._core.legal_moves_uci()])

    def __len__(self) -> int:
        return len(self._core.legal_move_ids())

    def count(self) -> int:
        return len(self)

    def __contains__(self, move) -> bool:
        return str(move) in self._core.legal_moves_uci()


class Board:
    def __init__(self, fen=None, _core=None):
        from allie_b200.chess import Board as Core

        self._core = _core if _core is not None else Core(fen)
        self.move_stack = []

    @property
    def turn(self) -> bool:
        return self._core.turn

    @property
    def legal_moves(self) -> _LegalMoves:
        return _LegalMoves(self._core)

    @property
    def fullmove_number(self) -> int:
        return self._core.fullmove_number

    def ply(self) -> int:
        return self._core.ply()

    def push(self, move: Move) -> None:
        self._core.push_uci(move.uci())
        self.move_stack.append(move)

    def push_uci(self, text: str) -> Move:
        move = Move(text)
        self.push(move)
        return move

    def parse_san(self, san: str) -> Move:
        return Move(self._core.parse_san(san))

    def push_san(self, san: str) -> Move:
        move = self.parse_san(san)
        self.push(move)
        return move

    def san(self, move: Move) -> str:
        return self._core.san(move.uci())

    def copy(self) -> "Board":
        b = Board(_core=self._core.copy())
        b.move_stack = list(self.move_stack)
        return b

    def fen(self) -> str:
        return self._core.fen()

    def is_game_over(self, claim_draw: bool = False) -> bool:
        return self.outcome(claim_draw=claim_draw) is not None

    def outcome(self, claim_draw: bool = False):
        return self._core.outcome(claim_draw=claim_draw)

    def is_castling(self, move: Move) -> bool:
        return self._core.is_castling(move.uci())

    def is_en_passant(self, move: Move) -> bool:
        return self._core.is_en_passant(move.uci())

    def can_claim_threefold_repetition(self) -> bool:
        return self._core.can_claim_threefold_repetition()
