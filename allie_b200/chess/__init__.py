"""Chess rules for the decode runtime: a thin Python face over the C++ bitboard core
(``csrc/chess.hpp``), with the small part of the python-chess ``Board`` API the reference decode code
relies on (``src/modeling/data.py:51-61``, ``src/evaluation/decode.py:96-101,345-353``): replay UCI
moves, list legal moves *in python-chess order*, side to move, game-over / winner.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_ulonglong, c_void_p

from ..moves import CHESS_MOVES
from ..ops import _lib

WHITE, BLACK = True, False
TERMINATIONS = {0: None, 1: "checkmate", 2: "stalemate", 3: "insufficient_material",
                4: "seventyfive_moves", 5: "fivefold_repetition"}

_configured = False


def _h():
    global _configured
    lib = _lib.host()
    if not _configured:
        lib.chess_new.restype = c_void_p
        lib.chess_copy.restype = c_void_p
        lib.chess_copy.argtypes = [c_void_p]
        lib.chess_free.argtypes = [c_void_p]
        lib.chess_reset.argtypes = [c_void_p]
        lib.chess_push_uci.argtypes = [c_void_p, c_char_p]
        lib.chess_push_id.argtypes = [c_void_p, c_int]
        lib.chess_legal_ids.argtypes = [c_void_p, ctypes.POINTER(c_int), c_int]
        for fn in ("chess_turn", "chess_ply", "chess_is_check", "chess_termination", "chess_winner",
                   "chess_halfmove_clock"):
            getattr(lib, fn).argtypes = [c_void_p]
        lib.chess_piece_at.argtypes = [c_void_p, c_int]
        lib.chess_perft.argtypes = [c_void_p, c_int]
        lib.chess_perft.restype = c_ulonglong
        lib.chess_set_fen.argtypes = [c_void_p, c_char_p]
        lib.chess_vocab_uci.argtypes = [c_int, ctypes.c_char_p]
        _configured = True
    return lib


class Outcome:
    def __init__(self, termination: str, winner):
        self.termination = termination
        self.winner = winner

    def __repr__(self):
        return f"Outcome(termination={self.termination!r}, winner={self.winner!r})"


class Board:
    def __init__(self, fen: str | None = None, _handle=None):
        lib = _h()
        self._h = _handle if _handle is not None else lib.chess_new()
        self.move_stack: list[str] = []
        if fen is not None and not lib.chess_set_fen(self._h, fen.encode()):
            raise ValueError(f"bad FEN {fen!r}")

    def __del__(self):
        try:
            _h().chess_free(self._h)
        except Exception:
            pass

    def copy(self) -> "Board":
        b = Board(_handle=_h().chess_copy(self._h))
        b.move_stack = list(self.move_stack)
        return b

    def push_uci(self, uci: str) -> None:
        if not _h().chess_push_uci(self._h, uci.encode()):
            raise ValueError(f"illegal uci: {uci!r} after {' '.join(self.move_stack[-6:])}")
        self.move_stack.append(uci)

    def legal_move_ids(self) -> list[int]:
        buf = (c_int * 256)()
        n = _h().chess_legal_ids(self._h, buf, 256)
        return list(buf[:n])

    def legal_moves_uci(self) -> list[str]:
        return [CHESS_MOVES[i] for i in self.legal_move_ids()]

    @property
    def turn(self) -> bool:
        return bool(_h().chess_turn(self._h))

    def is_check(self) -> bool:
        return bool(_h().chess_is_check(self._h))

    def is_game_over(self) -> bool:
        return _h().chess_termination(self._h) != 0

    def outcome(self) -> Outcome | None:
        t = _h().chess_termination(self._h)
        if t == 0:
            return None
        w = _h().chess_winner(self._h)
        return Outcome(TERMINATIONS[t], None if w < 0 else bool(w))

    def piece_at(self, sq: int) -> int:
        return _h().chess_piece_at(self._h, sq)

    def perft(self, depth: int) -> int:
        return int(_h().chess_perft(self._h, depth))


def vocab_uci(token_id: int) -> str:
    buf = ctypes.create_string_buffer(8)
    _h().chess_vocab_uci(token_id, buf)
    return buf.value.decode()
