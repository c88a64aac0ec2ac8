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
        for fn in ("chess_castling_mask", "chess_ep_square", "chess_fullmove"):
            getattr(lib, fn).argtypes = [c_void_p]
        lib.chess_is_repetition.argtypes = [c_void_p, c_int]
        lib.chess_parse_san.argtypes = [c_void_p, c_char_p, c_char_p]
        lib.chess_san.argtypes = [c_void_p, c_char_p, c_char_p]
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

    def outcome(self, claim_draw: bool = False) -> Outcome | None:
        """How the game ended, or None while it continues.  With ``claim_draw`` a position in
        which a player may claim the fifty-move or threefold-repetition draw counts as ended."""
        t = _h().chess_termination(self._h)
        if t == 0:
            if claim_draw and self.can_claim_fifty_moves():
                return Outcome("fifty_moves", None)
            if claim_draw and self.can_claim_threefold_repetition():
                return Outcome("threefold_repetition", None)
            return None
        w = _h().chess_winner(self._h)
        return Outcome(TERMINATIONS[t], None if w < 0 else bool(w))

    def can_claim_fifty_moves(self) -> bool:
        """Fifty moves without a capture or pawn move are complete, or a legal move completes them."""
        if self.halfmove_clock >= 100:
            return True
        if self.halfmove_clock >= 99:
            for mv in self.legal_moves_uci():
                if abs(self.piece_at(_sq(mv[:2]))) != 1 and not self.is_capture(mv):
                    return True
        return False

    def can_claim_draw(self) -> bool:
        return self.can_claim_fifty_moves() or self.can_claim_threefold_repetition()

    def piece_at(self, sq: int) -> int:
        return _h().chess_piece_at(self._h, sq)

    def perft(self, depth: int) -> int:
        return int(_h().chess_perft(self._h, depth))

    # ---- position text and move classification (used by annotation, PGN prompts and the UCI client)
    @property
    def fullmove_number(self) -> int:
        return int(_h().chess_fullmove(self._h))

    @property
    def halfmove_clock(self) -> int:
        return int(_h().chess_halfmove_clock(self._h))

    @property
    def ep_square(self) -> int | None:
        sq = int(_h().chess_ep_square(self._h))
        return None if sq < 0 else sq

    def ply(self) -> int:
        return int(_h().chess_ply(self._h))

    def is_capture(self, uci: str) -> bool:
        return self.piece_at(_sq(uci[2:4])) != 0 or self.is_en_passant(uci)

    def is_en_passant(self, uci: str) -> bool:
        """A pawn that changes file onto an empty square."""
        return (abs(self.piece_at(_sq(uci[:2]))) == 1 and uci[0] != uci[2]
                and self.piece_at(_sq(uci[2:4])) == 0)

    def is_castling(self, uci: str) -> bool:
        """A king that moves two files."""
        return abs(self.piece_at(_sq(uci[:2]))) == 6 and abs(ord(uci[0]) - ord(uci[2])) == 2

    def is_repetition(self, count: int = 3) -> bool:
        return bool(_h().chess_is_repetition(self._h, count))

    def can_claim_threefold_repetition(self) -> bool:
        """The position has occurred three times, or some legal move reaches such a position
        (the two cases in which a player may claim the draw)."""
        if self.is_repetition(3):
            return True
        for mv in self.legal_moves_uci():
            nxt = self.copy()
            nxt.push_uci(mv)
            if nxt.is_repetition(3):
                return True
        return False

    def fen(self) -> str:
        """Forsyth-Edwards notation; the en-passant field is set only when a capture onto it is legal."""
        rows = []
        for r in range(7, -1, -1):
            row, gap = "", 0
            for f in range(8):
                p = self.piece_at(r * 8 + f)
                if p == 0:
                    gap += 1
                    continue
                if gap:
                    row, gap = row + str(gap), 0
                ch = " pnbrqk"[abs(p)]
                row += ch.upper() if p > 0 else ch
            rows.append(row + (str(gap) if gap else ""))
        m = int(_h().chess_castling_mask(self._h))
        rights = "".join(c for i, c in enumerate("KQkq") if m >> i & 1) or "-"
        ep = "-"
        if self.ep_square is not None:
            name = "abcdefgh"[self.ep_square % 8] + str(self.ep_square // 8 + 1)
            if any(mv[2:4] == name and self.is_en_passant(mv) for mv in self.legal_moves_uci()):
                ep = name
        return (f"{'/'.join(rows)} {'w' if self.turn else 'b'} {rights} {ep} "
                f"{self.halfmove_clock} {self.fullmove_number}")

    def san(self, uci: str) -> str:
        """Standard algebraic notation of a legal move, with minimal disambiguation and the
        check / mate suffix (written by the C++ core)."""
        buf = ctypes.create_string_buffer(12)
        if not _h().chess_san(self._h, uci.encode(), buf):
            raise ValueError(f"illegal uci: {uci!r}")
        return buf.value.decode()

    def san_reference(self, uci: str) -> str:
        """The same notation computed in Python from the public board queries; the oracle of
        :meth:`san` in the tests."""
        legal = self.legal_moves_uci()
        if uci not in legal:
            raise ValueError(f"illegal uci: {uci!r}")
        src = _sq(uci[:2])
        piece = abs(self.piece_at(src))
        if self.is_castling(uci):
            text = "O-O" if uci[2] == "g" else "O-O-O"
        else:
            capture = self.is_capture(uci)
            if piece == 1:
                text = (uci[0] + "x" if capture else "") + uci[2:4]
                if len(uci) == 5:
                    text += "=" + uci[4].upper()
            else:
                others = [mv for mv in legal if mv != uci and mv[2:4] == uci[2:4]
                          and abs(self.piece_at(_sq(mv[:2]))) == piece]
                dis = ""
                if others:
                    if all(mv[0] != uci[0] for mv in others):
                        dis = uci[0]
                    elif all(mv[1] != uci[1] for mv in others):
                        dis = uci[1]
                    else:
                        dis = uci[:2]
                text = " PNBRQK"[piece] + dis + ("x" if capture else "") + uci[2:4]
        nxt = self.copy()
        nxt.push_uci(uci)
        if nxt.is_check():
            text += "#" if not nxt.legal_move_ids() else "+"
        return text

    def parse_san(self, san: str) -> str:
        """The legal move (UCI text) that a SAN token denotes; ValueError if none or several do.
        Check marks and annotations are ignored and more disambiguation than necessary is accepted
        (resolved by the C++ core)."""
        buf = ctypes.create_string_buffer(8)
        if not _h().chess_parse_san(self._h, san.encode(), buf):
            raise ValueError(f"cannot resolve SAN {san!r} in {self.fen()}")
        return buf.value.decode()

    def push_san(self, san: str) -> str:
        uci = self.parse_san(san)
        self.push_uci(uci)
        return uci

    def movetext(self, columns: int | None = None, result: str | None = None) -> str:
        """PGN movetext of the game so far: ``1. e4 e5 2. Nf3 ...`` (replayed from the start),
        optionally followed by a result marker.  With ``columns`` the text is wrapped the way
        python-chess's PGN exporter does it: tokens are a move number or a move, each with a
        trailing space, and a token that no longer fits into the line starts a new one."""
        b, tokens = Board(), []
        for i, mv in enumerate(self.move_stack):
            if i % 2 == 0:
                tokens.append(f"{i // 2 + 1}. ")
            tokens.append(b.san(mv) + " ")
            b.push_uci(mv)
        if result is not None:
            tokens.append(result)
        if columns is None:
            return "".join(tokens).rstrip()
        lines, cur = [], ""
        for tok in tokens:
            if columns - len(cur) < len(tok):
                if cur:
                    lines.append(cur.rstrip())
                cur = ""
            cur += tok
        if cur:
            lines.append(cur.rstrip())
        return "\n".join(lines)


def _sq(name: str) -> int:
    return (int(name[1]) - 1) * 8 + (ord(name[0]) - 97)


def vocab_uci(token_id: int) -> str:
    buf = ctypes.create_string_buffer(8)
    _h().chess_vocab_uci(token_id, buf)
    return buf.value.decode()
