"""The 1968-entry UCI move vocabulary; list index = token id.

The table is generated, not stored.  Order (it must match the reference table
``src/modeling/moves.py:3-1972`` exactly, because token ids are positions in it):

1. sliding ("queen-line") moves, 2. knight moves, 3. promotions.
   Groups 1 and 2 walk the from-squares file by file (a1, a2, ..., a8, b1, ...)
   and for each from-square scan the targets from rank 8 down to rank 1, and inside a rank from
   file h down to file a.  Group 3 walks files a..h; for each file first the white push/captures
   (rank 7 -> 8) then the black ones (rank 2 -> 1), target files in the order f+1, f-1, f, and the
   promotion piece in the order q, r, b, n.

``VOCAB_SHA256`` pins the result.
"""
from __future__ import annotations

import hashlib

FILES = "abcdefgh"
VOCAB_SHA256 = "48a68142d02bd6bfbe4ae97749c3416283d0e3e5195bd804477685bb37e657e8"


def _sq(f: int, r: int) -> str:
    return FILES[f] + str(r + 1)


def _generate() -> list[str]:
    sliding: list[str] = []
    knight: list[str] = []
    for f in range(8):
        for r in range(8):
            for tr in range(7, -1, -1):
                for tf in range(7, -1, -1):
                    df, dr = abs(tf - f), abs(tr - r)
                    if df == 0 and dr == 0:
                        continue
                    if df == 0 or dr == 0 or df == dr:
                        sliding.append(_sq(f, r) + _sq(tf, tr))
                    elif (df, dr) in ((1, 2), (2, 1)):
                        knight.append(_sq(f, r) + _sq(tf, tr))
    promo: list[str] = []
    for f in range(8):
        for r_from, r_to in ((6, 7), (1, 0)):
            for tf in (f + 1, f - 1, f):
                if 0 <= tf < 8:
                    for piece in "qrbn":
                        promo.append(_sq(f, r_from) + _sq(tf, r_to) + piece)
    return sliding + knight + promo


CHESS_MOVES: list[str] = _generate()
NUM_CHESS_MOVES = len(CHESS_MOVES)
MOVE_TO_ID = {m: i for i, m in enumerate(CHESS_MOVES)}


def vocabulary_digest() -> str:
    return hashlib.sha256("\n".join(CHESS_MOVES).encode()).hexdigest()


assert NUM_CHESS_MOVES == 1968, NUM_CHESS_MOVES
