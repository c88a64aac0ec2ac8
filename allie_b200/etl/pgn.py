"""PGN -> JSONL rows (reference ``src/data/process-lichess.py:1-147``).

Streams a (optionally zstd-compressed) Lichess PGN dump, keeps Blitz games longer than 8 plies and
writes one JSON object per game with the reference's keys: ``game-id, moves-uci, moves-seconds, event,
result, white-elo, black-elo, termination, time-control, opening``.  Seconds per move come from the clock
comments: previous clock of the same side minus the new clock plus the increment.  SAN is resolved
against the C++ move generator (python-chess is not a dependency); the whole movetext of a game is
parsed by one C++ call (``csrc/pgn_api.cpp``), with a Python statement of the same rules kept as its
oracle."""
from __future__ import annotations

import argparse
import ctypes
import io
import json
import re
import sys
from multiprocessing import get_context

from ..chess import Board

_TAG = re.compile(r'^\[(\w+) "(.*)"\]$')
_CLK = re.compile(r"\[%clk (\d+):(\d+):(\d+)\]")
_PIECES = {"N": 2, "B": 3, "R": 4, "Q": 5, "K": 6}


def san_to_uci(board: Board, san: str) -> str:
    """Resolves one SAN token against the legal moves of ``board``."""
    san = san.rstrip("+#!?")
    legal = board.legal_moves_uci()
    if san in ("O-O", "0-0"):
        return "e1g1" if board.turn else "e8g8"
    if san in ("O-O-O", "0-0-0"):
        return "e1c1" if board.turn else "e8c8"
    promo = ""
    if "=" in san:
        san, promo = san.split("=")[0], san.split("=")[1][0].lower()
    piece = _PIECES.get(san[0], 1)
    body = san[1:] if piece != 1 else san
    body = body.replace("x", "")
    dest, dis = body[-2:], body[:-2]
    cands = []
    for mv in legal:
        if mv[2:4] != dest or mv[4:] != promo:
            continue
        sq = (int(mv[1]) - 1) * 8 + (ord(mv[0]) - 97)
        if abs(board.piece_at(sq)) != piece:
            continue
        if all(ch in mv[:2] for ch in dis):
            cands.append(mv)
    if len(cands) != 1:
        raise ValueError(f"cannot resolve SAN {san!r} (candidates {cands})")
    return cands[0]


_native_ready = False


def _native():
    global _native_ready
    from ..ops import _lib

    lib = _lib.host()
    if not _native_ready:
        ip = ctypes.POINTER(ctypes.c_int)
        lib.pgn_parse_movetext.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_char_p,
                                           ctypes.c_int, ip, ctypes.c_int, ip]
        _native_ready = True
    return lib


def parse_movetext(movetext: str, base: int, inc: int, max_moves: int = 1024) -> tuple[list[str], list[int]] | None:
    """(UCI moves, seconds per move) of one game's movetext through the C++ parser
    (``csrc/pgn_api.cpp``); None when a move cannot be resolved."""
    out = ctypes.create_string_buffer(6 * max_moves + 8)
    secs = (ctypes.c_int * max_moves)()
    n_secs = ctypes.c_int(0)
    n = _native().pgn_parse_movetext(movetext.encode(), base, inc, out, len(out), secs, max_moves,
                                     ctypes.byref(n_secs))
    if n < 0:
        return None
    return out.value.decode().split(), list(secs[: n_secs.value])


def parse_game(text: str, native: bool = True) -> dict | None:
    """One PGN game -> JSONL row, or None when the game is filtered out (not Blitz, unknown ratings,
    no increment field, eight plies or fewer, clock comments missing, an unreadable move).
    ``native=False`` takes the pure-Python parser (the oracle of the C++ one)."""
    tags, body = {}, []
    for line in text.splitlines():
        m = _TAG.match(line.strip())
        if m:
            tags[m.group(1)] = m.group(2)
        elif line.strip():
            body.append(line)
    if "Blitz" not in tags.get("Event", "") or "?" in (tags.get("WhiteElo", "?") + tags.get("BlackElo", "?")):
        return None
    tc = tags.get("TimeControl", "")
    if "+" not in tc:
        return None
    base, inc = (int(x) for x in tc.split("+"))
    movetext = " ".join(body)
    if native:
        parsed = parse_movetext(movetext, base, inc)
        if parsed is None:
            return None
        moves, seconds = parsed
        return _row(tags, tc, moves, seconds)
    tokens = re.findall(r"\{[^}]*\}|\S+", movetext)
    board = Board()
    moves, seconds = [], []
    clocks = [base, base]
    for tok in tokens:
        if tok.startswith("{"):
            c = _CLK.search(tok)
            if c and moves:
                side = (len(moves) - 1) % 2
                now = int(c.group(1)) * 3600 + int(c.group(2)) * 60 + int(c.group(3))
                seconds.append(max(0, clocks[side] - now + inc))
                clocks[side] = now
            continue
        if tok[0].isdigit() and (tok.endswith(".") or "..." in tok) or tok in ("1-0", "0-1", "1/2-1/2", "*"):
            continue
        tok = re.sub(r"^\d+\.+", "", tok)
        if not tok:
            continue
        try:
            uci = san_to_uci(board, tok)
            board.push_uci(uci)
        except ValueError:
            return None
        moves.append(uci)
    return _row(tags, tc, moves, seconds)


def _row(tags: dict, tc: str, moves: list[str], seconds: list[int]) -> dict | None:
    if len(moves) <= 8 or len(seconds) != len(moves):
        return None
    return {"game-id": tags.get("Site", ""), "moves-uci": " ".join(moves), "moves-seconds": seconds,
            "event": tags.get("Event", ""), "result": tags.get("Result", "*"),
            "white-elo": int(tags["WhiteElo"]), "black-elo": int(tags["BlackElo"]),
            "termination": tags.get("Termination", ""), "time-control": tc, "opening": tags.get("Opening", "")}


def iter_games(stream: io.TextIOBase):
    buf, seen_moves = [], False
    for line in stream:
        if line.startswith("[Event ") and buf and seen_moves:
            yield "".join(buf)
            buf, seen_moves = [], False
        if line.strip() and not line.startswith("["):
            seen_moves = True
        buf.append(line)
    if buf:
        yield "".join(buf)


def open_pgn(path: str):
    """Text stream of a PGN file: plain, ``.zst`` (through the ``zstandard`` module, else the ``zstd``
    command line tool) or ``-`` for standard input (``zstdcat dump.pgn.zst | python -m allie_b200.etl.pgn - out.jsonl``)."""
    if path == "-":
        return sys.stdin
    if path.endswith(".zst"):
        try:
            import zstandard
        except ImportError:
            import shutil
            import subprocess

            if shutil.which("zstd") is None:
                raise RuntimeError("reading .zst needs the zstandard module or the zstd tool; "
                                   "or pipe the decompressed text to '-'") from None
            proc = subprocess.Popen(["zstd", "-dc", path], stdout=subprocess.PIPE)
            return io.TextIOWrapper(proc.stdout, encoding="utf-8")
        return io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(open(path, "rb")), encoding="utf-8")
    return open(path, encoding="utf-8")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("pgn")
    ap.add_argument("out")
    ap.add_argument("--workers", type=int, default=8)
    a = ap.parse_args(argv)
    # worker processes are spawned, not forked: the parent may already run threads (BLAS, prefetch)
    with open_pgn(a.pgn) as f, open(a.out, "w") as out, get_context("spawn").Pool(a.workers) as pool:
        n = 0
        for row in pool.imap(parse_game, iter_games(f), chunksize=64):
            if row is not None:
                out.write(json.dumps(row) + "\n")
                n += 1
        print(f"wrote {n} games", file=sys.stderr)


if __name__ == "__main__":
    main()
