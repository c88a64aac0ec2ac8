"""Minimal UCI engine client (Stockfish, lc0): the two things the evaluation code needs are a
position evaluation at a node budget and a best move.  The reference uses python-chess's engine
module (``src/evaluation/utils.py:9-38``, ``decode.py:128-182``); that package is not a dependency
here, so the protocol is spoken directly over a subprocess pipe."""
from __future__ import annotations

import shutil
import subprocess


class EngineUnavailable(RuntimeError):
    pass


class UCIEngine:
    def __init__(self, path: str, options: dict | None = None, args: list[str] | None = None):
        exe = shutil.which(path) or path
        try:
            self.proc = subprocess.Popen([exe, *(args or [])], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True, bufsize=1)
        except (FileNotFoundError, PermissionError) as e:
            raise EngineUnavailable(f"UCI engine {path!r} not found") from e
        self._send("uci")
        self._wait("uciok")
        for k, v in (options or {}).items():
            self._send(f"setoption name {k} value {v}")
        self._send("isready")
        self._wait("readyok")

    def _send(self, line: str) -> None:
        self.proc.stdin.write(line + "\n")
        self.proc.stdin.flush()

    def _wait(self, token: str) -> list[str]:
        lines = []
        while True:
            line = self.proc.stdout.readline()
            if not line:
                raise EngineUnavailable("engine exited")
            lines.append(line.strip())
            if line.startswith(token):
                return lines

    def analyse(self, moves: list[str], nodes: int, fen: str | None = None) -> tuple[int | None, int | None, str]:
        """(centipawns from the side to move's view or None, mate distance or None, best move) of
        the position reached by ``moves`` from the start position, or from ``fen``."""
        self._send(("position startpos" if fen is None else f"position fen {fen}")
                   + (" moves " + " ".join(moves) if moves else ""))
        self._send(f"go nodes {nodes}")
        cp = mate = None
        for line in self._wait("bestmove"):
            parts = line.split()
            if parts[:1] == ["info"] and "score" in parts:
                i = parts.index("score")
                if parts[i + 1] == "cp":
                    cp, mate = int(parts[i + 2]), None
                elif parts[i + 1] == "mate":
                    cp, mate = None, int(parts[i + 2])
            if parts[:1] == ["bestmove"]:
                return cp, mate, parts[1]
        return cp, mate, ""

    def quit(self) -> None:
        try:
            self._send("quit")
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
