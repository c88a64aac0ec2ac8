"""Allie as a UCI engine, so that any chess GUI or an unmodified lichess-bot can play it.

The reference reaches Lichess through its own fork of lichess-bot, which talks to the move server
(``scripts/run-server.sh:26-33``, ``src/server/main.py``); this front end needs no fork: it speaks
the UCI text protocol on stdin / stdout and asks a running move server for every move.

    python -m allie_b200.serve.uci --system humanlike            # registry alias or port number

Supported: ``uci``, ``isready``, ``ucinewgame``, ``setoption name <X> value <v>`` for ``WhiteElo``,
``BlackElo`` and ``TimeControl``, ``position startpos [moves ...]``, ``go [wtime btime winc binc
movetime ...]``, ``stop``, ``quit``.  The seconds each side spent on its moves are reconstructed
from the clocks that ``go`` reports (the model conditions on them), the time control from the first
``go`` of a game unless set as an option.  ``info string`` lines carry the predicted think time and
a resignation (UCI has no resign move: the best legal move is still returned).
"""
from __future__ import annotations

import argparse
import sys
from typing import Callable, TextIO

from ..data import Game
from .client import request_move


class UCIFrontEnd:
    def __init__(self, ask: Callable[[Game], dict], out: TextIO = sys.stdout, elo: int = 1500):
        self.ask, self.out = ask, out
        self.options = {"WhiteElo": elo, "BlackElo": elo, "TimeControl": None}
        self.new_game()

    def new_game(self) -> None:
        self.moves: list[str] = []
        self.seconds: dict[int, int] = {}          # ply -> seconds spent on it
        self.clock_seen: dict[bool, float] = {}    # colour -> clock (s) at its previous `go`
        self.time_control: str | None = None

    def say(self, line: str) -> None:
        self.out.write(line + "\n")
        self.out.flush()

    # ------------------------------------------------------------------ commands
    def handle(self, line: str) -> bool:
        """Processes one input line; False after ``quit``."""
        parts = line.split()
        if not parts:
            return True
        cmd = parts[0]
        if cmd == "uci":
            self.say("id name Allie (B200)")
            self.say("id author allie-b200")
            self.say("option name WhiteElo type spin default 1500 min 500 max 3000")
            self.say("option name BlackElo type spin default 1500 min 500 max 3000")
            self.say("option name TimeControl type string default <from clock>")
            self.say("uciok")
        elif cmd == "isready":
            self.say("readyok")
        elif cmd == "ucinewgame":
            self.new_game()
        elif cmd == "setoption" and "name" in parts and "value" in parts:
            name = " ".join(parts[parts.index("name") + 1:parts.index("value")])
            value = " ".join(parts[parts.index("value") + 1:])
            if name in ("WhiteElo", "BlackElo"):
                self.options[name] = int(value)
            elif name == "TimeControl":
                self.options[name] = value
        elif cmd == "position":
            self.position(parts[1:])
        elif cmd == "go":
            self.go(parts[1:])
        elif cmd == "quit":
            return False
        return True                                 # `stop`, `ponderhit` and unknown commands: nothing to do

    def position(self, args: list[str]) -> None:
        if args[:1] != ["startpos"]:
            self.say("info string only games from the start position are supported")
            return
        moves = args[2:] if args[1:2] == ["moves"] else []
        if moves[:len(self.moves)] != self.moves:   # a different game: forget the clocks
            self.new_game()
        self.moves = list(moves)

    def go(self, args: list[str]) -> None:
        vals = {args[i]: float(args[i + 1]) for i in range(0, len(args) - 1) if args[i] in
                ("wtime", "btime", "winc", "binc", "movetime")}
        white = len(self.moves) % 2 == 0
        base_ms, inc_ms = vals.get("wtime" if white else "btime"), vals.get("winc" if white else "binc", 0.0)
        if self.time_control is None and base_ms is not None:
            self.time_control = f"{int(round(base_ms / 1000))}+{int(round(inc_ms / 1000))}"
        # the opponent's last move took: its clock at our previous `go` minus its clock now, plus increment
        opp = not white
        opp_ms, opp_inc = vals.get("btime" if white else "wtime"), vals.get("binc" if white else "winc", 0.0)
        if self.moves and opp_ms is not None and opp in self.clock_seen:
            spent = self.clock_seen[opp] - opp_ms / 1000 + opp_inc / 1000
            self.seconds[len(self.moves) - 1] = max(0, int(round(spent)))
        if opp_ms is not None:
            self.clock_seen[opp] = opp_ms / 1000
        tc = self.options["TimeControl"] or self.time_control or "180+0"
        secs = [self.seconds.get(i, 0) for i in range(len(self.moves))]
        game = Game(tc, int(self.options["WhiteElo"]), int(self.options["BlackElo"]), None, False,
                    list(self.moves), secs)
        try:
            ans = self.ask(game)
        except (OSError, ValueError, KeyError) as e:     # server away, or it refused the game
            self.say(f"info string no move from the server: {type(e).__name__}: {e}")
            self.say("bestmove 0000")
            return
        think = ans.get("think_time")
        if think is not None:
            self.say(f"info string predicted think time {think:.1f}s")
            self.seconds[len(self.moves)] = max(0, int(round(think)))
        if ans.get("resigned"):
            self.say("info string the model would resign here")
        self.say(f"bestmove {ans['move']}")

    def run(self, inp: TextIO = sys.stdin) -> None:
        for line in inp:
            if not self.handle(line.strip()):
                break


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description="UCI front end of a running Allie move server")
    ap.add_argument("--system", default="humanlike", help="registry alias or port of the move server")
    ap.add_argument("--host", default="localhost")
    a = ap.parse_args(argv)
    system = int(a.system) if a.system.isdigit() else a.system
    UCIFrontEnd(lambda game: request_move(system, game, a.host)).run()


if __name__ == "__main__":
    main()
