"""Client side of the move server's wire format (the part of the reference's lichess-bot fork that
talks to ``src/server/main.py``: connect, send one ``Game`` dict, read one answer).

    from allie_b200.serve.client import request_move
    ans = request_move("humanlike", game)        # {"move": "e2e4", "think_time": 1.7, "resigned": False}

``BotSession`` keeps the state a bot needs between moves of one game (ratings, time control, moves
and the seconds each side spent) and asks the server whenever it is the bot's turn.
"""
from __future__ import annotations

import socket
from dataclasses import dataclass, field

from ..data import Game
from .server import SYSTEMS, recv_dict, send_dict


def request_move(system: str | int, game: Game, host: str = "localhost", timeout: float = 120.0) -> dict:
    """One request to the server of ``system`` (an alias of the registry or a port number)."""
    port = SYSTEMS[system].port if isinstance(system, str) else int(system)
    with socket.create_connection((host, port), timeout=timeout) as conn:
        send_dict(conn, game.to_dict())
        ans = recv_dict(conn)
    if not {"move", "think_time", "resigned"} <= set(ans):
        raise ValueError(f"malformed answer from the move server: {ans!r}")
    return ans


@dataclass
class BotSession:
    system: str | int
    time_control: str
    white_elo: int
    black_elo: int
    bot_is_white: bool
    host: str = "localhost"
    moves: list[str] = field(default_factory=list)
    moves_seconds: list[int] = field(default_factory=list)

    def push(self, move: str, seconds: float = 0.0) -> None:
        """Records a move of either side with the time it took."""
        self.moves.append(move)
        self.moves_seconds.append(int(round(seconds)))

    @property
    def bot_to_move(self) -> bool:
        return (len(self.moves) % 2 == 0) == self.bot_is_white

    def game(self) -> Game:
        return Game(self.time_control, self.white_elo, self.black_elo, None, False, list(self.moves),
                    list(self.moves_seconds))

    def play(self) -> dict:
        """Asks the server for the bot's move in the current position and records it."""
        if not self.bot_to_move:
            raise RuntimeError("not the bot's turn")
        ans = request_move(self.system, self.game(), self.host)
        if not ans["resigned"]:
            self.push(ans["move"], ans["think_time"] or 0.0)
        return ans
