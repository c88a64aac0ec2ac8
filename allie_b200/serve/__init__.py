"""TCP move server (reference ``src/server``): one process per "system" alias, JSON in / JSON out."""
from .client import BotSession, request_move
from .server import SYSTEMS, System, algorithm_test, recv_dict, send_dict, serve

__all__ = ["SYSTEMS", "System", "algorithm_test", "recv_dict", "send_dict", "serve", "BotSession", "request_move"]
