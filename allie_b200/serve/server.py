"""Move server with the reference's wire format and system registry
(``src/server/main.py:19-101``, ``src/server/utils.py:7-53``).

A client connects to ``localhost:port``, sends one JSON ``Game`` dict, receives one JSON
``{"move", "think_time", "resigned"}`` and the connection closes.  The bot plays at its opponent's
rating unless the system fixes one.  Unlike the reference (strictly one request at a time), all
connections waiting in the listen backlog when a request arrives are answered as one batch: their
positions share a single network evaluation (policy systems) or one batched tree search (MCTS
systems).  The requests of a batch are read concurrently under one shared deadline, so an idle
connection delays its batch by that deadline at most once, not by one timeout per connection.
Neither a broken client socket, nor a malformed request, nor an exception inside the decoder
takes the server down: the affected connections are closed with a warning and the loop goes on.
"""
from __future__ import annotations

import json
import logging
import select
import socket
import time
from dataclasses import dataclass, field

import torch

from ..data import Game, UCITokenizer
from ..search import DECODE_STRATEGIES, DecodeResult, DecodeStrategy, decode_batch

logger = logging.getLogger(__name__)


def send_dict(sock: socket.socket, data: dict) -> None:
    sock.sendall(json.dumps(data).encode())


MAX_MESSAGE_BYTES = 1 << 20       # a 512-ply game is a few KiB; anything near this size is not a request


def recv_dict(sock: socket.socket) -> dict:
    """Accumulates 8 KiB chunks until the bytes parse as JSON."""
    buf = b""
    while True:
        chunk = sock.recv(8192)
        if not chunk:
            raise ConnectionError("peer closed before a complete JSON document arrived")
        buf += chunk
        if len(buf) > MAX_MESSAGE_BYTES:
            raise ValueError("message larger than any request can be")
        try:
            return json.loads(buf.decode())
        except (json.JSONDecodeError, UnicodeDecodeError):
            continue


@dataclass(frozen=True)
class System:
    port: int
    elo: int | None
    algorithm: str
    algorithm_config: dict = field(default_factory=dict)


SYSTEMS: dict[str, System] = {
    "maia": System(20602, None, "maia", {}),
    "humanlike": System(20600, None, "policy", {"sample": True}),
    "grandmaster": System(20601, 2500, "policy", {"sample": False}),
    "humanlike-adaptive-rb": System(20607, None, "adaptive-mcts",
                                    {"mean_n_sims": 50, "c_puct": 1.25, "sample": "rating-based"}),
    "humanlike-mcts-rb": System(20608, None, "mcts", {"n_sims": 50, "c_puct": 1.25, "sample": "rating-based"}),
}

DEFAULT_SYSTEM = "humanlike"

# Deep Blue - Kasparov 1997, game 2 (the reference's start-up self test replays it)
SELF_TEST_MOVES = ("e2e4 e7e5 g1f3 b8c6 f1b5 a7a6 b5a4 g8f6 e1g1 f8e7 f1e1 b7b5 a4b3 d7d6 c2c3 e8g8 h2h3 h7h6 "
                   "d2d4 f8e8 b1d2 e7f8 d2f1 c8d7 f1g3 c6a5 b3c2 c7c5 b2b3 a5c6 d4d5 c6e7 c1e3 e7g6 d1d2 f6h7 "
                   "a2a4 h7f6 a4b5 a6b5 e1a1 d8b8 c2d3").split()


def assign_elo(game: Game, system: System) -> Game:
    """The bot takes its opponent's rating (or the system's fixed one)."""
    white_to_move = len(game.moves) % 2 == 0
    if system.elo is not None:
        if white_to_move:
            game.white_elo = system.elo
        else:
            game.black_elo = system.elo
    elif white_to_move:
        game.white_elo = game.black_elo
    else:
        game.black_elo = game.white_elo
    return game


def algorithm_test(algorithm: DecodeStrategy, every: int = 2, max_plies: int | None = None) -> float:
    """Decodes every other ply of the self-test game; returns the wall time."""
    t0 = time.time()
    moves = SELF_TEST_MOVES if max_plies is None else SELF_TEST_MOVES[:max_plies]
    for ply in range(0, len(moves), every):
        g = Game("5400+0", 2800, 2800, None, False, list(moves[:ply]), [5] * ply)
        res = algorithm.decode_full(g)
        if ply == 10:
            logger.info(f"self test, ply 10: {res}")
    dt = time.time() - t0
    logger.info(f"self test took {dt:.2f}s")
    return dt


def build_algorithm(alias: str, model, tokenizer: UCITokenizer, device: str | None = None,
                    batched: bool = False, max_batch: int = 64) -> DecodeStrategy:
    """The system's strategy.  With ``batched`` its many-games-per-call form is built when one is
    registered (``<algorithm>-batched``), with one search tree per connection of a full batch."""
    system = SYSTEMS[alias]
    if system.algorithm == "maia":
        # Maia plays its first ten plies from the default (policy) system, like the reference server
        book = build_algorithm(DEFAULT_SYSTEM, model, tokenizer, device)
        return DECODE_STRATEGIES["maia"](model, tokenizer, device=device, opening_strategy=book,
                                         **system.algorithm_config)
    if batched and f"{system.algorithm}-batched" in DECODE_STRATEGIES:
        extra = {} if system.algorithm == "policy" else {"n_trees": max_batch}
        return DECODE_STRATEGIES[f"{system.algorithm}-batched"](model, tokenizer, device=device,
                                                               **system.algorithm_config, **extra)
    if system.algorithm not in DECODE_STRATEGIES:
        raise RuntimeError(f"system {alias!r} needs the external engine {system.algorithm!r}, "
                           "which is not available in this installation")
    return DECODE_STRATEGIES[system.algorithm](model, tokenizer, device=device, **system.algorithm_config)


def read_requests(conns: list[socket.socket], timeout: float) -> list[tuple[socket.socket, dict | Exception]]:
    """Reads one JSON document from every connection, all of them concurrently (``select``) under
    ONE deadline of ``timeout`` seconds.  Returns, in the order of ``conns``, the parsed dict or the
    exception that ended the attempt (closed early, oversized, timed out)."""
    bufs = {c: b"" for c in conns}
    done: dict[socket.socket, dict | Exception] = {}
    for c in conns:
        c.setblocking(False)
    deadline = time.monotonic() + timeout
    while len(done) < len(conns):
        pending = [c for c in conns if c not in done]
        left = deadline - time.monotonic()
        if left <= 0:
            for c in pending:
                done[c] = TimeoutError("no complete request within the batch deadline")
            break
        readable = select.select(pending, [], [], left)[0]
        for c in readable:
            try:
                chunk = c.recv(8192)
            except BlockingIOError:
                continue
            except OSError as e:
                done[c] = e
                continue
            if not chunk:
                done[c] = ConnectionError("peer closed before a complete JSON document arrived")
                continue
            bufs[c] += chunk
            if len(bufs[c]) > MAX_MESSAGE_BYTES:
                done[c] = ValueError("message larger than any request can be")
                continue
            try:
                done[c] = json.loads(bufs[c].decode())
            except (json.JSONDecodeError, UnicodeDecodeError):
                pass                      # not complete yet
    for c in conns:
        try:
            c.setblocking(True)
        except OSError:
            pass
    return [(c, done[c]) for c in conns]


def _validated(game: Game) -> Game:
    """Type checks of a request before it reaches the model (a malformed field would otherwise
    surface as an exception in the middle of a batch)."""
    if not (isinstance(game.time_control, str) and isinstance(game.moves, list) and isinstance(game.moves_seconds, list)):
        raise ValueError("time_control must be a string, moves and moves_seconds lists")
    for name in ("white_elo", "black_elo"):
        elo = getattr(game, name)
        if elo is not None and (isinstance(elo, bool) or not isinstance(elo, int) or not 0 <= elo <= 10000):
            raise ValueError(f"{name} must be an integer rating")
    # the bot (the side to move) takes the opponent's rating or the system's fixed one; the
    # opponent's own rating has to come with the request, the tokenizer conditions on both
    white_to_move = len(game.moves) % 2 == 0
    if (game.black_elo if white_to_move else game.white_elo) is None:
        raise ValueError("the opponent's rating (the side not to move) is needed")
    if len(game.moves) != len(game.moves_seconds) or not all(isinstance(m, str) for m in game.moves):
        raise ValueError("moves must be strings, one entry of moves_seconds per move")
    if not all(isinstance(t, (int, float)) and not isinstance(t, bool) and t >= 0 for t in game.moves_seconds):
        raise ValueError("moves_seconds must be non-negative numbers")
    game.moves_seconds = [int(t) for t in game.moves_seconds]
    return game


def _answer(conn: socket.socket, res: DecodeResult) -> None:
    send_dict(conn, {"move": res.move, "think_time": res.think_time, "resigned": res.resigned})


def serve(alias: str, model, tokenizer: UCITokenizer, device: str | None = None, host: str = "localhost",
          port: int | None = None, self_test: bool = True, max_requests: int | None = None,
          max_batch: int = 64, batched: bool = True, client_timeout: float = 5.0) -> None:
    system = SYSTEMS[alias]
    algorithm = build_algorithm(alias, model, tokenizer, device, batched=batched, max_batch=max_batch)
    if self_test:
        algorithm_test(algorithm, max_plies=12)
    srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind((host, port if port is not None else system.port))
    srv.listen(64)
    logger.info(f"{alias} listening on {host}:{srv.getsockname()[1]}")
    served = 0
    try:
        while max_requests is None or served < max_requests:
            conns = [srv.accept()[0]]
            # everything already waiting in the backlog joins this batch
            while len(conns) < max_batch and select.select([srv], [], [], 0)[0]:
                conns.append(srv.accept()[0])
            ready: list[tuple[socket.socket, Game]] = []
            for conn, req in read_requests(conns, client_timeout):
                try:
                    if isinstance(req, Exception):
                        raise req
                    conn.settimeout(client_timeout)
                    game = assign_elo(_validated(Game(**req)), system)
                    if not game.legal_moves:              # replays the moves: an illegal game fails here
                        raise ValueError("the game is over: no legal move to answer with")
                    ready.append((conn, game))
                except (ConnectionError, OSError, ValueError, TypeError, KeyError, AttributeError, AssertionError) as e:
                    logger.warning(f"request failed: {type(e).__name__}: {e}")     # a malformed request never ends the server
                    conn.close()
            try:
                if hasattr(algorithm, "decode_batch"):
                    results = iter(decode_batch(algorithm, [g for _, g in ready]) if ready else [])
                else:                                     # one at a time: each answer leaves as soon as it exists
                    results = (algorithm.decode_full(g) for _, g in ready)
                for (conn, _), res in zip(ready, results):
                    try:
                        _answer(conn, res)
                    except (ConnectionError, OSError) as e:
                        logger.warning(f"reply failed: {type(e).__name__}: {e}")
            except KeyboardInterrupt:
                raise
            except Exception as e:
                # a request that passed validation but still broke the decoder: this batch's
                # clients get a closed connection (they retry), the server keeps listening
                logger.warning(f"decoding a batch of {len(ready)} request(s) failed: {type(e).__name__}: {e}")
            finally:
                for conn, _ in ready:
                    conn.close()
                served += len(conns)
    except KeyboardInterrupt:
        logger.info("interrupted")
    finally:
        algorithm.cleanup()
        srv.close()


def main(argv: list[str] | None = None) -> None:
    """``python -m allie_b200.serve.server <alias> [config.yaml] [options]`` - loads
    ``{output_dir}/best.pt`` (or ``--checkpoint``) and serves the system on its registry port."""
    import argparse
    from os.path import join

    from ..config import load_config
    from ..models import initialize_model, load_model_state
    from ..utils.logging import setup_logging

    ap = argparse.ArgumentParser(description="Allie move server")
    ap.add_argument("alias", choices=sorted(SYSTEMS))
    ap.add_argument("config", nargs="?", default="pretrain_config/medium.yaml")
    ap.add_argument("--sequential", action="store_true", help="one request at a time, like the reference server")
    ap.add_argument("--max-batch", type=int, default=64, help="connections answered per batch")
    ap.add_argument("--port", type=int, default=None, help="defaults to the system's registry port")
    ap.add_argument("--host", default="localhost")
    ap.add_argument("--device", default=None)
    ap.add_argument("--checkpoint", default=None, help="defaults to {output_dir}/best.pt; 'none' = random init")
    ap.add_argument("--no-self-test", action="store_true")
    a = ap.parse_args(argv)
    if a.device and a.device.startswith("cuda:") and torch.cuda.is_available():
        torch.cuda.set_device(a.device)         # kernels, streams and the status word follow the current device
    cfg = load_config(a.config)
    setup_logging()
    tokenizer = UCITokenizer(**cfg.data_config.tokenizer_config)
    model = initialize_model(tokenizer, **{**cfg.model_config, "use_pretrained": False})
    path = a.checkpoint or join(cfg.trainer_config.output_dir, "best.pt")
    if path != "none":
        load_model_state(model, torch.load(path, map_location="cpu", weights_only=False)["model"])
    model.eval()
    serve(a.alias, model, tokenizer, device=a.device, host=a.host, port=a.port, self_test=not a.no_self_test,
          max_batch=a.max_batch, batched=not a.sequential)


if __name__ == "__main__":
    main()
