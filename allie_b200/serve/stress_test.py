"""Load test for a running move server (reference ``src/server/stress-test.py:1-49``): ``runs``
identical ten-ply requests from a pool of client processes against one port; prints whether every
request was answered, plus the request rate and latency percentiles.

    python -m allie_b200.serve.stress_test 20600 [--runs 100] [--clients 4] [--host localhost]
"""
from __future__ import annotations

import argparse
import multiprocessing
import socket
import time

from ..data import Game
from .server import recv_dict, send_dict

MOVES = ["a2a3", "a7a6", "b2b3", "b7b6", "c2c3", "c7c6", "d2d3", "d7d6", "e2e3", "e7e6"]


def query(target: tuple[str, int]) -> float | None:
    """One request; the latency in seconds, or None if it failed."""
    t0 = time.perf_counter()
    try:
        with socket.create_connection(target, timeout=60) as conn:
            game = Game("180+2", 1234, 2345, None, False, list(MOVES), [0] * len(MOVES))
            send_dict(conn, game.to_dict())
            ans = recv_dict(conn)
        return time.perf_counter() - t0 if "move" in ans else None
    except (OSError, ValueError):
        return None


def run(port: int, runs: int = 100, clients: int = 4, host: str = "localhost") -> dict:
    t0 = time.perf_counter()
    with multiprocessing.get_context("spawn").Pool(clients) as pool:
        lat = pool.map(query, [(host, port)] * runs)
    wall = time.perf_counter() - t0
    ok = sorted(x for x in lat if x is not None)
    pct = lambda q: ok[min(len(ok) - 1, int(q * len(ok)))] if ok else None
    return {"success": len(ok) == runs, "answered": len(ok), "runs": runs, "seconds": wall,
            "requests_per_s": len(ok) / wall, "latency_p50_s": pct(0.5), "latency_p99_s": pct(0.99)}


def main(argv: list[str] | None = None) -> dict:
    ap = argparse.ArgumentParser()
    ap.add_argument("port", type=int)
    ap.add_argument("--runs", type=int, default=100)
    ap.add_argument("--clients", type=int, default=4)
    ap.add_argument("--host", default="localhost")
    a = ap.parse_args(argv)
    res = run(a.port, a.runs, a.clients, a.host)
    print("SUCCESS:", res["success"], res)
    return res


if __name__ == "__main__":
    main()
