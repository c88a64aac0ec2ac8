"""Move-server throughput: requests answered per second over real localhost sockets.

Starts the server of one system alias in a thread (random-init GPT-2-medium-shaped model unless
``--small``), then fires ``--requests`` requests from ``--clients`` concurrent client threads, every
request a different random legal game prefix.  Runs the same load twice: the reference's behaviour
(one request per network evaluation / tree search, ``--mode sequential``) and this framework's
(all connections waiting in the backlog share one evaluation or one batched search, ``--mode
batched``), or one of them.

    python bench_serve.py                                  # humanlike (policy), both modes
    python bench_serve.py --alias humanlike-mcts-rb --requests 128
Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _free_port() -> int:
    s = socket.socket()
    s.bind(("localhost", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_load(alias, model, tok, device, games, clients, batched, max_batch):
    from allie_b200.serve.server import recv_dict, send_dict, serve

    port = _free_port()
    n = len(games)
    th = threading.Thread(target=serve, kwargs=dict(alias=alias, model=model, tokenizer=tok, device=device,
                                                    port=port, self_test=False, max_requests=n + 1,
                                                    max_batch=max_batch, batched=batched), daemon=True)
    th.start()
    deadline = time.time() + 600
    while True:                                   # the strategy (engine, KV cache) is built before the socket opens
        try:
            with socket.create_connection(("localhost", port), timeout=5) as c:   # warm-up request
                send_dict(c, games[0].to_dict())
                recv_dict(c)
            break
        except OSError:
            if time.time() > deadline or not th.is_alive():
                raise RuntimeError("server did not come up")
            time.sleep(0.2)
    lat = [None] * n
    nxt = iter(range(n))
    lock = threading.Lock()

    def client():
        while True:
            with lock:
                i = next(nxt, None)
            if i is None:
                return
            t0 = time.perf_counter()
            try:
                with socket.create_connection(("localhost", port), timeout=600) as c:
                    send_dict(c, games[i].to_dict())
                    ans = recv_dict(c)
                if ans["move"] in games[i].legal_moves:
                    lat[i] = time.perf_counter() - t0
            except (OSError, ValueError, KeyError):
                pass

    t0 = time.perf_counter()
    ths = [threading.Thread(target=client) for _ in range(clients)]
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    wall = time.perf_counter() - t0
    th.join(timeout=30)
    ok = sorted(x for x in lat if x is not None)
    return {"answered": len(ok), "seconds": round(wall, 4), "requests_per_s": round(len(ok) / wall, 2),
            "latency_p50_ms": round(1e3 * ok[len(ok) // 2], 2) if ok else None,
            "latency_p99_ms": round(1e3 * ok[min(len(ok) - 1, int(0.99 * len(ok)))], 2) if ok else None}


def main(argv=None):
    import numpy as np
    import torch

    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from bench_mcts import random_games

    ap = argparse.ArgumentParser()
    ap.add_argument("--alias", default="humanlike")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--clients", type=int, default=64)
    ap.add_argument("--max-batch", type=int, default=64)
    ap.add_argument("--mode", default="both", choices=["both", "batched", "sequential"])
    ap.add_argument("--small", action="store_true", help="tiny model (smoke test)")
    ap.add_argument("--device", default=None)
    args = ap.parse_args(argv)
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    if args.small:
        tok = UCITokenizer(max_length=128, vocab_size_multiple_of=128)
        model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=2,
                                 n_embd=256, n_head=4, n_positions=128)
        games = random_games(args.requests, tok, rng, max_tokens=60)
    else:
        tok = UCITokenizer(max_length=512, vocab_size_multiple_of=128)
        model = initialize_model(tok, "gpt2-medium", use_control_token=True, use_regression_head=True)
        games = random_games(args.requests, tok, rng, max_tokens=200)
    model.eval()
    out = {"metric": "move server requests/s", "alias": args.alias, "requests": args.requests,
           "clients": args.clients, "max_batch": args.max_batch, "device": device,
           "model": "tiny" if args.small else "gpt2-medium shape, random init"}
    for mode in (["sequential", "batched"] if args.mode == "both" else [args.mode]):
        out[mode] = run_load(args.alias, model, tok, device, games, args.clients, mode == "batched", args.max_batch)
    if "batched" in out and "sequential" in out and out["sequential"]["requests_per_s"]:
        out["speedup"] = round(out["batched"]["requests_per_s"] / out["sequential"]["requests_per_s"], 2)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
