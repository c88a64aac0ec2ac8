"""Move-server throughput: requests answered per second over real localhost sockets.

Starts the server of one system alias in a thread (random-init GPT-2-medium-shaped model unless
``--small``), then fires ``--requests`` requests from ``--clients`` concurrent client threads, every
request a different random legal game prefix.  Runs the same load twice: the reference's behaviour
(one request per network evaluation / tree search, ``--mode sequential``) and this framework's
(all connections waiting in the backlog share one evaluation or one batched search, ``--mode
batched``), or one of them.

    python bench_serve.py                                  # humanlike (policy), both modes
    python bench_serve.py --alias humanlike-mcts-rb --requests 128
    python bench_serve.py --servers 8 --requests 2048 --clients 512   # one backend process per GPU behind a front door
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


def run_load(alias, model, tok, device, games, clients, batched, max_batch, pool=None):
    """``pool``: None for one in-process server, else ``(config_path, devices)`` for one backend
    process per device behind a front door (``allie_b200/serve/pool.py``)."""
    from allie_b200.serve.server import recv_dict, send_dict, serve

    port = _free_port()
    n = len(games)
    procs = []
    if pool is None:
        th = threading.Thread(target=serve, kwargs=dict(alias=alias, model=model, tokenizer=tok, device=device,
                                                        port=port, self_test=False, max_requests=n + 1,
                                                        max_batch=max_batch, batched=batched), daemon=True)
    else:
        from allie_b200.serve.pool import FrontDoor, start_backends, wait_until_listening

        config_path, devices = pool
        first = 24000 + (os.getpid() % 500) * 16 + (8 if batched else 0)
        procs, ports = start_backends(alias, config_path, devices, first, checkpoint="none", max_batch=max_batch,
                                      sequential=not batched)
        wait_until_listening(ports)
        th = threading.Thread(target=FrontDoor(ports).serve, kwargs=dict(port=port, max_requests=n + len(devices)),
                              daemon=True)
    th.start()
    deadline = time.time() + 600
    while True:                                   # the strategy (engine, KV cache) is built before the socket opens
        try:
            for _ in range(1 if pool is None else len(pool[1])):                   # warm-up request(s)
                with socket.create_connection(("localhost", port), timeout=600) as c:
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
    for p in procs:
        p.terminate()
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
    ap.add_argument("--servers", type=int, default=1,
                    help="more than one: a backend process per GPU (cuda:0..N-1) behind a front door")
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
    pool = None
    if args.servers > 1:
        import tempfile

        from allie_b200.config import save_config

        shape = (dict(base_model="gpt2", n_layer=2, n_embd=256, n_head=4, n_positions=128) if args.small
                 else dict(base_model="gpt2-medium"))
        cfg = {"trainer_config": {"output_dir": tempfile.mkdtemp(prefix="allie_serve_")},
               "data_config": {"tokenizer_config": {"max_length": tok.max_length, "vocab_size_multiple_of": 128}},
               "model_config": dict(use_control_token=True, use_regression_head=True, **shape)}
        path = os.path.join(cfg["trainer_config"]["output_dir"], "config.yaml")
        save_config(cfg, path)
        devices = [f"cuda:{i}" for i in range(args.servers)] if device.startswith("cuda") else ["cpu"] * args.servers
        pool = (path, devices)
    out = {"metric": "move server requests/s", "alias": args.alias, "requests": args.requests,
           "clients": args.clients, "max_batch": args.max_batch, "device": device, "servers": args.servers,
           "model": "tiny" if args.small else "gpt2-medium shape, random init"}
    for mode in (["sequential", "batched"] if args.mode == "both" else [args.mode]):
        out[mode] = run_load(args.alias, model, tok, device, games, args.clients, mode == "batched", args.max_batch,
                             pool)
    if "batched" in out and "sequential" in out and out["sequential"]["requests_per_s"]:
        out["speedup"] = round(out["batched"]["requests_per_s"] / out["sequential"]["requests_per_s"], 2)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
