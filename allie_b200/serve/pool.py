"""One move server per GPU behind the system's registry port.

The reference runs one server process per system alias on one GPU (``scripts/run-server.sh:26-29``).
On an 8-GPU box this module starts ``--gpus N`` backend servers of one alias (processes of their own,
each with its model on its own device, listening on consecutive private ports) and a front door on
the registry port that hands every incoming connection to the backend with the fewest requests in
flight.  Clients keep the reference's protocol and port; the backends keep batching whatever waits
in their backlog.

    python -m allie_b200.serve.pool humanlike-adaptive-rb pretrain_config/medium.yaml --gpus 8

A backend that cannot be reached is skipped (its request goes to the next one) and tried again
later; the front door itself only copies one JSON document in each direction per connection.
"""
from __future__ import annotations

import argparse
import logging
import multiprocessing
import socket
import threading
import time

from .server import SYSTEMS, recv_dict, send_dict

logger = logging.getLogger(__name__)


def _backend_main(alias: str, config: str, checkpoint: str | None, device: str, port: int, max_batch: int,
                  sequential: bool, n_backends: int = 1) -> None:
    import os

    import torch

    from .server import main as server_main

    # the backends share the host's cores: N processes that each start one worker thread per core
    # oversubscribe them (measured on 8 cores with 2 CPU backends: 90x slower under concurrent load)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, n_backends)))

    argv = [alias, config, "--device", device, "--port", str(port), "--max-batch", str(max_batch), "--no-self-test"]
    if checkpoint:
        argv += ["--checkpoint", checkpoint]
    if sequential:
        argv.append("--sequential")
    server_main(argv)


class FrontDoor:
    """Accepts client connections and relays each to the least busy backend port."""

    def __init__(self, backend_ports: list[int], host: str = "localhost", backend_timeout: float = 600.0):
        self.ports, self.host, self.timeout = list(backend_ports), host, backend_timeout
        self.in_flight = {p: 0 for p in self.ports}
        self.served = {p: 0 for p in self.ports}
        self.down_until = {p: 0.0 for p in self.ports}
        self.lock = threading.Lock()

    def _pick(self, exclude: set[int]) -> int | None:
        now = time.time()
        with self.lock:
            live = [p for p in self.ports if p not in exclude and self.down_until[p] <= now]
            if not live:
                live = [p for p in self.ports if p not in exclude]      # everything marked down: try anyway
            if not live:
                return None
            port = min(live, key=lambda p: (self.in_flight[p], self.served[p]))
            self.in_flight[port] += 1
            return port

    def relay(self, client: socket.socket) -> None:
        tried: set[int] = set()
        try:
            client.settimeout(30.0)
            request = recv_dict(client)
            while True:
                port = self._pick(tried)
                if port is None:
                    logger.warning("no backend could take the request")
                    return
                try:
                    with socket.create_connection((self.host, port), timeout=self.timeout) as backend:
                        send_dict(backend, request)
                        answer = recv_dict(backend)
                    send_dict(client, answer)
                    with self.lock:
                        self.served[port] += 1
                    return
                except (ConnectionRefusedError, socket.timeout):
                    tried.add(port)
                    with self.lock:
                        self.down_until[port] = time.time() + 5.0
                except ConnectionError:
                    return          # the backend refused this request (an illegal or finished game): pass that on
                finally:
                    with self.lock:
                        self.in_flight[port] -= 1
        except (ConnectionError, OSError, ValueError) as e:
            logger.warning(f"request failed at the front door: {type(e).__name__}: {e}")
        finally:
            client.close()

    def serve(self, port: int, max_requests: int | None = None) -> None:
        srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((self.host, port))
        srv.listen(256)
        logger.info(f"front door on {self.host}:{port} -> backends {self.ports}")
        n, threads = 0, []
        try:
            while max_requests is None or n < max_requests:
                conn, _ = srv.accept()
                t = threading.Thread(target=self.relay, args=(conn,), daemon=True)
                t.start()
                threads.append(t)
                threads = [t for t in threads if t.is_alive()]
                n += 1
        except KeyboardInterrupt:
            logger.info("interrupted")
        finally:
            for t in threads:
                t.join(timeout=self.timeout)
            srv.close()


def start_backends(alias: str, config: str, devices: list[str], first_port: int, checkpoint: str | None = None,
                   max_batch: int = 64, sequential: bool = False) -> tuple[list, list[int]]:
    """Starts one server process per device; returns (processes, ports)."""
    ctx = multiprocessing.get_context("spawn")
    procs, ports = [], []
    for i, dev in enumerate(devices):
        port = first_port + i
        p = ctx.Process(target=_backend_main,
                        args=(alias, config, checkpoint, dev, port, max_batch, sequential, len(devices)), daemon=True)
        p.start()
        procs.append(p)
        ports.append(port)
    return procs, ports


def wait_until_listening(ports: list[int], host: str = "localhost", timeout: float = 600.0) -> None:
    deadline = time.time() + timeout
    for port in ports:
        while True:
            try:
                socket.create_connection((host, port), timeout=1.0).close()
                break
            except OSError:
                if time.time() > deadline:
                    raise RuntimeError(f"backend on port {port} did not come up")
                time.sleep(0.2)


def main(argv: list[str] | None = None) -> None:
    from ..utils.logging import setup_logging

    ap = argparse.ArgumentParser(description="One Allie move server per GPU behind one port")
    ap.add_argument("alias", choices=sorted(SYSTEMS))
    ap.add_argument("config", nargs="?", default="pretrain_config/medium.yaml")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--devices", default=None, help="comma separated device list instead of cuda:0..N-1")
    ap.add_argument("--port", type=int, default=None, help="front door; defaults to the system's registry port")
    ap.add_argument("--backend-port", type=int, default=None, help="first backend port; defaults to front door + 1000")
    ap.add_argument("--max-batch", type=int, default=64)
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--sequential", action="store_true")
    a = ap.parse_args(argv)
    setup_logging()
    devices = a.devices.split(",") if a.devices else [f"cuda:{i}" for i in range(a.gpus)]
    port = a.port if a.port is not None else SYSTEMS[a.alias].port
    first = a.backend_port if a.backend_port is not None else port + 1000
    procs, ports = start_backends(a.alias, a.config, devices, first, a.checkpoint, a.max_batch, a.sequential)
    try:
        wait_until_listening(ports)
        FrontDoor(ports).serve(port)
    finally:
        for p in procs:
            p.terminate()


if __name__ == "__main__":
    main()
