"""Move server round trip over a real localhost socket (CPU)."""
import socket
import threading
import time

import torch

from allie_b200.data import Game, UCITokenizer
from allie_b200.models import initialize_model
from allie_b200.serve import SYSTEMS, recv_dict, send_dict
from allie_b200.serve.server import assign_elo, serve


def _free_port():
    s = socket.socket()
    s.bind(("localhost", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_registry_matches_reference_ports():
    assert SYSTEMS["humanlike"].port == 20600 and SYSTEMS["grandmaster"].elo == 2500
    assert SYSTEMS["humanlike-mcts-rb"].algorithm == "mcts" and SYSTEMS["humanlike-adaptive-rb"].algorithm_config["mean_n_sims"] == 50
    g = assign_elo(Game("180+0", 1200, 1900, None, False, ["e2e4"], [1]), SYSTEMS["humanlike"])
    assert g.black_elo == 1200
    g = assign_elo(Game("180+0", 1200, 1900, None, False, [], []), SYSTEMS["grandmaster"])
    assert g.white_elo == 2500


def test_round_trip_and_broken_client():
    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=1, n_positions=64).eval()
    port = _free_port()
    th = threading.Thread(target=serve, kwargs=dict(alias="grandmaster", model=model, tokenizer=tok, device="cpu",
                                                    port=port, self_test=False, max_requests=10), daemon=True)
    th.start()
    for _ in range(50):
        try:
            socket.create_connection(("localhost", port), timeout=0.2).close()   # broken client: sends nothing
            break
        except OSError:
            time.sleep(0.1)
    for bad in (["e2e5"], ["f2f3", "e7e5", "g2g4", "d8h4"]):             # an illegal move; a finished game
        with socket.create_connection(("localhost", port), timeout=10) as c:
            send_dict(c, Game("180+0", 1500, 1600, None, False, bad, [1] * len(bad)).to_dict())
            assert c.recv(100) == b""                                    # closed without an answer
    for junk in ([1, 2, 3], {"moves": [7]}, {"time_control": "180+0", "white_elo": 1, "black_elo": 2, "outcome": None,
                                             "normal_termination": False, "moves": [12, None], "moves_seconds": [0, 0]},
                 {"time_control": "180+0", "white_elo": "abc", "black_elo": 2, "outcome": None,
                  "normal_termination": False, "moves": ["e2e4"], "moves_seconds": [0]},
                 {"time_control": "180+0", "white_elo": 1500, "black_elo": 1500, "outcome": None,
                  "normal_termination": False, "moves": ["e2e4"], "moves_seconds": []}):
        with socket.create_connection(("localhost", port), timeout=10) as c:
            send_dict(c, junk)
            assert c.recv(100) == b""
    game = Game("180+0", 1500, 1600, None, False, ["e2e4", "e7e5"], [1, 2])
    for _ in range(2):
        with socket.create_connection(("localhost", port), timeout=10) as c:
            send_dict(c, game.to_dict())
            ans = recv_dict(c)
        assert ans["move"] in game.legal_moves and isinstance(ans["resigned"], bool)
        assert isinstance(ans["think_time"], float)
    th.join(timeout=10)
    assert not th.is_alive()


def test_missing_opponent_rating_idle_clients_and_decoder_failures_do_not_end_the_server(monkeypatch):
    """A request that carries only the bot's own rating is refused at validation (the tokenizer
    conditions on both ratings); several idle connections in one batch cost one shared deadline,
    not one timeout each; an exception inside the decoder closes that batch's connections and the
    accept loop goes on."""
    import allie_b200.serve.server as srv_mod

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=1, n_positions=64).eval()
    port = _free_port()
    real = srv_mod.decode_batch
    calls = {"n": 0}

    def flaky(algorithm, games):
        calls["n"] += 1
        if calls["n"] == 1:
            raise RuntimeError("decoder blew up")
        return real(algorithm, games)

    monkeypatch.setattr(srv_mod, "decode_batch", flaky)
    th = threading.Thread(target=serve, kwargs=dict(alias="humanlike", model=model, tokenizer=tok, device="cpu",
                                                    port=port, self_test=False, max_requests=9, client_timeout=1.0),
                          daemon=True)
    th.start()
    for _ in range(50):
        try:
            socket.create_connection(("localhost", port), timeout=0.2).close()
            break
        except OSError:
            time.sleep(0.1)
    # white to move, only white's (the bot's own) rating given
    with socket.create_connection(("localhost", port), timeout=10) as c:
        send_dict(c, Game("180+0", 1500, None, None, False, [], []).to_dict())
        assert c.recv(100) == b""
    game = Game("180+0", 1500, 1600, None, False, ["e2e4", "e7e5"], [1, 2])
    with socket.create_connection(("localhost", port), timeout=10) as c:      # first decode call raises
        send_dict(c, game.to_dict())
        assert c.recv(100) == b""
    with socket.create_connection(("localhost", port), timeout=10) as c:      # the server is still there
        send_dict(c, game.to_dict())
        assert recv_dict(c)["move"] in game.legal_moves
    # four idle connections and one real request arriving together: answered after ONE deadline
    idle = [socket.create_connection(("localhost", port), timeout=10) for _ in range(4)]
    time.sleep(0.3)
    t0 = time.time()
    with socket.create_connection(("localhost", port), timeout=10) as c:
        send_dict(c, game.to_dict())
        assert recv_dict(c)["move"] in game.legal_moves
    assert time.time() - t0 < 3.0
    for c in idle:
        c.close()
    th.join(timeout=10)
    assert not th.is_alive()


def test_waiting_connections_share_one_batched_search():
    """Several clients connect before the server looks at any of them; an MCTS system answers them
    from one batched search, and the stress-test client reports success against a policy system."""
    from allie_b200.serve import stress_test

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=1, n_positions=64).eval()
    port = _free_port()
    th = threading.Thread(target=serve, kwargs=dict(alias="humanlike-mcts-rb", model=model, tokenizer=tok,
                                                    device="cpu", port=port, self_test=False, max_requests=4,
                                                    max_batch=4), daemon=True)
    th.start()
    games = [Game("180+0", 1500, 1600, None, False, mv, [1] * len(mv))
             for mv in (["e2e4"], ["d2d4", "d7d5"], [], ["e2e4", "e7e5", "g1f3"])]
    conns = []
    for g in games:
        for _ in range(50):
            try:
                c = socket.create_connection(("localhost", port), timeout=30)
                break
            except OSError:
                time.sleep(0.1)
        send_dict(c, g.to_dict())
        conns.append(c)
    for c, g in zip(conns, games):
        ans = recv_dict(c)
        c.close()
        assert ans["move"] in g.legal_moves
    th.join(timeout=30)
    assert not th.is_alive()

    port = _free_port()
    th = threading.Thread(target=serve, kwargs=dict(alias="humanlike", model=model, tokenizer=tok, device="cpu",
                                                    port=port, self_test=False, max_requests=7), daemon=True)
    th.start()
    time.sleep(0.5)
    assert stress_test.query(("localhost", port)) is not None
    res = stress_test.run(port, runs=6, clients=2)
    assert res["success"] and res["answered"] == 6 and res["latency_p50_s"] > 0
    th.join(timeout=30)
    assert not th.is_alive()


def test_bot_session_plays_both_colours_against_a_server():
    from allie_b200.serve.client import BotSession, request_move

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=1, n_positions=64).eval()
    port = _free_port()
    th = threading.Thread(target=serve, kwargs=dict(alias="grandmaster", model=model, tokenizer=tok, device="cpu",
                                                    port=port, self_test=False, max_requests=4), daemon=True)
    th.start()
    time.sleep(0.5)
    white = BotSession(port, "180+0", 1500, 1500, bot_is_white=True)
    black = BotSession(port, "180+0", 1500, 1500, bot_is_white=False)
    for _ in range(2):
        a = white.play()
        assert not white.bot_to_move and white.moves[-1] == a["move"]
        black.push(a["move"], 1.0)
        b = black.play()
        white.push(b["move"], 2.0)
    assert white.moves == black.moves and len(white.moves) == 4 and white.moves_seconds[1] == 2
    try:
        black.push("a2a3")
        black.push("a7a6")
        white_turn = BotSession(port, "180+0", 1500, 1500, bot_is_white=False)
        white_turn.play()
        raise AssertionError("expected a turn error")
    except RuntimeError:
        pass
    th.join(timeout=10)
    assert not th.is_alive()
    assert request_move.__doc__


def test_uci_front_end_tracks_game_and_clocks():
    import io

    from allie_b200.serve.uci import UCIFrontEnd

    asked = []

    def ask(game):
        asked.append(game)
        return {"move": game.legal_moves[0], "think_time": 2.4, "resigned": len(game.moves) >= 2}

    out = io.StringIO()
    fe = UCIFrontEnd(ask, out)
    script = ["uci", "setoption name BlackElo value 2100", "isready", "ucinewgame", "position startpos",
              "go wtime 180000 btime 180000 winc 2000 binc 2000"]
    for line in script:
        assert fe.handle(line)
    first = asked[0].legal_moves[0]
    fe.handle(f"position startpos moves {first} e7e5")
    fe.handle("go wtime 179600 btime 175000 winc 2000 binc 2000")       # black used 180 - 175 + 2 = 7 s
    text = out.getvalue().splitlines()
    assert "uciok" in text and "readyok" in text and text[-1] == f"bestmove {asked[1].legal_moves[0]}"
    assert "info string predicted think time 2.4s" in text and "info string the model would resign here" in text
    g = asked[1]
    assert (g.time_control, g.white_elo, g.black_elo) == ("180+2", 1500, 2100)
    assert g.moves == [first, "e7e5"] and g.moves_seconds == [2, 7]      # own predicted time, opponent's from the clock
    fe.handle("position startpos moves d2d4")                            # another game: clocks forgotten
    fe.handle("go movetime 1000")
    assert asked[2].moves == ["d2d4"] and asked[2].moves_seconds == [0]
    down = UCIFrontEnd(lambda game: (_ for _ in ()).throw(ConnectionError("refused")), out)
    down.handle("position startpos")
    down.handle("go")
    assert out.getvalue().splitlines()[-1] == "bestmove 0000"
    assert fe.handle("stop") and not fe.handle("quit")


def test_front_door_spreads_requests_and_skips_a_dead_backend(tmp_path):
    from allie_b200.config import save_config
    from allie_b200.serve.client import request_move
    from allie_b200.serve.pool import FrontDoor, start_backends, wait_until_listening

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=1, n_positions=64).eval()
    ports = [_free_port(), _free_port()]
    dead = _free_port()                                    # nothing listens here
    backends = [threading.Thread(target=serve, kwargs=dict(alias="grandmaster", model=model, tokenizer=tok, device="cpu",
                                                           port=p, self_test=False, max_requests=50), daemon=True)
                for p in ports]
    for b in backends:
        b.start()
    wait_until_listening(ports, timeout=30)
    door = FrontDoor([dead] + ports)
    front = _free_port()
    th = threading.Thread(target=door.serve, kwargs=dict(port=front, max_requests=9), daemon=True)
    th.start()
    time.sleep(0.3)
    game = Game("180+0", 1500, 1600, None, False, ["e2e4", "e7e5"], [1, 2])
    answers = []
    clients = [threading.Thread(target=lambda: answers.append(request_move(front, game))) for _ in range(8)]
    for c in clients:
        c.start()
    for c in clients:
        c.join(timeout=60)
    assert len(answers) == 8 and all(a["move"] in game.legal_moves for a in answers)
    assert door.served[dead] == 0 and all(door.served[p] > 0 for p in ports) and sum(door.served.values()) == 8
    over = Game("180+0", 1500, 1600, None, False, ["f2f3", "e7e5", "g2g4", "d8h4"], [1] * 4)
    try:
        request_move(front, over)                           # refused by the backend, passed on as a closed connection
        raise AssertionError("expected a refusal")
    except ConnectionError:
        pass
    th.join(timeout=30)
    assert not th.is_alive() and all(v == 0 for v in door.in_flight.values())

    # one real backend process started from a config file, as the command line does it
    cfg = {"trainer_config": {"output_dir": str(tmp_path / "run")},
           "data_config": {"tokenizer_config": {"max_length": 64, "vocab_size_multiple_of": 128}},
           "model_config": dict(base_model="gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                                n_embd=32, n_head=1, n_positions=64)}
    save_config(cfg, str(tmp_path / "cfg.yaml"))
    bport = _free_port()
    procs, bports = start_backends("humanlike", str(tmp_path / "cfg.yaml"), ["cpu"], bport, checkpoint="none")
    try:
        wait_until_listening(bports, timeout=120)
        assert request_move(bport, game)["move"] in game.legal_moves
    finally:
        for p in procs:
            p.terminate()
