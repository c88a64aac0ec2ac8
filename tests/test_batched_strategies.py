"""The many-games-per-call strategies against their one-game counterparts, with a deterministic
fake network (CPU)."""
import torch

from allie_b200.data import Game
from allie_b200.search import (DECODE_STRATEGIES, MCTS, AdaptiveMCTS, BatchedAdaptiveMCTS, BatchedMCTSStrategy,
                               BatchedPolicy, Policy, decode_batch)
from test_batched_mcts import GAMES, FakeRunner, tok_model  # noqa: F401


def _games():
    return [Game("180+0", 1500, 2300, None, False, mv, [1] * len(mv)) for mv in GAMES]


def test_registry_names():
    assert DECODE_STRATEGIES["policy-batched"] is BatchedPolicy
    assert DECODE_STRATEGIES["mcts-batched"] is BatchedMCTSStrategy
    assert DECODE_STRATEGIES["adaptive-mcts-batched"] is BatchedAdaptiveMCTS


def test_policy_batch_matches_single(tok_model):
    tok, model = tok_model
    games = _games()
    one = Policy(model, tok, device="cpu", runner=FakeRunner(len(tok)))
    many = BatchedPolicy(model, tok, device="cpu", runner=FakeRunner(len(tok)))
    got = many.score_batch(games)
    for g, s in zip(games, got):
        want = one.score_full(g, g.legal_moves)
        assert torch.allclose(s.legal_move_probabilities, want.legal_move_probabilities)
        assert s.think_time == want.think_time and s.resigned == want.resigned
    moves = [r.move for r in many.decode_batch(games)]
    assert moves == [one.decode_full(g).move for g in games]
    assert many.runner.calls == 2 * len(games)          # the fake counts positions: two passes over four games


def test_mcts_batch_matches_sequential(tok_model):
    tok, model = tok_model
    games = _games()
    many = BatchedMCTSStrategy(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_trees=3, n_sims=25,
                               anc_max=64)
    got = many.score_batch(games)                       # four games through three trees: two chunks
    for g, s in zip(games, got):
        want = MCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_sims=25).score_full(g, g.legal_moves)
        assert torch.allclose(s.legal_move_probabilities, want.legal_move_probabilities, atol=1e-5)
        assert abs(s.think_time - want.think_time) < 1e-5 and s.resigned == want.resigned
    res = decode_batch(many, games)
    assert [r.move in g.legal_moves for r, g in zip(res, games)] == [True] * 4
    assert many.decode_full(games[2]).move == res[2].move
    assert many.run_stats()["total_rollouts"] == 25 * 9


def test_adaptive_batch_matches_sequential(tok_model):
    tok, model = tok_model
    games = _games()
    many = BatchedAdaptiveMCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_trees=4, mean_n_sims=20,
                               anc_max=64)
    got = many.score_batch(games)
    budgets = set()
    for g, s in zip(games, got):
        ref = AdaptiveMCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), mean_n_sims=20)
        want = ref.score_full(g, g.legal_moves)
        budgets.add(ref.total_rollouts)
        assert torch.allclose(s.legal_move_probabilities, want.legal_move_probabilities, atol=1e-5)
    assert len(budgets) > 1                             # the trees really ran different budgets
    human = BatchedAdaptiveMCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_trees=2, mean_n_sims=10,
                                use_human_move_time=True, anc_max=64)
    g = Game("180+0", 1500, 1600, None, False, GAMES[0], [1, 1, 1], next_move_seconds=30)
    human.score_batch([g])
    assert human.run_stats()["total_rollouts"] == human.convert_time_to_sims((30 - 4.64001) / 6.16533)


def test_decode_batch_falls_back_to_single(tok_model):
    tok, model = tok_model
    one = Policy(model, tok, device="cpu", runner=FakeRunner(len(tok)))
    games = _games()[:2]
    assert [r.move for r in decode_batch(one, games)] == [one.decode_full(g).move for g in games]
