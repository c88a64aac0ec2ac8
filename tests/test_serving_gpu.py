"""Many-games-per-call strategies on the sm_100a engine: one forward pass for a batch of policy
requests, one KV-cached batched search for a batch of MCTS requests (GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_batched_strategies_on_engine():
    from allie_b200.data import Game, UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.ops import _lib
    from allie_b200.search import BatchedAdaptiveMCTS, BatchedMCTSStrategy, BatchedPolicy, Policy, decode_batch

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=128, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=2,
                             n_embd=256, n_head=4, n_positions=128).eval()
    games = [Game("180+0", 1500, 1600, None, False, mv, [1] * len(mv)) for mv in
             (["e2e4", "e7e5", "g1f3"], ["d2d4", "d7d5", "c2c4", "e7e6", "b1c3", "g8f6"], [], ["f2f3", "e7e5", "g2g4"],
              ["e2e4"])]
    many = BatchedPolicy(model, tok, device="cuda")
    one = Policy(model, tok, device="cuda")
    assert type(many.runner).__name__ == "EngineRunner"
    before = many.runner.calls
    scores = many.score_batch(games)
    assert many.runner.calls == before + 1                      # one pass for the five games
    for g, s in zip(games, scores):
        want = one.score_full(g, g.legal_moves)
        assert torch.allclose(s.legal_move_probabilities, want.legal_move_probabilities, atol=2e-2)
        assert abs(s.white_advantage - want.white_advantage) < 2e-2
    mcts = BatchedMCTSStrategy(model, tok, device="cuda", n_trees=4, n_sims=24, anc_max=64)
    assert type(mcts.evaluator).__name__ == "KVStepEvaluator"
    res = decode_batch(mcts, games)                             # five games through four trees
    assert all(r.move in g.legal_moves for r, g in zip(res, games))
    assert mcts.run_stats()["total_rollouts"] == 24 * 5
    for s in mcts.score_batch(games[:2]):
        assert abs(float(s.legal_move_probabilities.sum()) - 1) < 1e-3
    ada = BatchedAdaptiveMCTS(model, tok, device="cuda", n_trees=4, mean_n_sims=10, anc_max=64)
    res = ada.decode_batch(games[:3])
    assert all(r.move in g.legal_moves for r, g in zip(res, games))
    torch.cuda.synchronize()
    _lib.check_status()
