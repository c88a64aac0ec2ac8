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


def test_float32_precision_runs_the_plain_model_on_the_gpu_and_agrees_with_the_engine():
    """``precision="float32"`` (what the reference's evaluation passes) selects the plain PyTorch
    model in fp32 / TF32 on the GPU; the bf16 engine on the same weights gives the same move
    distribution to within bf16 rounding."""
    import copy

    from allie_b200.data import Game, UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.search import MCTS, Policy

    torch.manual_seed(0)
    tok = UCITokenizer(max_length=128, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=2,
                             n_embd=256, n_head=4, n_positions=128).eval()
    exact = Policy(copy.deepcopy(model), tok, device="cuda", precision="float32")
    engine = Policy(model, tok, device="cuda", precision="bfloat16")
    assert type(exact.runner).__name__ == "TorchRunner" and str(exact.runner.device).startswith("cuda")
    assert next(exact.runner.model.parameters()).dtype == torch.float32
    assert type(engine.runner).__name__ == "EngineRunner"
    g = Game("180+0", 1500, 1600, None, False, ["e2e4", "e7e5", "g1f3", "b8c6"], [1, 2, 3, 4])
    a, b = exact.score_full(g, g.legal_moves), engine.score_full(g, g.legal_moves)
    assert torch.allclose(a.legal_move_probabilities, b.legal_move_probabilities, atol=2e-2)
    assert abs(a.white_advantage - b.white_advantage) < 2e-2
    search = MCTS(copy.deepcopy(model), tok, device="cuda", precision="float32", n_sims=8)
    assert search.decode_full(g).move in g.legal_moves
