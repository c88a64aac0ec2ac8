"""Decode strategies on the CPU oracle model with a tiny random network."""
import math
import zlib

import pytest
import torch

from allie_b200.data import Game, UCITokenizer
from allie_b200.models import initialize_model
from allie_b200.search import DECODE_STRATEGIES, AdaptiveMCTS, MCTS, Policy, kl_regularized_policy
from allie_b200.search.runner import Evaluation, ModelRunner


@pytest.fixture(scope="module")
def setup():
    torch.manual_seed(0)
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=2,
                             n_embd=64, n_head=2, n_positions=64)
    model.eval()
    game = Game("180+0", 1500, 1600, None, False, ["e2e4", "e7e5", "g1f3"], [1, 2, 3])
    return tok, model, game


def test_policy_probabilities(setup):
    tok, model, game = setup
    pol = Policy(model, tok, sample=False, device="cpu")
    res = pol.score_full(game, game.legal_moves)
    assert res.legal_move_probabilities.shape == (len(game.legal_moves),)
    assert abs(float(res.legal_move_probabilities.sum()) - 1) < 1e-5
    assert 0 <= res.sampled_move_legal <= 1 and res.all_move_probabilities.shape == (1968,)
    d = pol.decode_full(game)
    assert d.move in game.legal_moves and isinstance(d.resigned, bool)
    # matches a direct forward of the model
    batch = tok.pad_and_collate([game])
    out = model(**batch)
    ids = torch.tensor([tok.token_to_id[m] for m in game.legal_moves])
    want = torch.softmax(out["logits"][0, -1][ids], 0)
    assert torch.allclose(res.legal_move_probabilities, want, atol=1e-6)


class FakeRunner(ModelRunner):
    """Deterministic evaluator: logits/value are hashes of the move list."""

    def __init__(self, vocab):
        self.vocab = vocab
        self.calls = 0

    def evaluate(self, games):
        self.calls += len(games)
        logits, vals, times = [], [], []
        for g in games:
            gen = torch.Generator().manual_seed(zlib.crc32(" ".join(g.moves).encode()))
            logits.append(torch.randn(self.vocab, generator=gen))
            vals.append(torch.tanh(torch.randn((), generator=gen)))
            times.append(torch.randn((), generator=gen) * 0.3)
        return Evaluation(torch.stack(logits), torch.stack(vals), torch.stack(times))


def test_mcts_invariants(setup):
    tok, model, game = setup
    runner = FakeRunner(len(tok))
    m = MCTS(model, tok, sample=False, device="cpu", runner=runner, n_sims=40)
    legal = game.legal_moves
    res = m.score_full(game, legal)
    p = res.legal_move_probabilities
    assert p.shape == (len(legal),) and abs(float(p.sum()) - 1) < 1e-4 and (p >= 0).all()
    assert m.run_stats() == {"total_rollouts": 40}
    # 1 policy forward + 1 root expansion + one evaluation per non-terminal simulation
    assert runner.calls == 42
    # visit-count variant sums to one too
    m2 = MCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_sims=25, kl_reg_solution=False)
    p2 = m2.score_full(game, legal).legal_move_probabilities
    assert abs(float(p2.sum()) - 1) < 1e-6 and float(p2.max()) > 1.0 / len(legal)


def test_mcts_finds_mate_in_one(setup):
    tok, model, _ = setup
    # after 1.f3 e5 2.g4 black mates with Qh4#: a terminal child is worth +1 to the parent
    game = Game("180+0", 1500, 1500, None, False, ["f2f3", "e7e5", "g2g4"], [1, 1, 1])
    m = MCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_sims=300, kl_reg_solution=False)
    legal = game.legal_moves
    p = m.score_full(game, legal).legal_move_probabilities
    assert legal[int(p.argmax())] == "d8h4"


def test_adaptive_budget_and_kl(setup):
    tok, model, game = setup
    a = AdaptiveMCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), mean_n_sims=50)
    assert a.convert_time_to_sims(0.0) == 50 and a.convert_time_to_sims(-10) == 0 and a.convert_time_to_sims(10) == 200
    res = a.score_full(game, game.legal_moves)
    assert abs(float(res.legal_move_probabilities.sum()) - 1) < 1e-3
    assert math.isclose(a.c_puct, 1.25 * math.sqrt(50) / math.sqrt(max(a.total_rollouts, 1)), rel_tol=1e-6) or a.total_rollouts == 0
    pri = torch.tensor([1 / 3, 1 / 3, 1 / 3]); q = torch.tensor([0.1, 0.4, -0.2]); n = torch.tensor([10.0, 30.0, 5.0])
    pi = kl_regularized_policy(pri, q, n, 1.25)
    assert abs(float(pi.sum()) - 1) < 1e-6 and int(pi.argmax()) == 1
    assert set(DECODE_STRATEGIES) >= {"policy", "mcts", "adaptive-mcts"}


def test_precision_argument_is_checked_and_cpu_stays_fp32():
    """``precision`` is the reference's constructor argument: unknown values are refused, and on the
    CPU both accepted values run the fp32 PyTorch model."""
    import pytest

    from allie_b200.data import UCITokenizer
    from allie_b200.models import initialize_model
    from allie_b200.search import DECODE_STRATEGIES
    from allie_b200.search.runner import TorchRunner

    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1, n_embd=32,
                             n_head=1, n_positions=64).eval()
    for prec in (None, "float32", "bfloat16"):
        s = DECODE_STRATEGIES["policy"](model, tok, device="cpu", precision=prec)
        assert isinstance(s.runner, TorchRunner) and next(model.parameters()).dtype == torch.float32
    with pytest.raises(ValueError, match="precision"):
        DECODE_STRATEGIES["policy"](model, tok, device="cpu", precision="float16")
