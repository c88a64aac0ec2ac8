"""The batched C++ MCTS against the sequential Python statement of the algorithm, visit for visit,
with a deterministic fake network (CPU)."""
import zlib

import numpy as np
import pytest
import torch

from allie_b200.data import Game, UCITokenizer
from allie_b200.models import initialize_model
from allie_b200.search import MCTS
from allie_b200.search.batched import BatchedMCTS, RunnerStepEvaluator
from allie_b200.search.runner import Evaluation, ModelRunner


class FakeRunner(ModelRunner):
    def __init__(self, vocab):
        self.vocab, self.calls = vocab, 0

    def evaluate(self, games):
        self.calls += len(games)
        logits, vals, times = [], [], []
        for g in games:
            gen = torch.Generator().manual_seed(zlib.crc32(" ".join(g.moves).encode()))
            logits.append(torch.randn(self.vocab, generator=gen))
            vals.append(torch.tanh(torch.randn((), generator=gen)))
            times.append(torch.randn((), generator=gen) * 0.3)
        return Evaluation(torch.stack(logits), torch.stack(vals), torch.stack(times))


@pytest.fixture(scope="module")
def tok_model():
    torch.manual_seed(0)
    tok = UCITokenizer(max_length=128, vocab_size_multiple_of=128)
    model = initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=1,
                             n_embd=32, n_head=1, n_positions=128)
    return tok, model


GAMES = [
    ["e2e4", "e7e5", "g1f3"],
    ["d2d4", "d7d5", "c2c4", "e7e6", "b1c3"],
    ["f2f3", "e7e5", "g2g4"],                      # mate in one available
    [],
]


@pytest.mark.parametrize("n_sims", [1, 30, 120])
def test_visit_for_visit_parity(tok_model, n_sims):
    tok, model = tok_model
    games = [Game("180+0", 1500, 1600, None, False, mv, [1] * len(mv)) for mv in GAMES]
    bm = BatchedMCTS(tok, RunnerStepEvaluator(FakeRunner(len(tok)), tok, 4, 64, 224), n_trees=4, n_sims=n_sims,
                     anc_max=64)
    res = bm.search(games)
    for g, r in zip(games, res):
        ref = MCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_sims=n_sims)
        legal = g.legal_moves
        want = ref.score_full(g, legal)
        assert r.legal_moves == legal
        # rebuild the oracle's root statistics by running its search once more and reading the tree
        from allie_b200.search.strategies import MCTSNode
        root = MCTSNode(0.0, g)
        ref2 = MCTS(model, tok, device="cpu", runner=FakeRunner(len(tok)), n_sims=n_sims)
        ref2.evaluate_node(root)
        ref2._search(root, n_sims)
        visits = np.array([root.children[m].visit_count for m in legal])
        assert np.array_equal(r.visits, visits), (g.moves, r.visits, visits)
        vals = np.array([root.children[m].value() for m in legal], dtype=np.float32)
        assert np.allclose(r.values, vals, atol=1e-6)
        assert torch.allclose(r.policy, want.legal_move_probabilities, atol=1e-5)
        assert abs(r.think_time - want.think_time) < 1e-5 and r.resigned == want.resigned


def test_partial_batch_and_budget_callable(tok_model):
    tok, _ = tok_model
    games = [Game("180+0", 1500, 1600, None, False, GAMES[0], [1, 1, 1])]
    bm = BatchedMCTS(tok, RunnerStepEvaluator(FakeRunner(len(tok)), tok, 3, 64, 224), n_trees=3, anc_max=64)
    res = bm.search(games, n_sims=lambda t_norm, g: 17)
    assert len(res) == 1 and res[0].n_sims == 17 and int(res[0].visits.sum()) == 17
    res0 = bm.search(games, n_sims=0)
    assert torch.allclose(res0[0].policy, torch.from_numpy(res0[0].priors))


def test_search_refuses_positions_beyond_the_table(tok_model):
    """An evaluator that names the size of the model's position table: a game whose tokens plus the
    search depth would index past it is refused on the host, before anything is evaluated."""
    tok, _ = tok_model
    ev = RunnerStepEvaluator(FakeRunner(len(tok)), tok, 1, 64, 224)
    ev.max_positions = 40
    bm = BatchedMCTS(tok, ev, n_trees=1, n_sims=4, anc_max=64, depth_limit=30)
    game = Game("180+0", 1500, 1600, None, False, GAMES[1], [1] * len(GAMES[1]))     # 8 tokens + depth 30 fits
    assert int(bm.search([game])[0].visits.sum()) == 4
    bm2 = BatchedMCTS(tok, ev, n_trees=1, n_sims=4, anc_max=64, depth_limit=33)
    with pytest.raises(ValueError, match="positions"):
        bm2.search([game])
    assert ev.runner.calls == 1 + 4 + 0        # the refused search evaluated nothing
