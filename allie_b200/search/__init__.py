"""Decode / search runtime: strategies, model runners, the batched C++ MCTS and its KV-cached
GPU leaf evaluator."""
from .strategies import (DECODE_STRATEGIES, ActionValue, AdaptiveMCTS, DecodeResult, DecodeStrategy, MCTS,
                         MCTSNode, Policy, ScoreResult, kl_regularized_policy)

from . import external  # noqa: F401,E402  (registers the external baselines)
from .batched_strategies import (BatchedAdaptiveMCTS, BatchedMCTSStrategy, BatchedPolicy,  # noqa: E402
                                 decode_batch)

__all__ = ["DECODE_STRATEGIES", "ActionValue", "AdaptiveMCTS", "DecodeResult", "DecodeStrategy", "MCTS",
           "MCTSNode", "Policy", "ScoreResult", "kl_regularized_policy", "BatchedPolicy", "BatchedMCTSStrategy",
           "BatchedAdaptiveMCTS", "decode_batch"]
