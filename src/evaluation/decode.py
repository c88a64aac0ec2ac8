from allie_b200.search import (DECODE_STRATEGIES, ActionValue, AdaptiveMCTS, DecodeResult, DecodeStrategy,  # noqa: F401
                               MCTS, MCTSNode, Policy, ScoreResult)
