from allie_b200.moves import CHESS_MOVES, NUM_CHESS_MOVES  # noqa: F401
