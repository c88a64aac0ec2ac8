from allie_b200.evaluation.utils import (accuracy_from_win_percents, move_quality, stockfish_eval,  # noqa: F401
                                         win_percent)
from allie_b200.evaluation.utils import get_engine as get_stockfish_engine  # noqa: F401,E402


def compute_centipawn_loss_and_accuracy(board, move_uci: str):
    """Reference-compatible call shape: a board (anything with ``move_stack`` of UCI strings) and a move."""
    return move_quality([str(m) for m in board.move_stack], move_uci)
from allie_b200.evaluation.utils import accuracy_from_win_percents as compute_accuracy_from_win_percents  # noqa: F401,E402
from allie_b200.evaluation.utils import stockfish_eval_fen as compute_white_centipawn_score  # noqa: F401,E402
from allie_b200.evaluation.utils import win_percent as compute_win_percents_from_eval  # noqa: F401,E402
