from allie_b200.evaluation.utils import (accuracy_from_win_percents, move_quality, stockfish_eval,  # noqa: F401
                                         win_percent)
