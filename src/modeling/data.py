from allie_b200.data import (BLITZ_TIME_CONTROLS_TOKENS, NORMAL_TERMINATION_TOKEN, OUTCOME_MASKS,  # noqa: F401
                             TIME_MEAN, TIME_STDEV, Batch, Game, PlayResult, UCITokenizer,
                             apply_time_normalization, json_to_game, json_to_partial_game, load_data,
                             undo_time_normalization)
