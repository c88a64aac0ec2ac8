"""Tokenizer / vocabulary golden tests (CPU)."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from allie_b200.data import (BLITZ_TIME_CONTROLS_TOKENS, Game, TIME_MEAN, TIME_STDEV, UCITokenizer,
                             apply_time_normalization, json_to_game, json_to_partial_game,
                             undo_time_normalization)
from allie_b200.moves import CHESS_MOVES, NUM_CHESS_MOVES, VOCAB_SHA256, vocabulary_digest


def test_vocabulary_digest():
    assert NUM_CHESS_MOVES == 1968
    assert vocabulary_digest() == VOCAB_SHA256
    assert CHESS_MOVES[0] == "a1h8" and CHESS_MOVES[1456] == "a1b3" and CHESS_MOVES[-1] == "h2h1n"
    assert len(set(CHESS_MOVES)) == 1968


def test_special_ids_and_padding():
    tok = UCITokenizer(max_length=512)
    assert len(tok) == 1997
    assert (tok.token_to_id["180+0"], tok.resigned_token_id, tok.bos_token_id, tok.eos_token_id,
            tok.unk_token_id, tok.pad_token_id) == (1968, 1992, 1993, 1994, 1995, 1996)
    assert len(BLITZ_TIME_CONTROLS_TOKENS) == 24
    assert len(UCITokenizer(vocab_size_multiple_of=128)) == 2048
    assert len(UCITokenizer(vocab_size_multiple_of=64)) == 2048


def _game(moves, secs, outcome="1-0", normal=True):
    return Game("180+0", 1500, 1700, outcome, normal, moves, secs)


def test_tokenize_layout():
    tok = UCITokenizer(max_length=32, vocab_size_multiple_of=128)
    g = _game(["e2e4", "e7e5", "g1f3"], [3, 0, 12], outcome="0-1")
    w = tok.tokenize(g)
    ids = w & 0x3FFF
    assert list(ids[:2]) == [2048 + 1500, 2048 + 1700]
    assert ids[2] == tok.token_to_id["180+0"]
    assert [tok.tokens[i] for i in ids[3:6]] == ["e2e4", "e7e5", "g1f3"]
    assert ids[6] == tok.resigned_token_id and ids[7] == tok.eos_token_id
    # think time of move k rides on the word before it
    assert list(w[2:6] >> 16) == [4, 1, 13, 0]
    assert set(((w & 0xFFFF) >> 14).tolist()) == {2}
    # no elo / no time control variants
    w2 = tok.tokenize(g, add_elo=False, add_time_control=False)
    assert (w2[0] & 0x3FFF) == tok.bos_token_id and (w2[1] & 0x3FFF) == tok.unk_token_id


def test_pad_and_collate_labels():
    tok = UCITokenizer(max_length=16, vocab_size_multiple_of=128)
    g1 = _game(["e2e4", "e7e5"], [5, 70], outcome="1/2-1/2", normal=False)
    g2 = _game(["d2d4"], [1], outcome=None, normal=False)
    b = tok.pad_and_collate([g1, g2])
    assert b["input_ids"].shape == (2, 6)
    assert b["attention_mask"][1].tolist() == [1, 1, 1, 1, 0, 0]
    assert b["labels"][0, 0].item() == -100 and b["labels"][0, 1].item() == -100   # ELO ids ignored
    assert b["labels"][1, 4].item() == -100                                        # pad ignored
    assert b["value_labels"][0].tolist() == [0.0] * 6                               # draw
    assert b["value_labels"][1, :4].tolist() == [1.0] * 4 and b["value_labels"][1, 4].item() == -100
    t = b["time_labels"][0]
    assert t[0].item() == -100 and abs(t[2].item() - (5 - TIME_MEAN) / TIME_STDEV) < 1e-6
    assert abs(t[3].item() - (60 - TIME_MEAN) / TIME_STDEV) < 1e-6                  # clamped to 60 s
    assert b["position_ids"][1].tolist() == [0, 1, 2, 3, 3, 3]


def test_raw_window_path_matches():
    tok = UCITokenizer(max_length=8, vocab_size_multiple_of=128)
    g = _game(["e2e4", "e7e5", "g1f3", "b8c6"], [1, 2, 3, 4])
    w = tok.tokenize(g)[:8]
    a = tok.pad_and_collate([g])
    b = tok.pad_and_collate([w])
    for k in a:
        assert torch.equal(a[k].float(), b[k].float()), k


@settings(max_examples=50, deadline=None)
@given(st.lists(st.tuples(st.integers(0, 1967), st.integers(0, 600)), min_size=1, max_size=40),
       st.sampled_from(["1-0", "0-1", "1/2-1/2"]), st.integers(500, 3000), st.integers(500, 3000))
def test_bit_packing_round_trip(pairs, outcome, we, be):
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    moves = [CHESS_MOVES[i] for i, _ in pairs]
    secs = [s for _, s in pairs]
    g = Game("300+0", we, be, outcome, True, moves, secs)
    w = tok.tokenize(g)
    assert w.dtype == np.uint32
    ids = (w & 0x3FFF).tolist()
    assert ids[0] - len(tok) == we and ids[1] - len(tok) == be
    assert [tok.tokens[i] for i in ids[3:3 + len(moves)]] == moves
    assert ((w[2:2 + len(moves)] >> 16) - 1).tolist() == secs
    assert all(int(x) == {"1-0": 0, "1/2-1/2": 1, "0-1": 2}[outcome] for x in (w & 0xFFFF) >> 14)


def test_time_normalisation_and_json():
    assert abs(undo_time_normalization(apply_time_normalization(10)) - 10) < 1e-9
    assert apply_time_normalization(1000) == apply_time_normalization(60)
    row = {"time-control": "180+0", "white-elo": "1500", "black-elo": 1600, "result": "*",
           "termination": "Normal", "moves-uci": "e2e4 e7e5", "moves-seconds": [1, 2]}
    g = json_to_game(row)
    assert g.outcome == "1/2-1/2" and g.normal_termination and g.white_elo == 1500
    p = json_to_partial_game(row, 1)
    assert p.moves == ["e2e4"] and p.next_move_seconds == 2 and p.outcome is None
    assert Game.from_dict(g.to_dict()) == g
