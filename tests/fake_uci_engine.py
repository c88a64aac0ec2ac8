"""A stand-in for Stockfish / lc0 in the tests: speaks enough UCI for the client (``uci``,
``setoption``, ``isready``, ``position startpos moves ...``, ``go nodes N``, ``quit``).  Its
evaluation is material balance from the side to move's view (pawn 100 .. queen 900) and its best
move is the first legal move that captures the most valuable piece (else the first legal move).
Options it was given are echoed on ``info string`` lines so a test can see them."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from allie_b200.chess import Board  # noqa: E402

VALUE = {0: 0, 1: 100, 2: 300, 3: 300, 4: 500, 5: 900, 6: 0}


def main():
    board, options = Board(), {}
    for line in sys.stdin:
        parts = line.split()
        if not parts:
            continue
        if parts[0] == "uci":
            print("id name fake\nuciok", flush=True)
        elif parts[0] == "setoption":
            options[parts[2]] = parts[4]
        elif parts[0] == "isready":
            print("readyok", flush=True)
        elif parts[0] == "position":
            if parts[1] == "fen":
                board = Board(" ".join(parts[2:8]))
                rest = parts[8:]
            else:
                board, rest = Board(), parts[2:]
            for mv in rest[1:] if rest[:1] == ["moves"] else []:
                board.push_uci(mv)
        elif parts[0] == "go":
            sign = 1 if board.turn else -1
            cp = sign * sum((1 if board.piece_at(s) > 0 else -1) * VALUE[abs(board.piece_at(s))] for s in range(64))
            legal = board.legal_moves_uci()
            best = max(legal, key=lambda m: VALUE[abs(board.piece_at((int(m[3]) - 1) * 8 + ord(m[2]) - 97))]) if legal else "0000"
            print(f"info string options {sorted(options.items())}", flush=True)
            print(f"info depth 1 score cp {cp} nodes {parts[2] if len(parts) > 2 else 0}", flush=True)
            print(f"bestmove {best}", flush=True)
        elif parts[0] == "quit":
            return


if __name__ == "__main__":
    main()
