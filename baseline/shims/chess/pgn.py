"""Stand-in for ``chess.pgn``: ``str(Game().from_board(board))`` as python-chess prints it - the seven
tag roster headers with unknown values, a blank line, and the movetext ending in the result marker,
wrapped at 80 columns."""


class Game:
    def __init__(self):
        self._board = None

    def from_board(self, board) -> "Game":
        self._board = board
        return self

    def __str__(self) -> str:
        headers = "\n".join(f'[{k} "{v}"]' for k, v in (("Event", "?"), ("Site", "?"), ("Date", "????.??.??"),
                                                      ("Round", "?"), ("White", "?"), ("Black", "?"),
                                                      ("Result", "*")))
        body = self._board._core.movetext(columns=80, result="*")
        return headers + "\n\n" + body
