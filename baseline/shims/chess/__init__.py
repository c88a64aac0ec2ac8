"""Import stand-in for python-chess (not installed here).  The reference's training path only
imports the module; nothing on that path touches a board."""
WHITE, BLACK = True, False


class Board:
    def __init__(self, *a, **k):
        raise NotImplementedError("python-chess is not installed; the training benchmark never builds a board")
