"""Stand-in for ``chess.engine``: the names the reference imports.  Starting an engine through it is
not supported (the reference's Stockfish / lc0 paths are not run through the stand-in)."""


class Limit:
    def __init__(self, **kwargs):
        self.__dict__.update(kwargs)


class SimpleEngine:
    @classmethod
    def popen_uci(cls, *args, **kwargs):
        raise NotImplementedError("python-chess is not installed: no engine process through the stand-in")
