"""allie-b200: a Blackwell-native framework with the capabilities of y0mingzhang/allie.

The main entry points are importable from here (resolved on first use, so ``import allie_b200`` stays
cheap): ``UCITokenizer``, ``Game``, ``load_data``, ``load_config``, ``initialize_model``, ``Trainer``,
``DECODE_STRATEGIES``.  Sub-packages: ``models`` (PyTorch oracle + sm_100a engine),
``ops`` (kernel bindings), ``parallel`` (NVLink gradient path, expert parallelism), ``train``,
``search`` (decode strategies, batched MCTS), ``evaluation``, ``serve``, ``etl``, ``chess``.
"""
__version__ = "0.1.0"

_EXPORTS = {
    "UCITokenizer": "allie_b200.data", "Game": "allie_b200.data", "load_data": "allie_b200.data",
    "load_config": "allie_b200.config", "initialize_model": "allie_b200.models",
    "Trainer": "allie_b200.train.trainer", "DECODE_STRATEGIES": "allie_b200.search",
}
__all__ = ["__version__", *_EXPORTS]


def __getattr__(name: str):
    if name in _EXPORTS:
        import importlib

        value = getattr(importlib.import_module(_EXPORTS[name]), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module 'allie_b200' has no attribute {name!r}")
