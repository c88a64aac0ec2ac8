import os as _os
import sys as _sys

_ROOT = _os.path.abspath(_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "..", ".."))
if _ROOT not in _sys.path:          # the framework package sits beside src/: usable without installation
    _sys.path.insert(0, _ROOT)

from allie_b200.evaluation.annotate import annotate, annotate_row, main  # noqa: F401

if __name__ == "__main__":
    main()
