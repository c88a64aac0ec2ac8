#!/bin/bash
# Formats and type-checks the Python sources (isort, black, mypy; all three are configured in pyproject.toml).
set -Eeuo pipefail
cd "$(dirname "$0")"
targets=(allie_b200 src tests bench.py bench_moe.py bench_mcts.py bench_serve.py __graft_entry__.py)
isort "${targets[@]}"
black "${targets[@]}"
mypy allie_b200 src
