#!/bin/bash
# Fetches one year of the Lichess rated-games database (monthly .pgn.zst dumps), resumable.
#   allie_b200/etl/download-lichess.sh [year] [target_dir] [parallel_downloads]
# Next step: python -m allie_b200.etl.pgn <dump>.pgn.zst <games>.jsonl
set -Eeuo pipefail
year=${1:-2022}
out=${2:-data/lichess}
jobs=${3:-4}
mkdir -p "$out"
for month in $(seq -w 1 12); do
    name="lichess_db_standard_rated_${year}-${month}.pgn.zst"
    echo "https://database.lichess.org/standard/${name}"
done | xargs -P "$jobs" -I{} sh -c 'f="$1/$(basename "$0" | sed "s/lichess_db_standard_rated_//")"; echo "fetching $0 -> $f"; curl -fsS -C - -o "$f" "$0"' {} "$out"
echo "done: $(ls "$out" | wc -l) files in $out"
