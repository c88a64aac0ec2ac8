#!/bin/bash
# One B200 hosts every system alias: a move server per alias plus the lichess-bot client that
# forwards games to them.  Runs under SLURM (requeues itself shortly before the time limit) or
# directly from a shell.
#   sbatch allie_b200/serve/run-server.sh [config.yaml]        or        bash allie_b200/serve/run-server.sh
#SBATCH --job-name=allie-servers
#SBATCH --time=7-00:00:00
#SBATCH --gres=gpu:1
#SBATCH --cpus-per-task=16
#SBATCH --mem=100GB
#SBATCH --signal=B:SIGUSR1@600
set -Eeuo pipefail
config=${1:-pretrain_config/medium.yaml}
logs=${ALLIE_SERVER_LOGS:-server-logs}
bot_dir=${ALLIE_LICHESS_BOT_DIR:-lichess-bot}
mkdir -p "$logs"
pids=()

stop_children() {
    # only the processes this script started, by their ids
    for pid in "${pids[@]}"; do kill -INT "$pid" 2>/dev/null || true; done
}
requeue() {
    echo "time limit near at $(date): stopping children"
    stop_children
    if [ -n "${SLURM_JOB_ID:-}" ]; then
        echo "requeueing job $SLURM_JOB_ID"
        scontrol requeue "$SLURM_JOB_ID"
    fi
}
trap requeue SIGUSR1
trap 'stop_children; exit 0' SIGINT SIGTERM EXIT

aliases=$(python -c 'from allie_b200.serve import SYSTEMS; print(" ".join(SYSTEMS))')
# ALLIE_GPUS_PER_SYSTEM > 1: every system gets that many backend servers (one per GPU) behind its port
gpus_per_system=${ALLIE_GPUS_PER_SYSTEM:-1}
for alias in $aliases; do
    if [ "$gpus_per_system" -gt 1 ]; then
        python -u -m allie_b200.serve.pool "$alias" "$config" --gpus "$gpus_per_system" \
            >"$logs/$alias.out" 2>"$logs/$alias.err" &
    else
        python -u -m allie_b200.serve.server "$alias" "$config" >"$logs/$alias.out" 2>"$logs/$alias.err" &
    fi
    pids+=($!)
done

# the servers load weights and run their self test before they listen
sleep "${ALLIE_SERVER_WARMUP_SECONDS:-120}"
if [ -d "$bot_dir" ]; then
    (cd "$bot_dir" && exec python -u lichess-bot.py) >"$logs/bot.out" 2>"$logs/bot.err" &
    pids+=($!)
else
    echo "no $bot_dir directory: servers only"
fi
echo "all launched: ${pids[*]}"
wait
