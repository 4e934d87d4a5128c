# Shared helpers of the launchers: repository root, python, torchrun wrapper (always on 127.0.0.1 for single-node runs).
set -euo pipefail
REPO_ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
# storage settings of this checkout (data disk, caches, TMPDIR), written by setup_storage.sh; a file left by the reference's
# setup script under its own name is honoured too
for _env in "$REPO_ROOT/.minitrain-storage.env" "$REPO_ROOT/.mts-storage.env"; do
  if [[ -f "$_env" ]]; then source "$_env"; fi
done
unset _env
PYTHON="${PYTHON:-python}"
MASTER_PORT="${MASTER_PORT:-29500}"

# MAX_RESTARTS > 0: when a rank exits with an error (a crash, or exit code 3 after a peer was lost) torchrun stops the
# others and starts all of them again with the same command line; with `--resume auto` they continue from the latest
# committed checkpoint (set checkpoint.every_steps to bound what a restart repeats).
MAX_RESTARTS="${MAX_RESTARTS:-0}"

torchrun_local() {   # torchrun_local <nproc> <script> [args...]
  local nproc="$1"; shift
  if [[ "$MAX_RESTARTS" -gt 0 ]]; then
    # restarts need the launcher-hosted rendezvous: a static master address dies with rank 0
    "$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$nproc" --rdzv-backend c10d --rdzv-endpoint "127.0.0.1:$MASTER_PORT" \
      --local-addr 127.0.0.1 --max-restarts "$MAX_RESTARTS" "$@"
  else
    "$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$nproc" --master-addr 127.0.0.1 --master-port "$MASTER_PORT" "$@"
  fi
}

gpu_count() { "$PYTHON" -c 'import torch; print(torch.cuda.device_count())'; }
