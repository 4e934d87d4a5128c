# Shared helpers of the launchers: repository root, python, torchrun wrapper (always on 127.0.0.1 for single-node runs).
set -euo pipefail
REPO_ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
PYTHON="${PYTHON:-python}"
MASTER_PORT="${MASTER_PORT:-29500}"

torchrun_local() {   # torchrun_local <nproc> <script> [args...]
  local nproc="$1"; shift
  "$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$nproc" --master-addr 127.0.0.1 --master-port "$MASTER_PORT" "$@"
}

gpu_count() { "$PYTHON" -c 'import torch; print(torch.cuda.device_count())'; }
