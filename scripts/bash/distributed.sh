#!/usr/bin/env bash
# Multi-GPU training on one node:  scripts/bash/distributed.sh <ddp|fsdp|ep> [nproc] [extra train.py flags]
# Resumes from the latest committed checkpoint of the run when one exists.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
STRATEGY="${1:?strategy: ddp, fsdp or ep}"; shift
NPROC="${1:-$(gpu_count)}"; shift || true
CONFIG="${CONFIG:-configs/server/b200_180gb/runs/${STRATEGY}_${NPROC}gpu.yaml}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"
cd "$REPO_ROOT"
RESUME=()
RUN_DIR="$("$PYTHON" - "$CONFIG" <<'PY'
import sys
sys.path.insert(0, ".")
from mini_train_sys_b200.runtime.config import load_yaml_dict
cfg = load_yaml_dict(sys.argv[1])
print((cfg.get("checkpoint") or {}).get("directory", "checkpoints") + "/" + (cfg.get("run") or {}).get("name", "run"))
PY
)"
if compgen -G "${RUN_DIR}/epoch_*" > /dev/null; then RESUME=(--resume latest); fi
torchrun_local "$NPROC" scripts/train.py --config "$CONFIG" --model-config "$MODEL_CONFIG" "${RESUME[@]}" "$@"
