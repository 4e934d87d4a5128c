#!/usr/bin/env bash
# Single-process training:  scripts/bash/train.sh [config] [extra train.py flags]
# Environment: CONFIG (when no positional config is given), MODEL_CONFIG, DEVICE (auto | cpu | cuda), RESUME (a checkpoint
# directory, latest, safety or auto).
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
CONFIG="${1:-${CONFIG:-configs/train_single.yaml}}"; shift || true
ARGS=(--config "$CONFIG" --device "${DEVICE:-auto}")
if [[ -n "${MODEL_CONFIG:-}" ]]; then ARGS+=(--model-config "$MODEL_CONFIG"); fi
if [[ -n "${RESUME:-}" ]]; then ARGS+=(--resume "$RESUME"); fi
cd "$REPO_ROOT"
exec "$PYTHON" scripts/train.py "${ARGS[@]}" "$@"
