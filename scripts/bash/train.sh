#!/usr/bin/env bash
# Single-process training:  scripts/bash/train.sh [config] [extra train.py flags]
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
CONFIG="${1:-configs/train_single.yaml}"; shift || true
cd "$REPO_ROOT"
exec "$PYTHON" scripts/train.py --config "$CONFIG" "$@"
