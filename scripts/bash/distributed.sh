#!/usr/bin/env bash
# Multi-GPU training on one node:  scripts/bash/distributed.sh <ddp|fsdp|ep> [nproc] [extra train.py flags]
# Environment: NPROC (when no positional count is given; default: every GPU), CONFIG, MODEL_CONFIG, RESUME (default auto: the
# latest committed checkpoint of the run when one exists, a fresh start otherwise), MAX_RESTARTS, MASTER_PORT.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
STRATEGY="${1:?strategy: ddp, fsdp or ep}"; shift
case "$STRATEGY" in ddp|fsdp|ep) ;; *) echo "usage: $0 <ddp|fsdp|ep> [nproc] [train.py flags]" >&2; exit 2 ;; esac
if [[ "${1:-}" =~ ^[0-9]+$ ]]; then NPROC="$1"; shift; else NPROC="${NPROC:-$(gpu_count)}"; fi
CONFIG="${CONFIG:-configs/server/b200_180gb/runs/${STRATEGY}_${NPROC}gpu.yaml}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"
[[ -f "$REPO_ROOT/$CONFIG" || -f "$CONFIG" ]] || { echo "no run file $CONFIG (presets exist for 1, 2, 4 and 8 GPUs; set CONFIG for others)" >&2; exit 2; }
cd "$REPO_ROOT"
# the same command line serves torchrun's restarts (MAX_RESTARTS): with `auto` each attempt continues from the latest checkpoint
torchrun_local "$NPROC" scripts/train.py --config "$CONFIG" --model-config "$MODEL_CONFIG" --resume "${RESUME:-auto}" "$@"
