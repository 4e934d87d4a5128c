#!/usr/bin/env bash
# Multi-GPU training on one node:  scripts/bash/distributed.sh <ddp|fsdp|ep> [nproc] [extra train.py flags]
# Resumes from the latest committed checkpoint of the run when one exists.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
STRATEGY="${1:?strategy: ddp, fsdp or ep}"; shift
NPROC="${1:-$(gpu_count)}"; shift || true
CONFIG="${CONFIG:-configs/server/b200_180gb/runs/${STRATEGY}_${NPROC}gpu.yaml}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"
cd "$REPO_ROOT"
# `--resume auto`: the latest committed checkpoint of the run when there is one, a fresh start otherwise; the same command line
# therefore also serves torchrun's restarts (MAX_RESTARTS)
torchrun_local "$NPROC" scripts/train.py --config "$CONFIG" --model-config "$MODEL_CONFIG" --resume auto "$@"
