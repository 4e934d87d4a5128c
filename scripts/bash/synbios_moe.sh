#!/usr/bin/env bash
# SynBioS pretraining: prepare data once, then train (auto-resume).  scripts/bash/synbios_moe.sh <variant> <strategy> [nproc]
# Refuses to regenerate a dataset when checkpoints trained on it already exist.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
VARIANT="${1:-single}"; STRATEGY="${2:-fsdp}"; NPROC="${3:-$(gpu_count)}"
DATA="${DATA:-artifacts/synbios_moe/data/${VARIANT//+/_}}"
NUM_PEOPLE="${NUM_PEOPLE:-100000}"; SEED="${SEED:-1337}"; CODEC="${CODEC:-gpt2}"
cd "$REPO_ROOT"
RUN="synbios_moe_${VARIANT//+/_}_${STRATEGY}"
if [[ ! -f "$DATA/manifest.json" ]]; then
  if compgen -G "artifacts/synbios_moe/checkpoints/${RUN}*/epoch_*" > /dev/null; then
    echo "checkpoints of $RUN exist but $DATA is missing: refusing to regenerate the data under them" >&2; exit 2
  fi
  "$PYTHON" scripts/synbios_moe.py prepare --output "$DATA" --variant "$VARIANT" --num-people "$NUM_PEOPLE" --seed "$SEED" --codec "$CODEC"
fi
CONFIG="${CONFIG:-configs/synbios_moe/runs/${VARIANT//+/_}_${STRATEGY}.yaml}"
[[ -f "$CONFIG" ]] || CONFIG="configs/synbios_moe/runs/single_${STRATEGY}.yaml"
RESUME=(--resume auto)      # latest committed checkpoint when there is one; also what a torchrun restart (MAX_RESTARTS) needs
if [[ "$STRATEGY" == single ]]; then
  "$PYTHON" scripts/train.py --config "$CONFIG" "${RESUME[@]}"
else
  torchrun_local "$NPROC" scripts/train.py --config "$CONFIG" "${RESUME[@]}"
fi
