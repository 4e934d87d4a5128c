#!/usr/bin/env bash
# SynBioS pretraining: prepare data once, then train (auto-resume).  scripts/bash/synbios_moe.sh <variant> <strategy> [nproc]
# Refuses to regenerate a dataset when checkpoints trained on it already exist, and to train two variants whose tables of
# people differ (their comparison would mean nothing).
# Environment: NPROC, DATA, NUM_PEOPLE, SEED, CODEC, CONFIG, FORCE_PREPARE=1 (regenerate the data; refused under existing
# checkpoints), AUTO_RESUME=0 (start fresh although checkpoints exist), RESUME (what to resume from; default auto).
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
VARIANT="${1:-single}"; STRATEGY="${2:-fsdp}"; NPROC="${3:-${NPROC:-$(gpu_count)}}"
DATA="${DATA:-artifacts/synbios_moe/data/${VARIANT//+/_}}"
NUM_PEOPLE="${NUM_PEOPLE:-100000}"; SEED="${SEED:-1337}"; CODEC="${CODEC:-gpt2}"
cd "$REPO_ROOT"
RUN="synbios_moe_${VARIANT//+/_}_${STRATEGY}"
if [[ "${FORCE_PREPARE:-0}" == 1 || ! -f "$DATA/manifest.json" ]]; then
  if compgen -G "artifacts/synbios_moe/checkpoints/${RUN}*/epoch_*" > /dev/null; then
    echo "checkpoints of $RUN exist: refusing to (re)generate $DATA under them; move the checkpoints away first" >&2; exit 2
  fi
  "$PYTHON" scripts/synbios_moe.py prepare --output "$DATA" --variant "${VARIANT//_/+}" --num-people "$NUM_PEOPLE" --seed "$SEED" --codec "$CODEC"
fi
for other in artifacts/synbios_moe/data/*/profiles.jsonl; do       # every variant describes the same people
  if [[ -f "$other" && -f "$DATA/profiles.jsonl" ]] && ! cmp -s "$other" "$DATA/profiles.jsonl"; then
    echo "the people of $DATA differ from those of $(dirname "$other"): a comparison across them is invalid (same NUM_PEOPLE and SEED?)" >&2; exit 2
  fi
done
CONFIG="${CONFIG:-configs/synbios_moe/runs/${VARIANT//+/_}_${STRATEGY}.yaml}"
[[ -f "$CONFIG" ]] || CONFIG="configs/synbios_moe/runs/single_${STRATEGY}.yaml"
RESUME=(--resume "${RESUME:-auto}")   # latest committed checkpoint when there is one; also what a torchrun restart (MAX_RESTARTS) needs
if [[ "${AUTO_RESUME:-1}" != 1 ]]; then RESUME=(); fi
if [[ "$STRATEGY" == single ]]; then
  "$PYTHON" scripts/train.py --config "$CONFIG" ${RESUME[@]+"${RESUME[@]}"}
else
  torchrun_local "$NPROC" scripts/train.py --config "$CONFIG" ${RESUME[@]+"${RESUME[@]}"}
fi
