#!/usr/bin/env bash
# One study end to end: pretrain -> recall + cloze -> probes -> router analysis -> report -> audit.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
VARIANT="${1:-multi5+permute}"; STRATEGY="${2:-fsdp}"
cd "$REPO_ROOT"
DATA="artifacts/synbios_moe/data/${VARIANT//+/_}"; RUN="synbios_moe_${VARIANT//+/_}_${STRATEGY}"
STUDY="artifacts/synbios_moe/studies/$RUN"; CODEC="${CODEC:-gpt2}"; MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"
scripts/bash/synbios_moe.sh "$VARIANT" "$STRATEGY"
CKPT="$(ls -d artifacts/synbios_moe/checkpoints/${RUN}/epoch_* | tail -1)/model.pt"
mkdir -p "$STUDY"
COMMON=(--data "$DATA" --model-config "$MODEL_CONFIG" --checkpoint "$CKPT" --codec "$CODEC")
"$PYTHON" scripts/synbios_moe.py evaluate "${COMMON[@]}" --output "$STUDY/recall.json" --max-items 20000
"$PYTHON" scripts/synbios_moe.py cloze-evaluate "${COMMON[@]}" --output "$STUDY/cloze.json" --max-items 2000
"$PYTHON" scripts/synbios_moe.py analyze "${COMMON[@]}" --output "$STUDY/routes.json"
OUT="$STUDY/probes" scripts/bash/synbios_probes.sh "$DATA" "$CKPT"
"$PYTHON" scripts/synbios_moe.py report-formal-study "$STUDY" --output "$STUDY/report.json"
"$PYTHON" scripts/synbios_moe.py audit-synbios-repository --data "$DATA" --probe-cache "$STUDY/probes/cache" --pipeline "$STUDY/probes/formal"
