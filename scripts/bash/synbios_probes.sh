#!/usr/bin/env bash
# Probe study of a trained model: cache -> smoke -> pilot -> formal -> summary.  scripts/bash/synbios_probes.sh <data> <model.pt>
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
DATA="${1:?dataset directory}"; CKPT="${2:?exported model.pt}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"; OUT="${OUT:-artifacts/synbios_moe/probes/$(basename "$DATA")}"
CODEC="${CODEC:-gpt2}"; N="$(gpu_count)"; DEVICES="$(seq -s, -f 'cuda:%g' 0 $((N > 0 ? N - 1 : 0)))"; [[ "$N" -gt 0 ]] || DEVICES=cpu
cd "$REPO_ROOT"
[[ -f "$OUT/cache/manifest.json" ]] || "$PYTHON" scripts/synbios_moe.py cache-probes --data "$DATA" --output "$OUT/cache" --codec "$CODEC"
for STAGE in smoke pilot formal; do
  "$PYTHON" scripts/synbios_moe.py probe-pipeline --stage "$STAGE" --config configs/synbios_moe/probe_pipeline.yaml --data "$DATA" \
    --probe-cache "$OUT/cache" --model-config "$MODEL_CONFIG" --checkpoint "$CKPT" --devices "$DEVICES" --codec "$CODEC" --output "$OUT/$STAGE" --quiet
done
"$PYTHON" scripts/synbios_moe.py summarize-probes "$OUT/formal" --output "$OUT/formal/probes.csv"
