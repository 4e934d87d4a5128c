#!/usr/bin/env bash
# Probe batch-size benchmark on every visible GPU (one process per device), then the merged recommendation.
#   scripts/bash/synbios_probe_batch_benchmark.sh <model.pt> <probe cache> [training|validation]
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
CKPT="${1:?exported model.pt}"; CACHE="${2:?probe cache}"; MODE="${3:-training}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"; OUT="${OUT:-artifacts/synbios_moe/probe_batch_benchmark/$MODE}"; CODEC="${CODEC:-gpt2}"
N="$(gpu_count)"; cd "$REPO_ROOT"; mkdir -p "$OUT"
DEVICES=(cpu); [[ "$N" -gt 0 ]] && DEVICES=($(seq -f 'cuda:%g' 0 $((N - 1))))
pids=(); results=()
for DEVICE in "${DEVICES[@]}"; do
  FILE="$OUT/${DEVICE//:/_}.json"; results+=("$FILE")
  "$PYTHON" scripts/synbios_moe.py probe-batch-benchmark --probe-cache "$CACHE" --model-config "$MODEL_CONFIG" --checkpoint "$CKPT" \
    --mode "$MODE" --device "$DEVICE" --codec "$CODEC" --p-batch-sizes "${P_BATCHES:-25,50,100,200,400}" \
    --q-batch-sizes "${Q_BATCHES:-100,200,400,800,1600}" --memory-limit-percent "${MEMORY_LIMIT:-92}" --output "$FILE" --quiet &
  pids+=("$!")
done
for p in "${pids[@]}"; do wait "$p"; done
"$PYTHON" scripts/synbios_moe.py summarize-probe-batch-benchmarks "${results[@]}" --output "$OUT/summary.json"
