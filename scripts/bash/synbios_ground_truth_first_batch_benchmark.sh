#!/usr/bin/env bash
# Batch-size benchmark of the ground-truth-first whole probe (its inputs are one token longer than the P inputs and six
# times as many), per device, merged like the plain probe benchmark.
#   scripts/bash/synbios_ground_truth_first_batch_benchmark.sh <model.pt> <probe cache> <probe pipeline root> [training|validation]
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
CKPT="${1:?exported model.pt}"; CACHE="${2:?probe cache}"; PROBES="${3:?pipeline root with the original P probes}"; MODE="${4:-training}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"; OUT="${OUT:-artifacts/synbios_moe/ground_truth_first_batch_benchmark/$MODE}"
CODEC="${CODEC:-gpt2}"; N="$(gpu_count)"; cd "$REPO_ROOT"; mkdir -p "$OUT"
DEVICES=(cpu); [[ "$N" -gt 0 ]] && DEVICES=($(seq -f 'cuda:%g' 0 $((N - 1))))
pids=(); results=()
for DEVICE in "${DEVICES[@]}"; do
  FILE="$OUT/${DEVICE//:/_}.json"; results+=("$FILE")
  "$PYTHON" scripts/synbios_moe.py probe-batch-benchmark --probe-cache "$CACHE" --probe-dir "$PROBES" --ground-truth-first --kinds p \
    --attribute "${ATTRIBUTE:-university}" --target whole --model-config "$MODEL_CONFIG" --checkpoint "$CKPT" --mode "$MODE" \
    --device "$DEVICE" --codec "$CODEC" --p-batch-sizes "${P_BATCHES:-64,128,256,512,1024}" \
    --memory-limit-percent "${MEMORY_LIMIT:-92}" --output "$FILE" --quiet &
  pids+=("$!")
done
for p in "${pids[@]}"; do wait "$p"; done
"$PYTHON" scripts/synbios_moe.py summarize-probe-batch-benchmarks "${results[@]}" --output "$OUT/summary.json"
