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
# once both modes have been measured: one file of `export P_BATCH_SIZE=...` lines for synbios_probes.sh (PROBE_BATCH_ENV); it
# is written only when the merged benchmark is complete (every kind bracketed by a slower or infeasible larger batch)
PARENT="$(dirname "$OUT")"
if compgen -G "$PARENT/training/c*.json" > /dev/null && compgen -G "$PARENT/validation/c*.json" > /dev/null; then
  "$PYTHON" scripts/synbios_moe.py summarize-probe-batch-benchmarks "$PARENT"/training/c*.json "$PARENT"/validation/c*.json \
    --output "$PARENT/summary.json" --env-output "$PARENT/recommended.env" > /dev/null 2>&1 \
    && echo "batch sizes for the probe launcher: PROBE_BATCH_ENV=$PARENT/recommended.env" \
    || echo "no recommended.env yet: the merged benchmark is incomplete (see $PARENT/summary.json)" >&2
fi
