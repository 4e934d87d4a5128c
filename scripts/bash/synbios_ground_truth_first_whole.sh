#!/usr/bin/env bash
# Ground-truth-first whole probes of all five whole attributes, one job per device in turn, then the report.
#   scripts/bash/synbios_ground_truth_first_whole.sh <data> <model.pt> <probe pipeline root> [steps]
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
DATA="${1:?dataset directory}"; CKPT="${2:?exported model.pt}"; PROBES="${3:?pipeline root with the original P probes}"; STEPS="${4:-3000}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"; CACHE="${CACHE:-$PROBES/../cache}"; CODEC="${CODEC:-gpt2}"
OUT="${OUT:-$PROBES/../ground_truth_first}"; N="$(gpu_count)"
cd "$REPO_ROOT"; mkdir -p "$OUT/logs"
i=0; pids=()
for ATTRIBUTE in birth_city university major company company_city; do
  DEVICE=cpu; [[ "$N" -gt 0 ]] && DEVICE="cuda:$((i % N))"
  # an unfinished job continues from its recovery checkpoint; a finished one (marker newer than the model) is skipped
  if [[ -s "$OUT/$ATTRIBUTE.json" && "$OUT/$ATTRIBUTE.json" -nt "$CKPT" ]]; then i=$((i + 1)); continue; fi
  "$PYTHON" scripts/synbios_moe.py ground-truth-first-whole --probe-cache "$CACHE" --probe-dir "$PROBES" --model-config "$MODEL_CONFIG" \
    --checkpoint "$CKPT" --attribute "$ATTRIBUTE" --steps "$STEPS" --batch-size "${BATCH:-50}" --evaluation-batch-size "${EVAL_BATCH:-1024}" \
    --checkpoint-interval-steps "${CHECKPOINT_EVERY:-500}" --device "$DEVICE" --codec "$CODEC" --output "$OUT/$ATTRIBUTE.json" \
    --recovery-checkpoint "$OUT/recovery/$ATTRIBUTE.pt" --log-dir "$OUT/events/$ATTRIBUTE" --quiet > "$OUT/logs/$ATTRIBUTE.log" 2>&1 &
  pids+=("$!"); i=$((i + 1))
  if [[ "$N" -le 1 || $((i % N)) -eq 0 ]]; then for p in "${pids[@]}"; do wait "$p"; done; pids=(); fi
done
for p in "${pids[@]}"; do wait "$p"; done
"$PYTHON" scripts/synbios_moe.py ground-truth-first-report --run-dir "$OUT" --probe-dir "$PROBES" --output "$OUT/report"
