#!/usr/bin/env bash
# Smoke gate of the ground-truth-first whole probe: 20 steps with a recovery checkpoint at step 10, run twice; the second
# pass must pick the checkpoint up at exactly step 10 and the result must carry the protocol's fields.
#   OUTPUT=<new dir> scripts/bash/synbios_ground_truth_first_smoke.sh <data> <model.pt> <probe pipeline root>
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
DATA="${1:?dataset directory}"; CKPT="${2:?exported model.pt}"; PROBES="${3:?pipeline root with the original P probes}"
OUTPUT="${OUTPUT:?set OUTPUT to a new smoke-result directory}"
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"; CACHE="${CACHE:-$PROBES/../cache}"; CODEC="${CODEC:-gpt2}"
ATTRIBUTE="${ATTRIBUTE:-university}"; DEVICE="${DEVICE:-$([[ "$(gpu_count)" -gt 0 ]] && echo cuda:0 || echo cpu)}"
cd "$REPO_ROOT"; mkdir -p "$OUTPUT/logs"
run_pass() {   # run_pass <label> <steps>: an interrupted first pass is emulated by stopping at the checkpoint step
  "$PYTHON" scripts/synbios_moe.py ground-truth-first-whole --probe-cache "$CACHE" --probe-dir "$PROBES" --model-config "$MODEL_CONFIG" \
    --checkpoint "$CKPT" --attribute "$ATTRIBUTE" --steps 20 --batch-size "${BATCH:-128}" --evaluation-batch-size "${EVAL_BATCH:-3072}" \
    --checkpoint-interval-steps 10 --max-validation-examples "${MAX_VALIDATION:-12288}" --device "$DEVICE" --codec "$CODEC" \
    --output "$OUTPUT/p_$ATTRIBUTE.json" --recovery-checkpoint "$OUTPUT/p_$ATTRIBUTE.recovery.pt" --log-dir "$OUTPUT/events" --quiet \
    > "$OUTPUT/logs/p_$1.log" 2>&1
}
run_pass initial
run_pass resumed
"$PYTHON" scripts/audit_ground_truth_first_probe.py "$OUTPUT/p_$ATTRIBUTE.json" --expect-resumed-from 10 --max-validation-examples "${MAX_VALIDATION:-12288}"
echo "ground-truth-first smoke and exact-recovery gate passed"
