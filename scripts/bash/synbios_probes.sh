#!/usr/bin/env bash
# Probe study of a trained model: cache -> smoke -> pilot -> formal -> summary.
#   scripts/bash/synbios_probes.sh <data directory> <model.pt | checkpoint directory>
#   scripts/bash/synbios_probes.sh <variant> <strategy> [checkpoint | latest]      data and run directory follow from the names
# Environment: STAGE (one of smoke, pilot, formal; default: all three in order), MODEL_CONFIG, OUT, CODEC, PROBE_DEVICES
# (default: every GPU, else cpu), PROBE_GPUS, PROBE_BATCH_ENV (a file of P_BATCH_SIZE= ... lines, e.g. the batch benchmark's
# recommendation), P_BATCH_SIZE, Q_BATCH_SIZE, P_VALIDATION_BATCH_SIZE, Q_VALIDATION_BATCH_SIZE, PROBE_CHECKPOINT_INTERVAL,
# PROBE_LOG_INTERVAL, PROBE_HEARTBEAT_SECONDS, SKIP_PRETRAIN_GATE=1, IGNORE_STAGE_PREREQUISITE=1, REQUIRE_COVERAGE=0.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
FIRST="${1:?dataset directory, or variant (single | multi5_permute)}"; SECOND="${2:?exported model.pt, or strategy (single | ddp | fsdp | ep)}"
if [[ -d "$FIRST" ]]; then
  DATA="$FIRST"; CKPT="$SECOND"; NAME="$(basename "$DATA")"
else
  RUN="synbios_moe_${FIRST//+/_}_${SECOND}"
  DATA="${DATA:-artifacts/synbios_moe/data/${FIRST//+/_}}"; NAME="${RUN#synbios_moe_}"
  CKPT="${3:-latest}"
  if [[ "$CKPT" == latest ]]; then CKPT="artifacts/synbios_moe/checkpoints/$RUN/latest"; fi
  [[ -d "$DATA" ]] || { echo "no dataset at $DATA: run scripts/bash/synbios_moe.sh ${FIRST} ${SECOND} first" >&2; exit 2; }
fi
if [[ -n "${PROBE_BATCH_ENV:-}" ]]; then
  [[ -f "$PROBE_BATCH_ENV" ]] || { echo "PROBE_BATCH_ENV names no file: $PROBE_BATCH_ENV" >&2; exit 2; }
  source "$PROBE_BATCH_ENV"
fi
MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"; OUT="${OUT:-artifacts/synbios_moe/probes/$NAME}"
CODEC="${CODEC:-gpt2}"
if [[ -n "${PROBE_DEVICES:-}" && "$PROBE_DEVICES" != auto ]]; then
  DEVICES="$PROBE_DEVICES"
else
  N="${PROBE_GPUS:-$(gpu_count)}"; DEVICES="$(seq -s, -f 'cuda:%g' 0 $((N > 0 ? N - 1 : 0)))"; [[ "$N" -gt 0 ]] || DEVICES=cpu
fi
COVERAGE=(); if [[ "${REQUIRE_COVERAGE:-1}" == 1 ]]; then COVERAGE=(--require-coverage); fi
EXTRA=(${COVERAGE[@]+"${COVERAGE[@]}"})
if [[ "${SKIP_PRETRAIN_GATE:-0}" == 1 ]]; then EXTRA+=(--skip-gate); fi
if [[ "${IGNORE_STAGE_PREREQUISITE:-0}" == 1 ]]; then EXTRA+=(--ignore-prerequisite); fi
if [[ -n "${P_BATCH_SIZE:-}" ]]; then EXTRA+=(--p-batch-size "$P_BATCH_SIZE"); fi
if [[ -n "${Q_BATCH_SIZE:-}" ]]; then EXTRA+=(--q-batch-size "$Q_BATCH_SIZE"); fi
if [[ -n "${P_VALIDATION_BATCH_SIZE:-}" ]]; then EXTRA+=(--p-validation-batch-size "$P_VALIDATION_BATCH_SIZE"); fi
if [[ -n "${Q_VALIDATION_BATCH_SIZE:-}" ]]; then EXTRA+=(--q-validation-batch-size "$Q_VALIDATION_BATCH_SIZE"); fi
if [[ -n "${PROBE_CHECKPOINT_INTERVAL:-}" ]]; then EXTRA+=(--checkpoint-interval-steps "$PROBE_CHECKPOINT_INTERVAL"); fi
if [[ -n "${PROBE_LOG_INTERVAL:-}" ]]; then EXTRA+=(--log-interval "$PROBE_LOG_INTERVAL"); fi
if [[ -n "${PROBE_HEARTBEAT_SECONDS:-}" ]]; then EXTRA+=(--heartbeat-seconds "$PROBE_HEARTBEAT_SECONDS"); fi

# a cache that no longer matches the dataset is rebuilt, never used
if [[ ! -f "$OUT/cache/manifest.json" ]] || ! "$PYTHON" scripts/synbios_moe.py validate-probe-cache --probe-cache "$OUT/cache" --data "$DATA" > /dev/null 2>&1; then
  FORCE=(); if [[ -e "$OUT/cache" ]]; then FORCE=(--force); fi
  "$PYTHON" scripts/synbios_moe.py cache-probes --data "$DATA" --output "$OUT/cache" --codec "$CODEC" ${FORCE[@]+"${FORCE[@]}"} ${COVERAGE[@]+"${COVERAGE[@]}"}
fi
for S in ${STAGE:-smoke pilot formal}; do
  "$PYTHON" scripts/synbios_moe.py probe-pipeline --stage "$S" --config configs/synbios_moe/probe_pipeline.yaml --data "$DATA" \
    --probe-cache "$OUT/cache" --model-config "$MODEL_CONFIG" --checkpoint "$CKPT" --devices "$DEVICES" --codec "$CODEC" --output "$OUT/$S" --quiet \
    ${EXTRA[@]+"${EXTRA[@]}"}
done
if [[ -d "$OUT/formal" ]]; then
  "$PYTHON" scripts/synbios_moe.py summarize-probes "$OUT/formal" --output "$OUT/formal/probes.csv"
fi
