#!/usr/bin/env bash
# One study end to end: pretrain -> recall + cloze -> probes -> router analysis -> report -> audit.
#   scripts/bash/synbios_full_experiment.sh <variant> <strategy>     one corpus variant (default multi5+permute, fsdp)
#   CONFIRM_FULL_EXPERIMENT=1 scripts/bash/synbios_full_experiment.sh <single|ddp|fsdp|ep>
#       both variants (single, multi5_permute) with one strategy, then their comparison.  Days of GPU time and hundreds of GB
#       of checkpoints: it starts only with the confirmation set, and with more than one GPU only with measured probe batch
#       sizes (PROBE_BATCH_ENV=<probe batch benchmark>/recommended.env) unless ALLOW_DEFAULT_PROBE_BATCHES=1.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
CODEC="${CODEC:-gpt2}"; MODEL_CONFIG="${MODEL_CONFIG:-configs/synbios_moe/model.yaml}"

if [[ -n "${CONFIRM_FULL_EXPERIMENT:-}" || "${1:-}" =~ ^(ddp|fsdp|ep)$ ]]; then
  STRATEGY="${1:-single}"
  case "$STRATEGY" in single|ddp|fsdp|ep) ;; *) echo "usage: CONFIRM_FULL_EXPERIMENT=1 $0 <single|ddp|fsdp|ep>" >&2; exit 2 ;; esac
  if [[ "${CONFIRM_FULL_EXPERIMENT:-0}" != 1 ]]; then
    echo "this trains both corpus variants in full and runs every probe stage on each;" >&2
    echo "check the run files and the free space of the data disk, then set CONFIRM_FULL_EXPERIMENT=1" >&2; exit 2
  fi
  if [[ "$STRATEGY" != single && "${ALLOW_DEFAULT_PROBE_BATCHES:-0}" != 1 ]]; then
    [[ -n "${PROBE_BATCH_ENV:-}" && -f "$PROBE_BATCH_ENV" ]] || {
      echo "a multi-GPU study wants measured probe batch sizes: PROBE_BATCH_ENV=<probe batch benchmark>/recommended.env" >&2; exit 2; }
  fi
  for VARIANT in single multi5_permute; do
    env -u CONFIRM_FULL_EXPERIMENT "${BASH_SOURCE[0]}" "$VARIANT" "$STRATEGY"
  done
  S="artifacts/synbios_moe/studies/synbios_moe_single_${STRATEGY}"; M="artifacts/synbios_moe/studies/synbios_moe_multi5_permute_${STRATEGY}"
  "$PYTHON" scripts/synbios_moe.py compare-formal-studies --single "$S/probes/formal" --multi "$M/probes/formal" \
    --single-cache "$S/probes/cache" --multi-cache "$M/probes/cache" --output "artifacts/synbios_moe/studies/comparison_${STRATEGY}"
  echo "both variants done: artifacts/synbios_moe/studies/comparison_${STRATEGY}"
  exit 0
fi

VARIANT="${1:-multi5+permute}"; STRATEGY="${2:-fsdp}"
DATA="artifacts/synbios_moe/data/${VARIANT//+/_}"; RUN="synbios_moe_${VARIANT//+/_}_${STRATEGY}"
STUDY="artifacts/synbios_moe/studies/$RUN"
scripts/bash/synbios_moe.sh "${VARIANT/multi5_permute/multi5+permute}" "$STRATEGY"
CKPT="$(ls -d artifacts/synbios_moe/checkpoints/${RUN}/epoch_* | tail -1)/model.pt"
mkdir -p "$STUDY"
COMMON=(--data "$DATA" --model-config "$MODEL_CONFIG" --checkpoint "$CKPT" --codec "$CODEC")
"$PYTHON" scripts/synbios_moe.py evaluate "${COMMON[@]}" --output "$STUDY/recall.json" --max-items 20000
"$PYTHON" scripts/synbios_moe.py cloze-evaluate "${COMMON[@]}" --output "$STUDY/cloze.json" --max-items 2000
"$PYTHON" scripts/synbios_moe.py analyze "${COMMON[@]}" --output "$STUDY/routes.json"
OUT="$STUDY/probes" STAGE="" scripts/bash/synbios_probes.sh "$DATA" "$CKPT"
"$PYTHON" scripts/synbios_moe.py report-formal-study "$STUDY" --output "$STUDY/report.json"
"$PYTHON" scripts/synbios_moe.py audit-synbios-repository --data "$DATA" --probe-cache "$STUDY/probes/cache" --pipeline "$STUDY/probes/formal"
