#!/usr/bin/env bash
# Operator back ends compared on the study's model: validate the native attention first, then the backend suite.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
"$PYTHON" scripts/run_dist_bench.py validate-backend
"$PYTHON" scripts/run_dist_bench.py run --suite backend --config configs/bench/synbios_moe_fsdp.yaml --strategies fsdp \
  --world-sizes "${WORLD:-1}" --ops-backends torch,native --engines fused --batch-sizes "${BATCH:-96}" --repeats 2 "$@"
"$PYTHON" scripts/run_dist_bench.py present-backend
