#!/usr/bin/env bash
# Dense and MoE operator sweeps with parity gates, then the headline table.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
"$PYTHON" scripts/bench_ops.py run --suite all --profiles "${PROFILES:-project_formal}" --out results/operators "$@"
"$PYTHON" scripts/bench_ops.py summarize results/operators
