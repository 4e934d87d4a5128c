#!/usr/bin/env bash
# Weak-scaling and capacity suites of the headline configuration on 1/2/4/8 GPUs.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
"$PYTHON" scripts/run_dist_bench.py inventory > /dev/null
"$PYTHON" scripts/run_dist_bench.py run --suite weak --world-sizes "${WORLDS:-1,2,4,8}" --batch-sizes 96 --repeats 2 "$@"
"$PYTHON" scripts/run_dist_bench.py run --suite capacity --world-sizes "${CAP_WORLDS:-1,8}" --batch-sizes 32,64,96,128,192,256 --repeats 2 "$@"
"$PYTHON" scripts/run_dist_bench.py present-weak; "$PYTHON" scripts/run_dist_bench.py present-capacity
