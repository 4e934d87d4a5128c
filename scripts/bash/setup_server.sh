#!/usr/bin/env bash
# Preflight of a training node and in-tree build of the CUDA extension.  Changes no GPU setting.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
"$PYTHON" -m mini_train_sys_b200.runtime.server_check --expected-gpus "${EXPECTED_GPUS:-1}" || true
"$PYTHON" -c 'import __graft_entry__ as g; g.build(); print("extension built")'
