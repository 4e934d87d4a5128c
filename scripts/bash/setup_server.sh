#!/usr/bin/env bash
# Preflight of a training node and in-tree build of the CUDA extension.  Changes no GPU setting and installs nothing: the
# interpreter named by PYTHON must already have PyTorch (the image's, or a virtual environment made beforehand).
# Environment: EXPECTED_GPUS (default: every GPU nvidia-smi lists), SKIP_SERVER_CHECK=1, ALLOW_SYSTEM_DISK_STORAGE=1 (proceed
# although setup_storage.sh has not been run), MTS_BUILD_PROFILE.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
if [[ ! -f .mts-storage.env && ! -f .minitrain-storage.env && "${ALLOW_SYSTEM_DISK_STORAGE:-0}" != 1 ]]; then
  echo "note: no storage settings found; run scripts/bash/setup_storage.sh /mounted/disk first to keep checkpoints off the system disk" >&2
fi
"$PYTHON" -c 'import sys; assert sys.version_info[:2] >= (3, 10), sys.version'
if [[ "${SKIP_SERVER_CHECK:-0}" != 1 ]]; then
  EXPECTED_GPUS="${EXPECTED_GPUS:-$( (nvidia-smi --list-gpus 2>/dev/null || true) | wc -l)}"
  "$PYTHON" -m mini_train_sys_b200.runtime.server_check --expected-gpus "$EXPECTED_GPUS" --output artifacts/server_environment.json || true
fi
"$PYTHON" -c 'import __graft_entry__ as g; g.build(); print("extension built")'
