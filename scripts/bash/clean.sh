#!/usr/bin/env bash
# Remove build products and caches of this checkout (never data, checkpoints or results).
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
cd "$REPO_ROOT"
find . -name __pycache__ -type d -prune -exec rm -rf {} +
rm -rf mini_train_sys_b200/_build .pytest_cache
rm -f mini_train_sys_b200/_mts_b200_ext.so
