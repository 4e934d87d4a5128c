#!/usr/bin/env bash
# Freeze a results tree: catalogue, SHA-256 manifest, audit.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
ROOT_DIR="${1:-results}"
cd "$REPO_ROOT"
"$PYTHON" scripts/build_results_catalog.py "$ROOT_DIR"
"$PYTHON" scripts/audit_results_export.py "$ROOT_DIR"
"$PYTHON" scripts/build_results_manifest.py "$ROOT_DIR"
"$PYTHON" scripts/build_results_manifest.py "$ROOT_DIR" --check
