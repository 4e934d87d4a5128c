#!/usr/bin/env bash
# Create the artifact directories a study writes to (datasets, checkpoints, runs, results) under $STORAGE_ROOT.
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
STORAGE_ROOT="${STORAGE_ROOT:-$REPO_ROOT/artifacts}"
mkdir -p "$STORAGE_ROOT"/{synbios_moe/{data,checkpoints,runs,probes},results/{operators,distributed}}
df -h "$STORAGE_ROOT" | tail -1
