#!/usr/bin/env bash
# Put everything a run writes on a data disk:  scripts/bash/setup_storage.sh [/mounted/data/disk]
#
#   <disk>/mini-train-sys/artifacts   datasets, checkpoints, logs, probe studies; `artifacts` in the checkout becomes a link to it
#   <disk>/mini-train-sys/cache/...   torch extensions, torch hub, pip, XDG and tokenizer caches
#   <disk>/mini-train-sys/tmp         TMPDIR of the launchers
#
# and writes `.mts-storage.env` into the checkout, which every launcher sources (common.sh).  Without an argument the disk is
# $MTS_MOUNT_ROOT, else /data.  A path on the root filesystem is refused unless ALLOW_SYSTEM_DISK_STORAGE=1 (a 180 GB GPU
# writes checkpoints that fill a system disk within hours); an `artifacts` directory that already holds files is never moved.
REQUESTED_ROOT="${MTS_STORAGE_ROOT:-${MINITRAIN_STORAGE_ROOT:-}}"      # read before common.sh loads the settings of an earlier run
source "$(dirname "${BASH_SOURCE[0]}")/common.sh"
die() { echo "$*" >&2; exit 2; }

DISK="${1:-${MTS_MOUNT_ROOT:-${MINITRAIN_MOUNT_ROOT:-/data}}}"
[[ "$DISK" == /* && -d "$DISK" ]] || die "usage: $0 /absolute/path/of/a/mounted/disk   ($DISK is not an existing absolute directory)"
DISK="$(realpath "$DISK")"
FILESYSTEM="$(df --output=target "$DISK" 2>/dev/null | tail -n 1)"
[[ -n "$FILESYSTEM" ]] || die "cannot tell which filesystem holds $DISK"
if [[ "$FILESYSTEM" == "/" && "${ALLOW_SYSTEM_DISK_STORAGE:-0}" != "1" ]]; then
  die "$DISK is on the root filesystem: mount the data disk first, or set ALLOW_SYSTEM_DISK_STORAGE=1"
fi
[[ -w "$DISK" ]] || die "$DISK is not writable"

STORE="$(realpath -m "${REQUESTED_ROOT:-$DISK/mini-train-sys}")"
[[ "$STORE/" == "$DISK/"* ]] || die "the storage root $STORE must lie inside $DISK"
mkdir -p "$STORE"/artifacts/synbios_moe/{data,checkpoints,runs,probes} "$STORE"/artifacts/results/{operators,distributed} \
         "$STORE"/cache/{torch_extensions,torch,pip,xdg,huggingface} "$STORE/tmp"

LINK="$REPO_ROOT/artifacts"
if [[ -L "$LINK" ]]; then
  [[ "$(realpath "$LINK")" == "$STORE/artifacts" ]] || die "artifacts already links to $(realpath "$LINK"), not to $STORE/artifacts: remove the link first"
elif [[ -d "$LINK" && -z "$(ls -A "$LINK")" ]]; then
  rmdir "$LINK"; ln -s "$STORE/artifacts" "$LINK"
elif [[ -e "$LINK" ]]; then
  die "$LINK holds files and was left alone: copy it to $STORE/artifacts, move the original away, then run this again"
else
  ln -s "$STORE/artifacts" "$LINK"
fi

ENV_FILE="$REPO_ROOT/.mts-storage.env"
{
  echo "# written by scripts/bash/setup_storage.sh; sourced by the launchers; not for version control"
  printf 'export MTS_STORAGE_ROOT=%q\n' "$STORE"
  printf 'export MINITRAIN_STORAGE_ROOT=%q\n' "$STORE"
  printf 'export TORCH_EXTENSIONS_DIR=%q\n' "$STORE/cache/torch_extensions"
  printf 'export TORCH_HOME=%q\n' "$STORE/cache/torch"
  printf 'export PIP_CACHE_DIR=%q\n' "$STORE/cache/pip"
  printf 'export XDG_CACHE_HOME=%q\n' "$STORE/cache/xdg"
  printf 'export HF_HOME=%q\n' "$STORE/cache/huggingface"
  printf 'export TMPDIR=%q\n' "$STORE/tmp"
} > "$ENV_FILE.partial"
mv "$ENV_FILE.partial" "$ENV_FILE"

df -h "$REPO_ROOT" "$STORE" | sed 's/^/  /'
echo "checkout: $REPO_ROOT"
echo "storage:  $STORE   (artifacts -> $STORE/artifacts; settings in .mts-storage.env)"
echo "next:     scripts/bash/setup_server.sh"
