"""Build and load the sm_100a extension in-tree.

``build_extension()`` compiles every ``csrc`` source with ``-gencode arch=compute_100a,code=sm_100a``
through ``torch.utils.cpp_extension`` (ninja) into ``mini_train_sys_b200/_build`` and copies the
shared object next to the package as ``_mts_b200_ext.so``; nvcc cross-compiles without a GPU.
``load_extension()`` imports that file and never builds implicitly on a GPU box: a missing
extension is an error there, so that a silent library fallback cannot happen
(the reference JIT-builds its extension at import: minitrain/kernels/cuda_ext/build.py:317-355).
"""

from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import shlex
import shutil
import sys
from dataclasses import dataclass
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parents[1]
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
EXT_NAME = "_mts_b200_ext"
EXT_PATH = PKG_DIR / f"{EXT_NAME}.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]

# Build profiles (``MTS_BUILD_PROFILE``); the reference's counterpart selects head dimensions and dtypes to instantiate
# (minitrain/kernels/cuda_ext/build.py:57-71), here a profile only adds diagnostics to the one set of kernels.
PROFILES = {
    "release": [],
    "trace-gemm": ["-DMTS_GEMM_TRACE"],          # clock64 phase stamps of CTA 0 in the GEMM
    "trace-attention": ["-DMTS_ATTN_TRACE"],     # the same for the attention kernels
    # data-dependent indices (token ids, routing tables, peer slots) are range-checked; violations are recorded in a ring
    # that ``ext.debug_bounds_report()`` returns, the access is skipped and nothing traps (see csrc/debug_bounds.cuh)
    "debug-bounds": ["-DMTS_DEBUG_BOUNDS"],
}


@dataclass(frozen=True)
class BuildConfig:
    """What determines the binary: profile, extra flags, and the content of every source file."""

    profile: str = "release"
    extra_nvcc_flags: tuple[str, ...] = ()
    verbose: bool = False

    @classmethod
    def from_env(cls, env=os.environ) -> "BuildConfig":
        profile = env.get("MTS_BUILD_PROFILE", "release")
        if profile not in PROFILES:
            raise ValueError(f"MTS_BUILD_PROFILE={profile!r}: expected one of {sorted(PROFILES)}")
        extra = tuple(shlex.split(env.get("MTS_EXTRA_NVCC_FLAGS", "")))
        return cls(profile, extra, env.get("MTS_BUILD_VERBOSE", "0") == "1")

    def nvcc_flags(self) -> list[str]:
        return [*NVCC_FLAGS, *PROFILES[self.profile], *self.extra_nvcc_flags]

    def cache_key(self) -> str:
        digest = hashlib.sha256(json.dumps([self.profile, list(self.extra_nvcc_flags), NVCC_FLAGS, "host-defines"]).encode())
        for path in sorted(CSRC.iterdir()):
            if path.suffix in (".cu", ".cpp", ".cuh", ".h"):
                digest.update(path.name.encode())
                digest.update(path.read_bytes())
        return digest.hexdigest()[:16]


def sources() -> list[str]:
    return sorted(str(p) for p in CSRC.iterdir() if p.suffix in (".cu", ".cpp"))


def _stale() -> bool:
    if not EXT_PATH.exists():
        return True
    built = EXT_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in CSRC.iterdir() if p.suffix in (".cu", ".cpp", ".cuh", ".h"))


KEY_PATH = PKG_DIR / "_build" / "cache_key.txt"


def build_extension(force: bool = False, verbose: bool = False, config: BuildConfig | None = None) -> Path:
    config = config or BuildConfig.from_env()
    key = config.cache_key()
    same_key = KEY_PATH.is_file() and KEY_PATH.read_text().strip() == key
    if not force and EXT_PATH.exists() and (same_key or (not KEY_PATH.is_file() and not _stale())):
        return EXT_PATH
    from torch.utils import cpp_extension

    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"   # keeps torch from appending its own arch list
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    BUILD_DIR.mkdir(exist_ok=True)
    # the profile's defines go to the host compiler too: the bindings expose what a diagnostic profile adds
    cpp_extension.load(name=EXT_NAME, sources=sources(), extra_cflags=["-O3", "-std=c++17", *PROFILES[config.profile]],
                       extra_cuda_cflags=config.nvcc_flags(), extra_include_paths=[str(CSRC)], extra_ldflags=["-lcuda"],
                       build_directory=str(BUILD_DIR), verbose=verbose or config.verbose, is_python_module=False)
    shutil.copy2(BUILD_DIR / f"{EXT_NAME}.so", EXT_PATH)
    KEY_PATH.write_text(key + "\n")
    return EXT_PATH


_module = None


def load_extension():
    """Import the in-tree shared object (building it first only when no GPU is present)."""

    global _module
    if _module is not None:
        return _module
    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    if not EXT_PATH.exists():
        if torch.cuda.is_available() and os.environ.get("MTS_ALLOW_JIT_BUILD", "0") != "1":
            raise RuntimeError(f"{EXT_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                               "before using the native backend on a GPU machine")
        build_extension()
    spec = importlib.util.spec_from_file_location(EXT_NAME, EXT_PATH)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[EXT_NAME] = module
    _module = module
    return module
