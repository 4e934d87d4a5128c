"""Build and load the sm_100a extension in-tree.

``build_extension()`` compiles every ``csrc`` source with ``-gencode arch=compute_100a,code=sm_100a``
through ``torch.utils.cpp_extension`` (ninja) into ``mini_train_sys_b200/_build`` and copies the
shared object next to the package as ``_mts_b200_ext.so``; nvcc cross-compiles without a GPU.
``load_extension()`` imports that file and never builds implicitly on a GPU box: a missing
extension is an error there, so that a silent library fallback cannot happen
(the reference JIT-builds its extension at import: minitrain/kernels/cuda_ext/build.py:317-355).
"""

from __future__ import annotations

import importlib.util
import os
import shutil
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parents[1]
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
EXT_NAME = "_mts_b200_ext"
EXT_PATH = PKG_DIR / f"{EXT_NAME}.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources() -> list[str]:
    return sorted(str(p) for p in CSRC.iterdir() if p.suffix in (".cu", ".cpp"))


def _stale() -> bool:
    if not EXT_PATH.exists():
        return True
    built = EXT_PATH.stat().st_mtime
    return any(p.stat().st_mtime > built for p in CSRC.iterdir() if p.suffix in (".cu", ".cpp", ".cuh", ".h"))


def build_extension(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return EXT_PATH
    from torch.utils import cpp_extension

    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"   # keeps torch from appending its own arch list
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    BUILD_DIR.mkdir(exist_ok=True)
    cpp_extension.load(name=EXT_NAME, sources=sources(), extra_cflags=["-O3", "-std=c++17"],
                       extra_cuda_cflags=NVCC_FLAGS, extra_include_paths=[str(CSRC)], extra_ldflags=["-lcuda"],
                       build_directory=str(BUILD_DIR), verbose=verbose, is_python_module=False)
    shutil.copy2(BUILD_DIR / f"{EXT_NAME}.so", EXT_PATH)
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
