"""Ahead-of-time build and loading of the sm_100a extension (`csrc/`).

The shared object is produced in-tree (``csrc/_build/lm_engine_b200_C.so``) with nvcc cross-compiling for
``sm_100a`` so that it can be built on a machine without a GPU and shipped next to the sources.
"""

from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

_EXT_NAME = "lm_engine_b200_C"
_REPO_ROOT = Path(__file__).resolve().parents[2]
_CSRC = _REPO_ROOT / "csrc"
_BUILD_DIR = _CSRC / "_build"

_MODULE = None


def extension_sources() -> list[str]:
    sources = []
    for pattern in ("*.cpp", "*.cu", "*/*.cpp", "*/*.cu"):
        sources.extend(str(p) for p in sorted(_CSRC.glob(pattern)) if "_build" not in p.parts)
    return sources


def shared_object_path() -> Path:
    return _BUILD_DIR / f"{_EXT_NAME}.so"


def _is_stale() -> bool:
    so = shared_object_path()
    if not so.exists():
        return True
    built = so.stat().st_mtime
    deps = extension_sources() + [str(p) for p in _CSRC.glob("*/*.h")] + [str(p) for p in _CSRC.glob("*/*.cuh")]
    return any(os.path.getmtime(p) > built for p in deps)


def build_extension(verbose: bool = False, force: bool = False):
    """Compile every source under ``csrc/`` for sm_100a and return the loaded module."""
    from torch.utils import cpp_extension

    _BUILD_DIR.mkdir(parents=True, exist_ok=True)
    if force and shared_object_path().exists():
        shared_object_path().unlink()
    os.environ.setdefault("MAX_JOBS", str(min(32, os.cpu_count() or 8)))
    module = cpp_extension.load(
        name=_EXT_NAME,
        sources=extension_sources(),
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=[
            "-O3",
            "-std=c++17",
            "-gencode",
            "arch=compute_100a,code=sm_100a",
            "-lineinfo",
            "--expt-relaxed-constexpr",
            "-Xptxas",
            "-v",
        ],
        build_directory=str(_BUILD_DIR),
        with_cuda=True,
        verbose=verbose,
    )
    return module


def _import_prebuilt():
    spec = importlib.util.spec_from_file_location(_EXT_NAME, shared_object_path())
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[_EXT_NAME] = module
    return module


def load_extension(build_if_missing: bool = True):
    """Return the extension module, importing the prebuilt object when it is up to date."""
    global _MODULE
    if _MODULE is not None:
        return _MODULE
    import torch  # noqa: F401  (libtorch symbols must be loaded before the extension)

    if not _is_stale():
        _MODULE = _import_prebuilt()
    elif build_if_missing:
        _MODULE = build_extension()
    else:
        raise ImportError(f"{shared_object_path()} is missing or older than its sources; run __graft_entry__.build()")
    return _MODULE


def is_extension_built() -> bool:
    return shared_object_path().exists()
