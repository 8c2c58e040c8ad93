"""Build and load the sm_100a native library (``axon_b200/_C.so``).

The library is plain CUDA C++ behind ``extern "C"`` launchers; Python talks to it through
``ctypes`` with raw device pointers and the current CUDA stream, so it has no dependency on
the PyTorch C++ ABI and a source file rebuilds in seconds.

``build()`` cross-compiles every ``csrc/*.cu`` for ``sm_100a`` only (no GPU needed) and links
one shared object next to this file. ``lib()`` loads it; on a machine with a GPU a missing
library is an error, never a silent fallback.

A second flavour, ``axon_b200/_C_debug.so``, is the same sources compiled with ``-DAXB_DEBUG``: kernels that
take indices from data (token ids, page tables, replayed expert ids, sync-plan ranks) record the first index
that falls outside its buffer (``csrc/debug.cuh``) in addition to skipping it. ``AXON_NATIVE_DEBUG=1`` makes
``lib()`` load that flavour; ``ops._common.check_status`` then also reports such records.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_ROOT = _PKG.parent
_CSRC = _ROOT / "csrc"
_BUILD = _ROOT / "build"
_SO = _PKG / "_C.so"
_SO_DEBUG = _PKG / "_C_debug.so"
_BUILD_DEBUG = _ROOT / "build" / "debug"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]

_lib = None


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _sources() -> list[Path]:
    return sorted(_CSRC.glob("*.cu"))


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def debug_requested() -> bool:
    return os.environ.get("AXON_NATIVE_DEBUG", "0") not in ("", "0", "false", "False")


def needs_build(debug: bool = False) -> bool:
    so, bdir = (_SO_DEBUG, _BUILD_DEBUG) if debug else (_SO, _BUILD)
    stamp = bdir / "stamp.txt"
    if not so.exists() or not stamp.exists():
        return True
    deps = list(_CSRC.glob("*.cu")) + list(_CSRC.glob("*.cuh")) + list(_CSRC.glob("*.h"))
    return stamp.read_text().strip() != _digest(deps)


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> Path:
    """Compile csrc/*.cu for sm_100a and link axon_b200/_C.so (``debug``: _C_debug.so with -DAXB_DEBUG).
    Returns the library path."""
    global _SO, _BUILD
    if debug:
        # same code path with the debug names and the extra define
        saved = (_SO, _BUILD, list(NVCC_FLAGS))
        _SO, _BUILD = _SO_DEBUG, _BUILD_DEBUG
        NVCC_FLAGS.append("-DAXB_DEBUG")
        try:
            _BUILD.parent.mkdir(exist_ok=True)
            return _build_impl(force, verbose, debug=True)
        finally:
            _SO, _BUILD = saved[0], saved[1]
            NVCC_FLAGS[:] = saved[2]
    return _build_impl(force, verbose, debug=False)


def _build_impl(force: bool, verbose: bool, debug: bool) -> Path:
    if not force and not needs_build(debug):
        return _SO
    _BUILD.mkdir(exist_ok=True)
    nvcc = _nvcc()
    headers = list(_CSRC.glob("*.cuh")) + list(_CSRC.glob("*.h"))
    hdig = _digest(headers)

    def compile_one(src: Path) -> Path:
        obj = _BUILD / (src.stem + ".o")
        tag = _BUILD / (src.stem + ".tag")
        want = _digest([src]) + hdig
        if not force and obj.exists() and tag.exists() and tag.read_text() == want:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(_CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (_BUILD / (src.stem + ".log")).write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-4000:]}")
        if verbose:
            sys.stderr.write(r.stderr)
        tag.write_text(want)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(_SO),
           *map(str, objs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    deps = list(_CSRC.glob("*.cu")) + headers
    (_BUILD / "stamp.txt").write_text(_digest(deps))
    return _SO


def available() -> bool:
    return _SO.exists()


def lib() -> ctypes.CDLL:
    """Load the native library (building it first if the sources are newer and nvcc exists)."""
    global _lib
    if _lib is not None:
        return _lib
    debug = debug_requested()
    so = _SO_DEBUG if debug else _SO
    if not so.exists():
        try:
            build(debug=debug)
        except Exception as e:  # noqa: BLE001
            raise RuntimeError(
                "axon_b200 native library is missing and could not be built; run "
                "`python -c 'import __graft_entry__ as g; g.build()'`"
            ) from e
    _lib = ctypes.CDLL(str(so))
    return _lib
