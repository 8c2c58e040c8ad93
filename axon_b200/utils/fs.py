"""File-system helpers (reference: axon/utils/fs.py)."""
from __future__ import annotations

import os
import shutil


def local_mkdir_safe(path: str) -> str:
    """``mkdir -p`` that tolerates concurrent creators; returns the absolute path."""
    path = os.path.abspath(path)
    os.makedirs(path, exist_ok=True)
    return path


def copy_to_local(src: str, cache_dir: str | None = None) -> str:
    """Local paths are returned unchanged; with ``cache_dir`` a directory is mirrored there once."""
    if cache_dir is None or not os.path.exists(src):
        return src
    dst = os.path.join(local_mkdir_safe(cache_dir), os.path.basename(os.path.normpath(src)))
    if not os.path.exists(dst):
        (shutil.copytree if os.path.isdir(src) else shutil.copy2)(src, dst)
    return dst
