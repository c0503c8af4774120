"""File helpers with optional HDFS paths (reference: siirl/utils/extras/fs.py, hdfs_io.py).  ``hdfs://`` paths go
through the ``hdfs dfs`` command line when it is installed; everything else is the local file system."""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from typing import Optional

_HDFS_PREFIX = "hdfs://"


def is_non_local(path: str) -> bool:
    return str(path).startswith(_HDFS_PREFIX)


def _hdfs(*args: str) -> int:
    exe = shutil.which("hdfs")
    if exe is None:
        raise RuntimeError("an hdfs:// path was given but the 'hdfs' command is not installed")
    return subprocess.call([exe, "dfs", *args])


def exists(path: str) -> bool:
    return _hdfs("-test", "-e", path) == 0 if is_non_local(path) else os.path.exists(path)


def makedirs(path: str, exist_ok: bool = True) -> None:
    if is_non_local(path):
        _hdfs("-mkdir", "-p", path)
    else:
        os.makedirs(path, exist_ok=exist_ok)


def copy(src: str, dst: str) -> None:
    """Local<->local, local->hdfs or hdfs->local copy of a file or directory tree."""
    if is_non_local(src) and not is_non_local(dst):
        _hdfs("-get", "-f", src, dst)
    elif is_non_local(dst):
        _hdfs("-put", "-f", src, dst)
    elif os.path.isdir(src):
        shutil.copytree(src, dst, dirs_exist_ok=True)
    else:
        os.makedirs(os.path.dirname(os.path.abspath(dst)) or ".", exist_ok=True)
        shutil.copy2(src, dst)


def md5_encode(path: str) -> str:
    return hashlib.md5(path.encode()).hexdigest()


def get_local_temp_path(hdfs_path: str, cache_dir: str) -> str:
    return os.path.join(cache_dir, md5_encode(hdfs_path), os.path.basename(hdfs_path.rstrip("/")))


def copy_to_local(src: str, cache_dir: Optional[str] = None, always_recopy: bool = False) -> str:
    """Return a local path for ``src`` (downloads hdfs paths into ``cache_dir`` once)."""
    if not is_non_local(src):
        return src
    cache_dir = cache_dir or os.path.join(os.path.expanduser("~"), ".cache", "siirl_b200")
    local = get_local_temp_path(src, cache_dir)
    if always_recopy and os.path.exists(local):
        shutil.rmtree(local, ignore_errors=True) if os.path.isdir(local) else os.remove(local)
    if not os.path.exists(local):
        os.makedirs(os.path.dirname(local), exist_ok=True)
        copy(src, local)
    return local
