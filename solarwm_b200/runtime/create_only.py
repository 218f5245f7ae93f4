"""Create-only filesystem primitives: a published name is never replaced.

* ``rename_noreplace``: ``renameat2(RENAME_NOREPLACE)`` through libc (falls back to link+unlink for
  files when the syscall is unavailable).
* ``publish_directory_no_replace``: move a finished staging directory to its public name, under
  an flock on the parent so concurrent publishers are serialised; the loser gets
  ``FileExistsError`` and the winner's content is left untouched.
* ``write_file_create_only``: write to a temp name, fsync, commit with ``link(2)`` (which fails if
  the target exists), unlink the temp name.
* ``link_file_create_only``: publish an existing file under a second name with a hard link.

Reference: solar/runtime/create_only.py:18-172.
"""
from __future__ import annotations

import ctypes
import errno
import fcntl
import os
import uuid
from pathlib import Path

_RENAME_NOREPLACE = 1
_AT_FDCWD = -100
_libc = None


def _renameat2():
    global _libc
    if _libc is None:
        try:
            _libc = ctypes.CDLL(None, use_errno=True)
        except OSError:
            _libc = False
    if not _libc or not hasattr(_libc, "renameat2"):
        return None
    fn = _libc.renameat2
    fn.argtypes = [ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint]
    fn.restype = ctypes.c_int
    return fn


def rename_noreplace(src, dst) -> None:
    src, dst = os.fspath(src), os.fspath(dst)
    fn = _renameat2()
    if fn is not None:
        rc = fn(_AT_FDCWD, src.encode(), _AT_FDCWD, dst.encode(), _RENAME_NOREPLACE)
        if rc == 0:
            return
        err = ctypes.get_errno()
        if err == errno.EEXIST:
            raise FileExistsError(err, os.strerror(err), dst)
        if err not in (errno.ENOSYS, errno.EINVAL):
            raise OSError(err, os.strerror(err), dst)
    if os.path.isdir(src):
        if os.path.exists(dst):
            raise FileExistsError(errno.EEXIST, os.strerror(errno.EEXIST), dst)
        os.rename(src, dst)
        return
    os.link(src, dst)
    os.unlink(src)


def _fsync_dir(path: Path) -> None:
    fd = os.open(path, os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def publish_directory_no_replace(staging, target) -> Path:
    staging, target = Path(staging), Path(target)
    target.parent.mkdir(parents=True, exist_ok=True)
    lock = os.open(target.parent / ".publish.lock", os.O_CREAT | os.O_RDWR, 0o644)
    try:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if target.exists():
            raise FileExistsError(errno.EEXIST, "publication target already exists", str(target))
        rename_noreplace(staging, target)
        _fsync_dir(target.parent)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        os.close(lock)
    return target


def write_file_create_only(target, data: bytes) -> Path:
    target = Path(target)
    target.parent.mkdir(parents=True, exist_ok=True)
    tmp = target.with_name(f".{target.name}.{uuid.uuid4().hex}.tmp")
    try:
        with tmp.open("xb") as handle:
            handle.write(data)
            handle.flush()
            os.fsync(handle.fileno())
        os.link(tmp, target)          # fails with FileExistsError when the name is taken
        _fsync_dir(target.parent)
    finally:
        tmp.unlink(missing_ok=True)
    return target


def link_file_create_only(source, target) -> Path:
    target = Path(target)
    target.parent.mkdir(parents=True, exist_ok=True)
    os.link(source, target)
    _fsync_dir(target.parent)
    return target
