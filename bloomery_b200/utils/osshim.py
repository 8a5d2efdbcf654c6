"""The one owner of the operating-system calls the host side makes: CPU masks and pinning, page size and host memory,
free bytes of a directory, page-cache residency of a mapped file (``mincore``), advice on mappings (``madvise``) and on
files (``posix_fadvise``), page locking, ``O_DIRECT`` opens, a rename that never replaces, peak resident size.

Every call has its Linux body; on another platform a call that has no counterpart raises :class:`Unsupported` by name, so
a caller handles the refusal as it handles the kernel's own error (:class:`OsError` carries ``errno``).  Counterpart of
the reference's ``crates/os/src/lib.rs`` (``mask_cpus``, ``set_mask``, ``pin``, ``free_bytes``, ``host_memory``,
``page_bytes``, ``open_direct``, ``rename_noreplace``, ``fadvise_dontneed``, ``max_rss_bytes``, ``Populated``).
"""
from __future__ import annotations

import ctypes
import ctypes.util
import dataclasses
import errno
import mmap
import os
import resource
import sys
from typing import List, Optional, Sequence

LINUX = sys.platform.startswith("linux")


class OsError(OSError):
    """The kernel refused the call ``what``."""

    def __init__(self, what: str, err: int):
        super().__init__(err, f"{what}: {os.strerror(err)}")
        self.what = what


class Unsupported(OsError):
    """This platform has no such call."""

    def __init__(self, what: str):
        OSError.__init__(self, errno.ENOSYS, f"{what}: not on {sys.platform}")
        self.what = what


_libc = None


def _c():
    global _libc
    if _libc is None:
        _libc = ctypes.CDLL(ctypes.util.find_library("c") or "libc.so.6", use_errno=True)
    return _libc


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise OsError(what, ctypes.get_errno() or errno.EIO)


# ---------------------------------------------------------------------------------------------------------- CPUs
def mask_cpus() -> List[int]:
    """The CPUs this thread may run on (a container's cpuset shows here, not in ``os.cpu_count``)."""
    if hasattr(os, "sched_getaffinity"):
        return sorted(os.sched_getaffinity(0))
    return list(range(os.cpu_count() or 1))


def set_mask(cpus: Sequence[int]) -> None:
    if not hasattr(os, "sched_setaffinity"):
        raise Unsupported("sched_setaffinity")
    if not cpus:
        raise OsError("sched_setaffinity", errno.EINVAL)
    try:
        os.sched_setaffinity(0, set(int(c) for c in cpus))
    except OSError as exc:
        raise OsError("sched_setaffinity", exc.errno or errno.EINVAL) from None


def pin(cpu: int) -> None:
    """Bind the calling thread to one CPU."""
    set_mask([cpu])


# -------------------------------------------------------------------------------------------------------- memory
def page_bytes() -> int:
    return mmap.PAGESIZE


@dataclasses.dataclass(frozen=True)
class HostMemory:
    total: int
    available: int          # what a new allocation can take without swapping (MemAvailable)
    locked_limit: int       # RLIMIT_MEMLOCK of this process; -1 = unlimited


def host_memory(meminfo: str = "/proc/meminfo") -> HostMemory:
    total = avail = None
    try:
        with open(meminfo) as fh:
            for line in fh:
                key, _, rest = line.partition(":")
                if key in ("MemTotal", "MemAvailable"):
                    kb = int(rest.split()[0])
                    if key == "MemTotal":
                        total = kb << 10
                    else:
                        avail = kb << 10
    except OSError:
        pass
    if total is None:
        try:
            total = os.sysconf("SC_PHYS_PAGES") * os.sysconf("SC_PAGE_SIZE")
        except (ValueError, OSError, AttributeError):
            raise Unsupported("host_memory") from None
    if avail is None:
        try:
            avail = os.sysconf("SC_AVPHYS_PAGES") * os.sysconf("SC_PAGE_SIZE")
        except (ValueError, OSError, AttributeError):
            avail = total
    soft, _ = resource.getrlimit(resource.RLIMIT_MEMLOCK)
    return HostMemory(total, avail, -1 if soft == resource.RLIM_INFINITY else int(soft))


def max_rss_bytes(children: bool = False) -> int:
    """Peak resident size of this process (or of its waited-for children)."""
    ru = resource.getrusage(resource.RUSAGE_CHILDREN if children else resource.RUSAGE_SELF)
    return int(ru.ru_maxrss) * (1 if sys.platform == "darwin" else 1024)


def free_bytes(directory: str) -> int:
    """Bytes an unprivileged writer can still put under ``directory``."""
    try:
        st = os.statvfs(directory)
    except OSError as exc:
        raise OsError("statvfs", exc.errno or errno.EIO) from None
    return int(st.f_bavail) * int(st.f_frsize)


def _addr(m: mmap.mmap) -> int:
    """Address of a mapping (read-only ones included)."""
    import numpy as np
    return int(np.frombuffer(m, dtype=np.uint8).ctypes.data) if len(m) else 0


@dataclasses.dataclass(frozen=True)
class Populated:
    pages: int
    resident: int

    @property
    def fraction(self) -> float:
        return self.resident / self.pages if self.pages else 1.0


def populated(m: mmap.mmap, offset: int = 0, length: Optional[int] = None) -> Populated:
    """How much of a mapped file already sits in memory (``mincore``): a cold multi-GB model file reads at the drive's
    rate, a warm one at memory's, and the load record says which it was."""
    if not LINUX and sys.platform != "darwin":
        raise Unsupported("mincore")
    size = len(m)
    length = size - offset if length is None else length
    if offset < 0 or length < 0 or offset + length > size or offset % page_bytes():
        raise OsError("mincore", errno.EINVAL)
    if length == 0:
        return Populated(0, 0)
    pages = (length + page_bytes() - 1) // page_bytes()
    vec = (ctypes.c_ubyte * pages)()
    _check(_c().mincore(ctypes.c_void_p(_addr(m) + offset), ctypes.c_size_t(length), vec), "mincore")
    return Populated(pages, sum(v & 1 for v in vec))


ADVICE = {"normal": 0, "random": 1, "sequential": 2, "willneed": 3, "dontneed": 4, "hugepage": 14}


def advise(m: mmap.mmap, advice: str, offset: int = 0, length: Optional[int] = None) -> None:
    """``madvise`` on a mapping: ``sequential`` + ``willneed`` ahead of a whole-file upload, ``random`` for row tables
    read by hash, ``dontneed`` behind an upload, ``hugepage`` for big anonymous arenas."""
    if advice not in ADVICE:
        raise OsError(f"madvise {advice}", errno.EINVAL)
    if advice == "hugepage" and not LINUX:
        raise Unsupported("madvise hugepage")
    size = len(m)
    length = size - offset if length is None else length
    if offset < 0 or length < 0 or offset + length > size or offset % page_bytes():
        raise OsError("madvise", errno.EINVAL)
    if length == 0:
        return
    if hasattr(m, "madvise") and advice != "hugepage":
        try:
            m.madvise(ADVICE[advice], offset, length)
            return
        except OSError as exc:
            raise OsError(f"madvise {advice}", exc.errno or errno.EINVAL) from None
    _check(_c().madvise(ctypes.c_void_p(_addr(m) + offset), ctypes.c_size_t(length), ctypes.c_int(ADVICE[advice])), f"madvise {advice}")


def lock_pages(m: mmap.mmap, offset: int = 0, length: Optional[int] = None) -> None:
    """``mlock`` a span (refused with ENOMEM past RLIMIT_MEMLOCK: the caller names the limit from ``host_memory``)."""
    length = len(m) - offset if length is None else length
    if length:
        _check(_c().mlock(ctypes.c_void_p(_addr(m) + offset), ctypes.c_size_t(length)), "mlock")


def unlock_pages(m: mmap.mmap, offset: int = 0, length: Optional[int] = None) -> None:
    length = len(m) - offset if length is None else length
    if length:
        _check(_c().munlock(ctypes.c_void_p(_addr(m) + offset), ctypes.c_size_t(length)), "munlock")


# --------------------------------------------------------------------------------------------------------- files
def fadvise_dontneed(fd: int, offset: int = 0, length: int = 0) -> None:
    """Drop a file span from the page cache once its bytes are on the card (length 0 = to the end)."""
    if not hasattr(os, "posix_fadvise"):
        raise Unsupported("posix_fadvise")
    try:
        os.posix_fadvise(fd, offset, length, os.POSIX_FADV_DONTNEED)
    except OSError as exc:
        raise OsError("posix_fadvise", exc.errno or errno.EIO) from None


def open_direct(path: str) -> int:
    """A read-only descriptor that bypasses the page cache (expert side files read at the drive's own rate)."""
    if not hasattr(os, "O_DIRECT"):
        raise Unsupported("O_DIRECT")
    try:
        return os.open(path, os.O_RDONLY | os.O_DIRECT)
    except OSError as exc:
        raise OsError("open O_DIRECT", exc.errno or errno.EIO) from None


RENAME_NOREPLACE = 1


def rename_noreplace(src: str, dst: str) -> None:
    """Move ``src`` to ``dst`` unless ``dst`` exists (EEXIST then): two writers of one cache entry never overwrite
    each other."""
    if LINUX and hasattr(_c(), "renameat2"):
        at_fdcwd = -100
        rc = _c().renameat2(ctypes.c_int(at_fdcwd), os.fsencode(src), ctypes.c_int(at_fdcwd), os.fsencode(dst),
                            ctypes.c_uint(RENAME_NOREPLACE))
        if rc == 0:
            return
        err = ctypes.get_errno()
        if err not in (errno.ENOSYS, errno.EINVAL):
            raise OsError("renameat2", err)
    # a file system without the flag: link + unlink gives the same "never replaces"
    try:
        os.link(src, dst)
    except OSError as exc:
        raise OsError("link", exc.errno or errno.EIO) from None
    os.unlink(src)
