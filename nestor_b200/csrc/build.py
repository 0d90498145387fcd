"""Build the sm_100a kernel library in-tree: ``nestor_b200/_C/libnestor_b200.so``.

``python -m nestor_b200.csrc.build`` compiles every ``.cu`` file of this directory with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into one shared library with a C ABI
(no PyTorch headers; the Python side passes raw device pointers and the current stream
through ``ctypes``). Objects are cached by source hash, so a rebuild only recompiles
what changed. The library never links ``libcuda``: the one driver entry point it needs
(tensor-map encoding) is resolved at run time through the CUDA runtime.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

SRC = Path(__file__).resolve().parent
OUT = SRC.parent / "_C"
LIB = OUT / "libnestor_b200.so"
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def nvcc() -> str | None:
    return shutil.which("nvcc") or (str(p) if (p := Path("/usr/local/cuda/bin/nvcc")).is_file() else None)


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    for f in [path, *sorted(SRC.glob("*.cuh")), *sorted(SRC.glob("*.h"))]:
        h.update(f.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()[:16]


CHECKED_LIB = OUT / "libnestor_b200_checked.so"      # the same sources with -DNESTOR_BOUNDS_CHECK


def build(verbose: bool = False, force: bool = False, checked: bool = False) -> Path:
    """Build the library (``checked``: the index-checking variant, objects cached under their own names).

    Several processes may get here at once (every rank of a multi-GPU launch checks the library when it loads it):
    the whole build runs under an exclusive file lock, so one of them compiles and the others find the objects of
    the current digests when their turn comes; objects and the library are written under temporary names and renamed.
    """

    import fcntl

    OUT.mkdir(exist_ok=True)
    with open(OUT / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(verbose, force, checked)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose: bool, force: bool, checked: bool) -> Path:
    cc = nvcc()
    if cc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernel library")
    objs, rebuilt = [], False
    extra = ["-DNESTOR_BOUNDS_CHECK"] if checked else []
    kind = "chk" if checked else ""
    for cu in sorted(SRC.glob("*.cu")):
        obj = OUT / f"{cu.stem}{kind}.{_digest(cu)}.o"
        if force or not obj.is_file():
            for old in OUT.glob(f"{cu.stem}{kind}.*.o"):
                old.unlink(missing_ok=True)
            tmp = obj.with_suffix(f".{os.getpid()}.tmp")
            cmd = [cc, *FLAGS, *extra, "-c", str(cu), "-o", str(tmp)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode:
                tmp.unlink(missing_ok=True)
                raise RuntimeError(f"nvcc failed on {cu.name}")
            tmp.replace(obj)
            if not checked:
                (OUT / f"{cu.stem}.ptxas.txt").write_text(res.stderr)
            rebuilt = True
        objs.append(obj)
    lib = CHECKED_LIB if checked else LIB
    if rebuilt or not lib.is_file():
        tmp = lib.with_suffix(f".{os.getpid()}.tmp")
        cmd = [cc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            tmp.unlink(missing_ok=True)
            raise RuntimeError("link failed")
        tmp.replace(lib)
    return lib


def stale_sources(checked: bool = False) -> list[str]:
    """Sources whose cached object (named by source digest) is missing: the built library predates them."""

    kind = "chk" if checked else ""
    return [cu.name for cu in sorted(SRC.glob("*.cu")) if not (OUT / f"{cu.stem}{kind}.{_digest(cu)}.o").is_file()]


def ensure(checked: bool = False) -> Path:
    """The up-to-date library: rebuild what changed when a compiler is present, else refuse a stale binary.

    A library older than its sources would be called with argument structures it does not know (the Python
    side mirrors the C structs), so loading it is never safe.
    """

    if nvcc() is not None:
        return build(checked=checked)
    lib = CHECKED_LIB if checked else LIB
    stale = stale_sources(checked)
    if stale or not lib.is_file():
        raise RuntimeError(
            f"{lib} is missing or older than {', '.join(stale) or 'its sources'} and there is no nvcc to rebuild it")
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, checked="--checked" in sys.argv))
