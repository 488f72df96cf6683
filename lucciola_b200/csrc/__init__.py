"""Build and load the kernel library.

The CUDA sources in this folder are compiled with nvcc for sm_100a into one
shared library with a C interface, loaded through ctypes.  No torch headers
are involved, so a cold build takes well under a minute per file and the files
are compiled in parallel.  The build happens at the first call of `library()`
when no library that matches the sources is found; it prints a line per file
and a heartbeat while nvcc runs.

Where the library goes: `<this folder>/_build/` when that is writable (so the
built file travels with the tree), else `$LUCCIOLA_B200_BUILD_DIR`, else a
per-user folder under the system's temporary directory.

There is no fallback: if the library cannot be built or loaded, `library()`
raises, and every operation of the engine raises with it.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_HERE = Path(__file__).resolve().parent
ABI_VERSION = 3
LIB_NAME = "liblucciola_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


class KernelLibraryError(RuntimeError):
    """The kernel library is missing, stale, or could not be built."""


def _say(msg: str) -> None:
    print(f"[lucciola_b200] {msg}", file=sys.stderr, flush=True)


def sources() -> list[Path]:
    return sorted(_HERE.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(_HERE.glob("*.cuh")) + list(_HERE.glob("*.h")))


def find_nvcc() -> str:
    cand = os.environ.get("LUCCIOLA_B200_NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").exists():
            return str(Path(root) / "bin" / "nvcc")
    raise KernelLibraryError("nvcc not found (set LUCCIOLA_B200_NVCC or CUDA_HOME); the kernel library cannot be built")


def _digest(paths: list[Path], extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def source_digest() -> str:
    return _digest(sources() + _headers(), " ".join(NVCC_FLAGS) + f"|abi{ABI_VERSION}")


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe-{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    cands = []
    if os.environ.get("LUCCIOLA_B200_BUILD_DIR"):
        cands.append(Path(os.environ["LUCCIOLA_B200_BUILD_DIR"]))
    cands.append(_HERE / "_build")
    cands.append(Path(tempfile.gettempdir()) / f"lucciola_b200-{os.getuid()}")
    for d in cands:
        if _writable(d):
            return d
    raise KernelLibraryError("no writable folder for the kernel library; tried " + ", ".join(map(str, cands)))


def _existing_library() -> Path | None:
    """A built library whose stamp matches the sources, wherever it may be."""
    want = source_digest()
    cands = []
    if os.environ.get("LUCCIOLA_B200_BUILD_DIR"):
        cands.append(Path(os.environ["LUCCIOLA_B200_BUILD_DIR"]))
    cands += [_HERE / "_build", Path(tempfile.gettempdir()) / f"lucciola_b200-{os.getuid()}"]
    for d in cands:
        lib, stamp = d / LIB_NAME, d / "stamp"
        try:
            if lib.exists() and stamp.read_text().strip() == want:
                return lib
        except OSError:
            continue
    return None


def _compile_one(nvcc: str, src: Path, obj: Path) -> tuple[Path, float]:
    t0 = time.time()
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(_HERE), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelLibraryError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    return src, time.time() - t0


def build(verbose: bool = True) -> Path:
    """Compile what changed and link the library.  Returns its path."""
    nvcc = find_nvcc()
    out = build_dir()
    want = source_digest()
    lib, stamp = out / LIB_NAME, out / "stamp"
    import fcntl

    with open(out / ".lock", "w") as lockf:
        fcntl.flock(lockf, fcntl.LOCK_EX)
        if lib.exists() and stamp.exists() and stamp.read_text().strip() == want:
            return lib
        hdr = _digest(_headers(), " ".join(NVCC_FLAGS))
        jobs, objs = [], []
        for src in sources():
            obj = out / f"{src.stem}-{_digest([src], hdr)}.o"
            objs.append(obj)
            if not obj.exists():
                jobs.append((src, obj))
        keep = {o.name for o in objs}
        for old in out.glob("*.o"):
            if old.name not in keep:
                old.unlink(missing_ok=True)
        if verbose and jobs:
            _say(f"building the kernel library for sm_100a in {out}: {len(jobs)} file(s) to compile")
        t0 = last_beat = time.time()
        done = 0
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4) or 1) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o.with_suffix(".o.tmp")) for s, o in jobs]
            pending = set(futs)
            while pending:
                finished = {f for f in pending if f.done()}
                for f in finished:
                    src, dt = f.result()
                    done += 1
                    if verbose:
                        _say(f"  compiled {src.name} in {dt:.1f} s ({done}/{len(jobs)})")
                pending -= finished
                if pending:
                    time.sleep(0.25)
                    if verbose and time.time() - last_beat > 10:
                        last_beat = time.time()
                        _say(f"  still compiling, {len(pending)} file(s) left, {last_beat - t0:.0f} s so far")
        for s, o in jobs:
            os.replace(o.with_suffix(".o.tmp"), o)
        tmp = out / (LIB_NAME + ".tmp")
        r = subprocess.run([nvcc, "-shared", "-o", str(tmp), *map(str, objs)], capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelLibraryError(f"linking the kernel library failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        stamp.write_text(want + "\n")
        if verbose:
            _say(f"kernel library ready: {lib} ({time.time() - t0:.1f} s)")
    return lib


def library() -> ctypes.CDLL:
    """The loaded kernel library; builds it first if needed.  Raises on failure."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _existing_library() or build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelLibraryError(f"cannot load {path}: {e}") from e
        lib.lb_abi_version.restype = ctypes.c_int
        if lib.lb_abi_version() != ABI_VERSION:
            raise KernelLibraryError(f"{path} has interface version {lib.lb_abi_version()}, expected {ABI_VERSION}")
        lib.lb_last_error.restype = ctypes.c_char_p
        _lib = lib
        return lib
