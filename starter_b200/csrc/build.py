"""Compiles the CUDA sources of this folder for sm_100a into one shared library.

The library is built on first use (or by ``__graft_entry__.build``) with nvcc,
one object per source in parallel, into ``_build/`` beside the sources, or into
a per-user folder under the system's temporary directory when the source tree
cannot be written.  A stamp per object records the hash of the source, of the
headers and of the flags, so an object is rebuilt only when one of them changed.
While it compiles it prints a line per finished object and one every few
seconds in between.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_NAME = "libstarter_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


class BuildError(RuntimeError):
    """The CUDA extension could not be built or loaded; nothing falls back to another path."""


def sources():
    return sorted(p for p in HERE.glob("*.cu"))


def headers():
    return sorted(list(HERE.glob("*.cuh")) + list(HERE.glob("*.h")))


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    which = shutil.which("nvcc")
    if which:
        candidates.append(Path(which))
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for c in candidates:
        if c.is_file() and os.access(c, os.X_OK):
            return str(c)
    raise BuildError("nvcc was not found (looked in $CUDA_HOME/bin, $PATH and /usr/local/cuda/bin); "
                     "the kernels of this library are compiled from source")


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}"
        probe.write_text("ok")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("STARTER_B200_BUILD_DIR")
    if override:
        folder = Path(override)
        if not _writable(folder):
            raise BuildError(f"STARTER_B200_BUILD_DIR={override} cannot be written")
        return folder
    in_tree = HERE / "_build"
    if _writable(in_tree):
        return in_tree
    fallback = Path(tempfile.gettempdir()) / f"starter_b200_build_{os.getuid()}"
    if _writable(fallback):
        return fallback
    raise BuildError(f"neither {in_tree} nor {fallback} can be written; set STARTER_B200_BUILD_DIR")


def _digest(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[starter_b200 build] {msg}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path, extra_flags) -> float:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *extra_flags, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{' '.join(cmd)}\n{proc.stdout}")
    if proc.stdout.strip() and "-Xptxas" in " ".join(extra_flags):
        print(proc.stdout, file=sys.stderr)
    return time.time() - t0


def build(verbose: bool = True, force: bool = False, extra_flags=()) -> Path:
    """Compile what is out of date and link the library; returns its path.  STARTER_B200_NVCC_FLAGS in the
    environment adds flags (for experiments: a changed flag rebuilds everything)."""
    extra_flags = tuple(extra_flags) + tuple(os.environ.get("STARTER_B200_NVCC_FLAGS", "").split())
    folder = build_dir()
    lib = folder / LIB_NAME
    hdr_digest = _digest(headers(), " ".join([*ARCH_FLAGS, *NVCC_FLAGS, *extra_flags]))
    with open(folder / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        todo, objects = [], []
        for src in sources():
            obj = folder / (src.stem + ".o")
            stamp = folder / (src.stem + ".stamp")
            want = _digest([src], hdr_digest)
            objects.append(obj)
            if force or not obj.is_file() or not stamp.is_file() or stamp.read_text() != want:
                todo.append((src, obj, stamp, want))
        if not todo and lib.is_file():
            return lib
        nvcc = find_nvcc()
        if todo:
            _say(f"compiling {len(todo)} CUDA source(s) for sm_100a into {folder} (first use, or sources changed)", verbose)
            t0 = time.time()
            stop = threading.Event()

            def heartbeat():
                while not stop.wait(10.0):
                    _say(f"still compiling ... {time.time() - t0:.0f} s", verbose)

            beat = threading.Thread(target=heartbeat, daemon=True)
            beat.start()
            try:
                with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as pool:
                    futures = {pool.submit(_compile_one, nvcc, src, obj, list(extra_flags)): (src, stamp, want)
                               for src, obj, stamp, want in todo}
                    done = 0
                    for fut in as_completed(futures):
                        src, stamp, want = futures[fut]
                        seconds = fut.result()
                        stamp.write_text(want)
                        done += 1
                        _say(f"  {src.name} done in {seconds:.1f} s ({done}/{len(todo)})", verbose)
            finally:
                stop.set()
        tmp = folder / (LIB_NAME + f".{os.getpid()}.tmp")
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objects]]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking failed:\n{' '.join(cmd)}\n{proc.stdout}")
        os.replace(tmp, lib)
        _say(f"linked {lib.name}", verbose)
    return lib


_LIB = None


def load(verbose: bool = True) -> ctypes.CDLL:
    """The compiled library, built first if needed.  Raises BuildError; never substitutes anything."""
    global _LIB
    if _LIB is None:
        path = build(verbose=verbose)
        try:
            _LIB = ctypes.CDLL(str(path))
        except OSError as exc:
            raise BuildError(f"{path} could not be loaded: {exc}") from None
    return _LIB


def register_report(names=()) -> int:
    """Registers and spills of every kernel, as ptxas reports them (``python -m starter_b200.csrc.build [file.cu ...]``).
    The decode product sits exactly at the register count that four 8-warp blocks per SM allow: read this after
    every change to it."""
    import re
    nvcc = find_nvcc()
    worst = 0
    for src in sources():
        if names and src.name not in names:
            continue
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-Xptxas", "-v", "-I", str(HERE), "-c", str(src), "-o", os.devnull]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}")
        kernel, spills = None, (0, 0)
        for line in proc.stdout.splitlines():
            m = re.search(r"Compiling entry function '(\S+)'", line)
            if m:
                kernel = subprocess.run(["c++filt", m.group(1)], stdout=subprocess.PIPE, text=True).stdout.strip() or m.group(1)
                kernel = kernel.split("(")[0]
            m = re.search(r"(\d+) bytes spill stores, (\d+) bytes spill loads", line)
            if m:
                spills = (int(m.group(1)), int(m.group(2)))
            m = re.search(r"Used (\d+) registers", line)
            if m and kernel:
                print(f"{src.name:26s} {kernel[:78]:78s} {int(m.group(1)):4d} registers  spill {spills[0]}/{spills[1]} bytes")
                worst = max(worst, spills[0], spills[1])
    return worst


if __name__ == "__main__":
    register_report(tuple(sys.argv[1:]))
