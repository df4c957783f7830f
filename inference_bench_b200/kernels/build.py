"""Builds the CUDA kernel library for sm_100a with nvcc, in-tree, on first use.

Every `csrc/*.cu` becomes an object file and all of them are linked into one shared library that
`kernels/lib.py` loads with ctypes. Nothing here needs a GPU (nvcc cross-compiles) or the torch
C++ headers, so a fresh checkout compiles in well under a minute. Objects are keyed by a hash of
their source, the headers and the flags; a second call does nothing.

The reference compiles its kernels at load time too (NVRTC, crates/specrt/src/jit.rs:44-85); here
the compiler is nvcc and the cache is a folder beside the sources.
"""
from __future__ import annotations

import fcntl
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
LIB_NAME = "libib200_kernels.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inference_bench_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and (Path(cand) / "bin" / "nvcc").is_file():
            return str(Path(cand) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); the CUDA kernels cannot be built")


def _writable_dir(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    """In-tree `_build/` when the checkout is writable, else a per-user cache, else a temp folder."""
    cands = []
    if os.environ.get("IB200_BUILD_DIR"):
        cands.append(Path(os.environ["IB200_BUILD_DIR"]))
    cands.append(CSRC.parent / "_build")
    home = os.environ.get("HOME")
    if home:
        cands.append(Path(home) / ".cache" / "inference_bench_b200")
    cands.append(Path(tempfile.gettempdir()) / f"inference_bench_b200-{os.getuid()}")
    for c in cands:
        if _writable_dir(c):
            return c
    raise BuildError("no writable folder for the kernel build: tried " + ", ".join(map(str, cands)))


def _digest(parts: list[bytes]) -> str:
    h = hashlib.sha256()
    for p in parts:
        h.update(p)
        h.update(b"\0")
    return h.hexdigest()[:16]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(verbose: bool = True) -> Path:
    """Compile what changed and return the path of the shared library."""
    srcs = sources()
    if not srcs:
        raise BuildError(f"no CUDA sources under {CSRC}")
    out = build_dir()
    headers = b"".join(p.read_bytes() for p in sorted([*CSRC.glob("*.cuh"), *CSRC.glob("*.h")]))
    flags = " ".join(NVCC_FLAGS).encode()
    keys = {s: _digest([s.read_bytes(), headers, flags]) for s in srcs}
    lib_key = _digest([k.encode() for k in keys.values()])
    lib = out / f"{lib_key}-{LIB_NAME}"
    if lib.is_file():
        return lib
    nvcc = find_nvcc()
    with open(out / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if lib.is_file():
                return lib
            todo = [(s, out / f"{s.stem}-{keys[s]}.o") for s in srcs]
            missing = [(s, o) for s, o in todo if not o.is_file()]
            t0 = time.time()
            if verbose and missing:
                _say(f"compiling {len(missing)} CUDA source file(s) for sm_100a into {out} (first call only)")
            done = threading.Event()

            def ticker():
                while not done.wait(10.0):
                    _say(f"still compiling ... {time.time() - t0:.0f} s")

            tick = threading.Thread(target=ticker, daemon=True)
            if verbose and missing:
                tick.start()

            def compile_one(job):
                src, obj = job
                tmp = obj.with_suffix(f".tmp{os.getpid()}.o")
                cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(tmp)]
                r = subprocess.run(cmd, capture_output=True, text=True)
                if r.returncode != 0:
                    raise BuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
                os.replace(tmp, obj)
                if verbose:
                    _say(f"compiled {src.name} ({time.time() - t0:.0f} s)")

            try:
                with ThreadPoolExecutor(max_workers=min(8, max(1, len(missing)))) as pool:
                    list(pool.map(compile_one, missing))
            finally:
                done.set()
            tmp_lib = lib.with_suffix(f".tmp{os.getpid()}.so")
            cmd = [nvcc, "-shared", "-o", str(tmp_lib), *[str(o) for _, o in todo], "-Xcompiler", "-fPIC", "-cudart", "static"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp_lib, lib)
            if verbose:
                _say(f"built {lib.name} in {time.time() - t0:.0f} s")
            # Drop this library's files of older source versions (the host library's are its own business).
            keep = {lib.name, *[o.name for _, o in todo]}
            stems = {s.stem for s in srcs}
            for f in out.iterdir():
                mine = f.name.endswith("-" + LIB_NAME) or (f.suffix == ".o" and f.name.rsplit("-", 1)[0] in stems)
                if mine and f.name not in keep and ".tmp" not in f.name:
                    try:
                        f.unlink()
                    except OSError:
                        pass
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


HOST_LIB_NAME = "libib200_host.so"
HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-Wall"]


def build_host(verbose: bool = True) -> Path:
    """The host-side library (`csrc/host/*.cpp`: cache bookkeeping and scheduling decisions), built with
    the C++ compiler alone: it needs neither nvcc nor a GPU."""
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        raise BuildError(f"no C++ sources under {CSRC / 'host'}")
    out = build_dir()
    key = _digest([*(s.read_bytes() for s in srcs), " ".join(HOST_FLAGS).encode()])
    lib = out / f"{key}-{HOST_LIB_NAME}"
    if lib.is_file():
        return lib
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++") or shutil.which("clang++")
    if not cxx:
        raise BuildError("no C++ compiler was found (g++, c++, clang++ or $CXX); the host library cannot be built")
    with open(out / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if lib.is_file():
                return lib
            t0 = time.time()
            tmp_lib = lib.with_suffix(f".tmp{os.getpid()}.so")
            r = subprocess.run([cxx, *HOST_FLAGS, "-o", str(tmp_lib), *map(str, srcs)], capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"compiling {HOST_LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp_lib, lib)
            if verbose:
                _say(f"built {lib.name} in {time.time() - t0:.0f} s")
            for f in out.iterdir():
                if f.name.endswith("-" + HOST_LIB_NAME) and f.name != lib.name and ".tmp" not in f.name:
                    try:
                        f.unlink()
                    except OSError:
                        pass
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


if __name__ == "__main__":
    print(build_host())
    print(build())
