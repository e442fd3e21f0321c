"""In-tree build of the native library (``comprex_b200/lib/libcomprex_b200.so``).

The reference builds ``libPyGPI.so`` with CMake (CMakeLists.txt:8-70,
src/CMakeLists.txt:3-23) and loads it with ctypes; this build keeps the same
shape (one shared library with a flat C ABI) but compiles the CUDA sources for
sm_100a with nvcc directly, object by object and in parallel, and relinks only
when a source or header is newer than its object.

Run ``python -m comprex_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "build"
LIB = LIBDIR / "libcomprex_b200.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# -fmad=false: no multiply-add contraction, so that the kernels and the host
# implementation of the same primitive agree bit for bit (all of them are
# memory-bound; the extra instruction is free).
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-fmad=false", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-ffp-contract=off", "--threads", "2"] + ARCH
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, verbose: bool, ptxas_v: bool) -> Path:
    obj = OBJDIR / (src.name + ".o")
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [Path(__file__)]
    if not _stale(obj, [src] + headers):
        return obj
    if src.suffix == ".cu":
        extra = os.environ.get("COMPREX_NVCC_EXTRA", "").split()   # e.g. -DCX_COMPRESS_MIN_BLOCKS=3
        cmd = ([_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if ptxas_v else [])
               + ["-c", str(src), "-o", str(obj)])
    else:
        cmd = [os.environ.get("CXX", "g++")] + CXX_FLAGS + ["-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src.name} failed:\n{res.stdout}\n{res.stderr}")
    if ptxas_v and res.stderr:
        print(res.stderr, flush=True)
    return obj


def build(verbose: bool = False, force: bool = False, ptxas_v: bool = False) -> Path:
    """Compile every source under csrc/ for sm_100a and link the shared library."""
    LIBDIR.mkdir(exist_ok=True)
    OBJDIR.mkdir(exist_ok=True)
    if force:
        for f in OBJDIR.glob("*.o"):
            f.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, ptxas_v), srcs))
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ARCH + ["-lrt", "-lpthread"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"linking failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def build_selftest(sanitizer: str = "address,undefined", verbose: bool = False) -> Path:
    """Build the host back end together with its self-test under a sanitizer
    (``address,undefined`` or ``thread``); returns the executable."""
    OBJDIR.mkdir(exist_ok=True)
    exe = OBJDIR / ("host_selftest_" + sanitizer.replace(",", "_"))
    srcs = [CSRC / "selftest" / "host_selftest.cpp", CSRC / "host_ref.cpp"]
    if not _stale(exe, srcs + list(CSRC.glob("*.h")) + [Path(__file__)]):
        return exe
    # not every g++ ships the sanitizer runtimes: take the first one that links
    tried = []
    for cxx in dict.fromkeys([os.environ.get("CXX") or "g++", "/usr/bin/g++", "g++", "clang++"]):
        if not shutil.which(cxx):
            continue
        cmd = ([cxx, "-O1", "-g", "-std=c++17", "-ffp-contract=off", "-Wall", "-fno-omit-frame-pointer",
                f"-fsanitize={sanitizer}", "-fno-sanitize-recover=all"]
               + [str(x) for x in srcs] + ["-o", str(exe), "-lpthread", "-lrt"])
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode == 0:
            return exe
        tried.append(f"{cxx}:\n{res.stdout}\n{res.stderr}")
    raise RuntimeError("building the self-test failed:\n" + "\n".join(tried))


if __name__ == "__main__":
    if "--selftest" in sys.argv:
        for san, args in (("address,undefined", []), ("thread", ["--protocol"])):
            exe = build_selftest(san, verbose=True)
            print(exe, flush=True)
            sys.exit_code = subprocess.run([str(exe)] + args).returncode
            if sys.exit_code:
                sys.exit(sys.exit_code)
        sys.exit(0)
    path = build(verbose=True, force="--force" in sys.argv, ptxas_v="--ptxas" in sys.argv)
    print(path)
