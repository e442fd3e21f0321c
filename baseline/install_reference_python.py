"""Put a runnable copy of the reference's Python package under baseline/_ref (git-ignored).

`pip install <reference>` cannot work: the tree has no setup.py / pyproject.toml and its library
needs GPI-2 and GaspiCxx.  This script does what the reference's CMake build does for Python users
(src/CMakeLists.txt:3-23): it compiles the C shims src/*_C.cpp into lib/libPyGPI.so - against the
shared-memory GaspiCxx stand-in of baseline/gaspicxx_shim instead of GaspiCxx - next to an
unmodified copy of the reference's Python modules.  The TensorFlow ops and the Keras optimizer are
copied too but stay unusable without TensorFlow.

    python baseline/install_reference_python.py --reference <root of the Comprex tree>
    python baseline/install_reference_python.py --reference <...> --run test/BigRingAllreduce.py --ranks 2
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys
import uuid

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref", "Comprex")


def install(reference: str) -> str:
    os.makedirs(os.path.join(DEST, "lib"), exist_ok=True)
    for rel in ("__init__.py", "common.py", "gpi.py", "GaspiEx.py", "ComprEx.py", "allreduce.py", "allreduceOp.py"):
        shutil.copy(os.path.join(reference, rel), os.path.join(DEST, rel))
    for sub in ("keras", "test", "examples"):
        dst = os.path.join(DEST, sub)
        os.makedirs(dst, exist_ok=True)
        for f in glob.glob(os.path.join(reference, sub, "*.py")):
            shutil.copy(f, dst)
    cmd = [os.environ.get("CXX", "g++"), "-O3", "-march=native", "-std=c++14", "-fpermissive", "-w", "-fPIC", "-shared",
           "-I", os.path.join(HERE, "gaspicxx_shim", "include"), "-I", os.path.join(reference, "include"),
           "-I", os.path.join(reference, "src")]
    cmd += [os.path.join(reference, "src", f) for f in ("comprEx_C.cpp", "GPI_C.cpp", "gaspiEx_C.cpp", "allreduce_C.cpp")]
    cmd += ["-o", os.path.join(DEST, "lib", "libPyGPI.so"), "-lrt", "-lpthread"]
    subprocess.run(cmd, check=True)
    return DEST


def run(script: str, ranks: int, timeout: int = 900) -> int:
    """Run one of the installed package's scripts as `ranks` processes (what gaspi_run does)."""
    job = uuid.uuid4().hex[:10]
    with open(f"/dev/shm/cxshim_{job}_ctl", "wb") as f:
        f.truncate(2 << 20)
    path = os.path.join(DEST, script)
    procs, rc = [], 0
    try:
        for r in range(ranks):
            env = dict(os.environ, CXSHIM_RANK=str(r), CXSHIM_SIZE=str(ranks), CXSHIM_JOB=job)
            procs.append(subprocess.Popen([sys.executable, path], env=env, cwd=os.path.dirname(path),
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        for r, p in enumerate(procs):
            out, _ = p.communicate(timeout=timeout)
            rc |= p.returncode
            print(f"--- rank {r} (exit {p.returncode}) ---\n{out[-1500:]}", flush=True)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        for shm in glob.glob(f"/dev/shm/cxshim_{job}_*"):
            os.unlink(shm)
    return rc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--run", default=None, help="script of the package to run afterwards, e.g. test/BigRingAllreduce.py")
    ap.add_argument("--ranks", type=int, default=2)
    args = ap.parse_args()
    print("installed to", install(args.reference), flush=True)
    if args.run:
        sys.exit(run(args.run, args.ranks))


if __name__ == "__main__":
    main()
