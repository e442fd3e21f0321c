"""Build and run the reference's own allreduce benchmark (examples/allreduce_speed.cpp) against
the GaspiCxx stand-in of baseline/gaspicxx_shim: the reference's sources are compiled unmodified,
its ranks run as processes on this host, and GPI-2's write + notify is a memcpy into the peer's
shared-memory segment plus an atomic counter.  The numbers are "reference algorithms on a shim
transport": CPU compression code and CPU memory bandwidth, no network, no GPU.

    python baseline/run_reference_on_shim.py --reference <root of the Comprex tree> --ranks 2 \
        --variants 5 3 1 --out results/reference_shim

Variants (examples/allreduce_speed.cpp:17-19): 0 AllToOne, 1 Comprex_AllToOne, 2 Ring,
3 Comprex_Ring, 4 BigRing, 5 Comprex_BigRing.  One CSV per variant and rank lands in --out
(columns: size(MB); compression; time_mean(us); time_stddev(us); sparsity_mean; sparsity_stddev).
"""
import argparse
import glob
import os
import subprocess
import sys
import tempfile
import uuid

HERE = os.path.dirname(os.path.abspath(__file__))


def build(reference: str, exe: str, source: str = "examples/allreduce_speed.cpp") -> None:
    inc = [os.path.join(HERE, "gaspicxx_shim", "include"), os.path.join(reference, "include"),
           os.path.join(reference, "src"), os.path.join(reference, "examples")]
    cmd = [os.environ.get("CXX", "g++"), "-O3", "-march=native", "-std=c++14", "-fpermissive", "-w"]
    for i in inc:
        cmd += ["-I", i]
    inc_test = os.path.join(reference, "test")
    cmd += ["-I", inc_test, os.path.join(reference, source), "-o", exe, "-lrt", "-lpthread"]
    subprocess.run(cmd, check=True)


def run(exe: str, ranks: int, variant, out: str, timeout: int) -> int:
    job = uuid.uuid4().hex[:10]
    ctl = f"/dev/shm/cxshim_{job}_ctl"
    with open(ctl, "wb") as f:
        f.truncate(2 << 20)                      # zero-filled control block
    procs = []
    try:
        for r in range(ranks):
            env = dict(os.environ, CXSHIM_RANK=str(r), CXSHIM_SIZE=str(ranks), CXSHIM_JOB=job)
            log = open(os.path.join(out, f"{variant}_rank{r:02d}.log"), "w")
            argv = [exe] + ([str(variant)] if isinstance(variant, int) else [])
            procs.append(subprocess.Popen(argv, env=env, cwd=out, stdout=log, stderr=subprocess.STDOUT))
        rc = 0
        for p in procs:
            try:
                rc |= p.wait(timeout=timeout)
            except subprocess.TimeoutExpired:
                rc |= 1
        return rc
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
        for path in glob.glob(f"/dev/shm/cxshim_{job}_*"):
            os.unlink(path)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference's source tree")
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--variants", type=int, nargs="+", default=[5])
    ap.add_argument("--program", default=None,
                    help="another program of the reference instead of the benchmark, e.g. test/comprex.cpp "
                         "or examples/comprEx.cpp (runs once; its output goes to <name>_rankNN.log)")
    ap.add_argument("--out", default="results/reference_shim")
    ap.add_argument("--timeout", type=int, default=3600)
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "allreduce_speed")
        if args.program:
            name = os.path.splitext(os.path.basename(args.program))[0]
            build(args.reference, exe, args.program)
            rc = run(exe, args.ranks, name, os.path.abspath(args.out), args.timeout)
            print(f"{args.program}: exit code {rc}", flush=True)
            print(open(os.path.join(args.out, f"{name}_rank00.log")).read()[-600:], flush=True)
            sys.exit(rc)
        build(args.reference, exe)
        for v in args.variants:
            rc = run(exe, args.ranks, v, os.path.abspath(args.out), args.timeout)
            print(f"variant {v}: exit code {rc}", flush=True)
            if rc:
                sys.exit(rc)


if __name__ == "__main__":
    main()
