"""The reference's own compression code on one CPU core, as a baseline for the kernel table.

The reference cannot run as a whole here (it needs GPI-2 / GaspiCxx), but its compression math
is header-only C++ (src/threshold.hxx, src/compressor.hxx).  This script compiles
``bench/reference_cpu_kernels.cpp`` against those headers, unmodified, and times
``ThresholdTopK::prepare_with``, ``CompressorIndexPairs::compress_add_update`` and ``::add``
(the three steps the GPU kernels threshold / compress / apply_add replace).

    python bench/reference_cpu.py --reference /path/to/Comprex --out results/reference_cpu.jsonl
"""
import argparse
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the reference's source tree")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    inc = os.path.join(args.reference, "src")
    if not os.path.exists(os.path.join(inc, "compressor.hxx")):
        sys.exit(f"{inc}/compressor.hxx not found")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "reference_cpu_kernels")
        # -fpermissive: the headers do arithmetic on void* (a GNU extension)
        cmd = [os.environ.get("CXX", "g++"), "-O3", "-march=native", "-std=c++14", "-fpermissive", "-w",
               "-I", inc, os.path.join(HERE, "reference_cpu_kernels.cpp"), "-o", exe]
        subprocess.run(cmd, check=True)
        res = subprocess.run([exe, str(args.reps)], check=True, capture_output=True, text=True)
    print(res.stdout, end="")
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            f.write(res.stdout)


if __name__ == "__main__":
    main()
