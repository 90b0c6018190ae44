"""Cycles per ``tcgen05.mma`` (M 128, K 16, bf16) for several N and operand layouts, one or two issuing threads.

    python -m lbi_b200.benchmarks.mma_issue

Compiles ``mma_issue_bench.cu`` with nvcc for sm_100a into a temporary directory and runs it on one GPU.  Every CTA (one
per SM) issues 2000 instructions on zero operands and reports cycles per instruction as seen by the issuing thread and
until completion.  Measured on B200: N 256 -> 128 cycles, N 128 -> 64, N <= 64 -> 54.5 (a floor), independent of the
operand layout; the issuing thread is back-pressured, so issue time equals execution time.
"""
from __future__ import annotations

import os
import subprocess
import sys
import tempfile


def main() -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    csrc = os.path.join(os.path.dirname(here), "csrc")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "mma_issue_bench")
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-I", csrc,
                        os.path.join(here, "mma_issue_bench.cu"), "-o", exe, "-lcuda"], check=True)
        sys.exit(subprocess.run([exe]).returncode)


if __name__ == "__main__":
    main()
