"""Build the CPU oracle (test infrastructure): oracle/liboxm_oracle.so.

`python oracle/build.py`.  -O2, no fast-math, no FP contraction: the order and
rounding of every operation in the triple loop is part of the oracle's
definition.  The reference itself is Rust with `todo!()` bodies and cannot be
compiled, so there is no oracle/_ref.
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oxm_oracle.c")
OUT = os.path.join(HERE, "liboxm_oracle.so")


def build_oracle(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "oxm_oracle.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps):
        return OUT
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-std=c11", "-fPIC", "-shared", "-o", OUT, SRC,
           "-lm", "-lpthread"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{' '.join(cmd)}\n{res.stderr}")
    return OUT


if __name__ == "__main__":
    print(build_oracle(force=True))
