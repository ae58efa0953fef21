"""Compile the CPU oracle (test infrastructure) into oracle/_build/libaion_oracle.so.

Plain g++; no reference sources are compiled (the reference is Zig and has no
toolchain here), so there is no oracle/_ref target.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libaion_oracle.so")
SOURCES = ["aion_oracle.cpp", "aion_oracle_fast.cpp"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(
        os.path.getmtime(os.path.join(HERE, s)) > t for s in SOURCES if os.path.exists(os.path.join(HERE, s))
    )


def build(force: bool = False) -> str:
    if not force and not _stale():
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    srcs = [os.path.join(HERE, s) for s in SOURCES if os.path.exists(os.path.join(HERE, s))]
    cmd = [
        "g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp",
        # Keep a*b+c as two roundings, as the reference's Zig does.
        "-ffp-contract=off", "-fno-fast-math",
        "-fvisibility=hidden", "-Wall", "-Wextra",
        "-o", LIB, *srcs,
    ]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
