"""Compile the CPU oracle (test infrastructure) into oracle/libg2d_oracle.so.

Usage: python oracle/build_oracle.py [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = ["g2d_oracle.c", "g2d_oracle_impl.h"]
TARGET = os.path.join(HERE, "libg2d_oracle.so")


def needs_build() -> bool:
    if not os.path.exists(TARGET):
        return True
    built = os.path.getmtime(TARGET)
    return any(os.path.getmtime(os.path.join(HERE, s)) > built for s in SOURCES)


def build(force: bool = False) -> str:
    if force or needs_build():
        cmd = [
            "gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
            "-Wall", "-Wno-unknown-pragmas", "-o", TARGET, os.path.join(HERE, "g2d_oracle.c"), "-lm",
        ]
        subprocess.run(cmd, check=True, cwd=HERE)
    return TARGET


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
