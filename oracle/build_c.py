"""Compile the C restatement next to this file into oracle/_build/libint8_ref.so (gcc)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libint8_ref.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "int8_ref.c")
    os.makedirs(OUT_DIR, exist_ok=True)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.check_call(
            ["gcc", "-O2", "-fno-fast-math", "-shared", "-fPIC", "-o", LIB, src, "-lm"]
        )
    return LIB


if __name__ == "__main__":
    print(build(force=True))
