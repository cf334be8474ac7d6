"""Builds the C restatement (oracle/lutgemm_oracle.c) into oracle/_build/liblutgemm_oracle.so.

The reference has no CPU implementation of this path and its CUDA extension needs libtorch and a
GPU, so there is nothing under the reference tree that gcc alone can turn into a CPU checker;
oracle/_ref/ therefore stays empty and the timed CPU baseline is this port (kind "port").
"""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "lutgemm_oracle.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_OUT = os.path.join(_OUT_DIR, "liblutgemm_oracle.so")


def build_oracle(force: bool = False) -> str:
    os.makedirs(_OUT_DIR, exist_ok=True)
    if not force and os.path.exists(_OUT) and os.path.getmtime(_OUT) >= os.path.getmtime(_SRC):
        return _OUT
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-shared", "-fPIC", "-o", _OUT + ".tmp", _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    os.replace(_OUT + ".tmp", _OUT)
    return _OUT


def load_oracle() -> ctypes.CDLL:
    try:
        path = build_oracle()
    except (subprocess.CalledProcessError, FileNotFoundError):
        if not os.path.exists(_OUT):
            raise
        path = _OUT
    return ctypes.CDLL(path)


if __name__ == "__main__":
    print(build_oracle(force=True))
