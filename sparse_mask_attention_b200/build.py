"""Builds libsma_b200.so (the C-ABI library declared in include/sma.h) in-tree with nvcc for sm_100a.

Run as ``python sparse_mask_attention_b200/build.py`` (a plain script: the package itself refuses to import
until the library exists); ``build_library()`` is what ``__graft_entry__.build()`` calls.
nvcc cross-compiles without a GPU, so this works on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_NAME = "libsma_b200.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)
# The same sources with -DSMA_WAIT_TEST_BUILD: waits that give up after milliseconds and a switch that leaves one load
# unrequested.  Loaded only by the test of the bounded waits; the package never touches it.
WAIT_TEST_LIB_PATH = os.path.join(PKG_DIR, "libsma_b200_waittest.so")

SOURCES = ["sma_capi.cu"]
# every header next to the sources, so that a new one cannot be forgotten here
HEADERS = sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cuh")) + [os.path.join("..", "..", "include", "sma.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libsma_b200.so cannot be built")
    return nvcc


def is_stale(lib_path: str = LIB_PATH) -> bool:
    if not os.path.exists(lib_path):
        return True
    built = os.path.getmtime(lib_path)
    deps = [os.path.join(CSRC_DIR, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def _compile(lib_path: str, extra: list, verbose: bool) -> str:
    cmd = [find_nvcc(), *NVCC_FLAGS, *extra]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", lib_path, *[os.path.join(CSRC_DIR, s) for s in SOURCES]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building %s (exit %d)" % (os.path.basename(lib_path), proc.returncode))
    return lib_path


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/sma_capi.cu into libsma_b200.so next to this file; returns the path."""
    if not force and not is_stale():
        return LIB_PATH
    return _compile(LIB_PATH, [], verbose)


def build_wait_test_library(force: bool = False, verbose: bool = False) -> str:
    """The test build of the same sources (see WAIT_TEST_LIB_PATH); returns the path."""
    if not force and not is_stale(WAIT_TEST_LIB_PATH):
        return WAIT_TEST_LIB_PATH
    return _compile(WAIT_TEST_LIB_PATH, ["-DSMA_WAIT_TEST_BUILD"], verbose)


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_wait_test_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
