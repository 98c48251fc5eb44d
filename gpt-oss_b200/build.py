"""Build steps for the native code: one nvcc command for the CUDA library.

Kept as plain command lines (no JIT cache): the .so lands beside this file so
that it is what every process loads.
"""
from __future__ import annotations

import os
import pathlib
import shutil
import subprocess

PKG_DIR = pathlib.Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB = PKG_DIR / "libgptoss_moe_b200.so"

CU_SOURCES = ["moe_api.cu", "router.cu", "permute.cu", "grouped_gemm.cu", "grouped_gemm_pair.cu",
              "weights.cu", "mxfp4.cu", "ep.cu", "decode.cu"]
HEADERS = ["common.cuh", "engine.h", "ep.h", "gemm_epilogue.cuh", "umma_2sm.cuh"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--threads", "0",
    "-Xcompiler", "-fPIC,-fvisibility=default", "-shared",
]


def _nvcc() -> str:
    for cand in ("/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: pathlib.Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(pathlib.Path(d).stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compile every CUDA source for sm_100a into libgptoss_moe_b200.so."""
    srcs = [CSRC / s for s in CU_SOURCES]
    deps = (srcs + [CSRC / h for h in HEADERS] +
            [PKG_DIR.parent / "include" / n for n in ("gptoss_moe_b200.h", "gptoss_decode_b200.h")])
    if not force and not _stale(LIB, deps):
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(LIB), *map(str, srcs), "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    env = dict(os.environ)
    # the image exports CC/CXX that point at a wrapper; let nvcc pick the system g++
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    res = subprocess.run(cmd, cwd=str(CSRC), env=env, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stdout + res.stderr)
    return LIB


HOST_LIB = PKG_DIR / "libgptoss_getp_b200.so"
HARNESS = PKG_DIR.parent / "tests" / "host" / "_build" / "getp_harness"
AGREEMENT_TEST = PKG_DIR.parent / "tests" / "host" / "_build" / "step_agreement_test"


def build_host(force: bool = False) -> pathlib.Path:
    """Compile the C++17 getp entry points (host/getp_run_b200.cpp, no CUDA in it) into
    libgptoss_getp_b200.so next to the CUDA library, and the test host program that calls
    them (tests/host/getp_harness.cpp), plus the CPU test program of the step agreement
    (tests/host/step_agreement_test.cpp).  `encode` stays undefined in the library: the
    host program supplies its tokenizer."""
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")
    src = PKG_DIR / "host" / "getp_run_b200.cpp"
    deps = [src, PKG_DIR / "host" / "getp_abi.h", PKG_DIR / "host" / "step_agreement.h",
            PKG_DIR.parent / "include" / "gptoss_decode_b200.h",
            PKG_DIR.parent / "include" / "gptoss_moe_b200.h"]
    if force or _stale(HOST_LIB, deps):
        cmd = [gxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", "-Wall", "-o", str(HOST_LIB),
               str(src), "-L", str(PKG_DIR), "-lgptoss_moe_b200", "-Wl,-rpath,$ORIGIN"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    hsrc = PKG_DIR.parent / "tests" / "host" / "getp_harness.cpp"
    if hsrc.exists() and (force or _stale(HARNESS, deps + [hsrc, HOST_LIB])):
        HARNESS.parent.mkdir(parents=True, exist_ok=True)
        cmd = [gxx, "-std=c++17", "-O2", "-pthread", "-Wall", "-o", str(HARNESS), str(hsrc),
               "-L", str(PKG_DIR), "-lgptoss_getp_b200", "-lgptoss_moe_b200",
               "-Wl,-rpath," + str(PKG_DIR), "-Wl,-rpath,$ORIGIN/../../../gpt-oss_b200"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    tsrc = PKG_DIR.parent / "tests" / "host" / "step_agreement_test.cpp"
    if tsrc.exists() and (force or _stale(AGREEMENT_TEST, [tsrc, PKG_DIR / "host" / "step_agreement.h"])):
        AGREEMENT_TEST.parent.mkdir(parents=True, exist_ok=True)
        cmd = [gxx, "-std=c++17", "-O2", "-pthread", "-Wall", "-o", str(AGREEMENT_TEST), str(tsrc)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return HOST_LIB
