"""Builds the in-tree CUDA library for sm_100a with nvcc (no GPU needed: nvcc cross-compiles).

    python -m albatross_b200.build [--force] [--verbose]

Output: albatross_b200/_C/libalbatross_b200.so (git-ignored; it ships with the source tree) and, next to it,
librwkv7_state_fwd_fp16.so: the torch operator shim (g++, csrc/torch_op.cpp).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_C")
LIB = os.path.join(OUT_DIR, "libalbatross_b200.so")
LIB_CHECKED = os.path.join(OUT_DIR, "libalbatross_b200_checked.so")   # -DAB_BOUNDS_CHECK build (see csrc/common.cuh)
# -fmad=false: a*b+c is fused only where the source says fmaf(). The same device functions are compiled into several
# kernels (the persistent decode kernel and the per-phase launches share their matrix-vector and head code); left to
# the compiler, which products get fused depends on the code around them, and two kernels that should agree bit for
# bit differ in a last fp16 digit once in a few hundred tokens.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-fmad=false",
              "-Xcompiler", "-fPIC", "-shared", "-Xptxas", "-v"]


def _sources():
    out = [os.path.join(HERE, "..", "include", "albatross_b200.h"), os.path.abspath(__file__)]   # (this file holds the flags)
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, f))
    return out


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in _sources())


def build(force: bool = False, verbose: bool = False, bounds_check: bool = False) -> str:
    """bounds_check: the debugging variant whose kernels range-check their computed indices and record a status bit
    instead of making an out-of-range access (loaded by `_lib` when AB_BOUNDS_CHECK=1 is in the environment)."""
    lib = LIB_CHECKED if bounds_check else LIB
    if not force and os.path.exists(lib) and all(os.path.getmtime(s) <= os.path.getmtime(lib) for s in _sources()):
        return lib
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-DAB_BOUNDS_CHECK"] if bounds_check else []) + [os.path.join(CSRC, "albatross_b200.cu"), "-o", lib]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OUT_DIR, "build_checked.log" if bounds_check else "build.log")
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed (exit {res.returncode}); see {log}")
    return lib


TORCH_OP_LIB = os.path.join(OUT_DIR, "librwkv7_state_fwd_fp16.so")


def build_torch_op(force: bool = False) -> str:
    """Builds the operator shim csrc/torch_op.cpp (plain C++, g++): `torch.ops.rwkv7_state_fwd_fp16.forward` backed by
    ab_wkv7_fwd. Links against the kernel library next to it (found at run time through $ORIGIN)."""
    src = os.path.join(CSRC, "torch_op.cpp")
    if not force and os.path.exists(TORCH_OP_LIB) and os.path.getmtime(TORCH_OP_LIB) >= max(os.path.getmtime(src), os.path.getmtime(LIB)):
        return TORCH_OP_LIB
    import torch
    from torch.utils import cpp_extension as ce
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", src, "-o", TORCH_OP_LIB,
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    cmd += ["-I" + p for p in ce.include_paths("cuda")] + ["-I/usr/local/cuda/include"]
    cmd += ["-L" + p for p in ce.library_paths("cuda")] + ["-L" + OUT_DIR]
    cmd += ["-lalbatross_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-Wl,-rpath,$ORIGIN"]
    cmd += ["-Wl,-rpath," + p for p in ce.library_paths("cuda")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    with open(os.path.join(OUT_DIR, "build_torch_op.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("building the torch operator shim failed; see " + os.path.join(OUT_DIR, "build_torch_op.log"))
    return TORCH_OP_LIB


def resource_usage(log_path: str = os.path.join(OUT_DIR, "build.log")) -> dict:
    """Per kernel: registers and spill bytes as ptxas reported them in the last build (kernel name -> dict).

    The streaming kernels sit at their register cap (128 registers x 512 threads); a spill in them costs tens of
    percent of decode throughput, so the tests keep an eye on this."""
    import re
    out, name, props_of = {}, None, None
    for line in open(log_path):
        m = re.search(r"Compiling entry function '(\S+)'", line)
        if m:
            name = props_of = m.group(1)
            continue
        m = re.search(r"Function properties for (\S+)", line)
        if m:
            props_of = m.group(1)     # the entry itself, or a device function it calls (not inlined)
            continue
        m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m and name:
            # spills of the entry and of the functions it calls add up
            out.setdefault(name, {}).setdefault("spill_bytes", 0)
            out[name]["spill_bytes"] += int(m.group(2)) + int(m.group(3))
            continue
        m = re.search(r"Used (\d+) registers", line)
        if m and name:
            out.setdefault(name, {})["registers"] = int(m.group(1))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--bounds-check" in sys.argv:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, bounds_check=True))
    print(build_torch_op(force="--force" in sys.argv))
