"""Builds libetcuda.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m effect_torch_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The library sits next to this file so it travels with the
source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libetcuda.so")
# stand-alone measurement program of the tensor-core issue rates (bench.py --workload tensor-issue runs it)
PROBE_SRC = os.path.join(CSRC, "probes", "tensor_issue_probe.cu")
PROBE = os.path.join(HERE, "tensor_issue_probe.bin")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA backend cannot be built")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    deps.append(os.path.join(os.path.dirname(HERE), "include", "et_cuda.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build_probe(force: bool = False) -> str:
    if force or not os.path.exists(PROBE) or os.path.getmtime(PROBE) < os.path.getmtime(PROBE_SRC):
        host_cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
        subprocess.run([_nvcc(), "-ccbin", host_cxx, "-O3", "-std=c++17", "-lineinfo"] + ARCH_FLAGS + ["-o", PROBE, PROBE_SRC], check=True)
    return PROBE


def build(force: bool = False, verbose: bool = False) -> str:
    build_probe(force)
    if not force and not _stale():
        return LIB
    objs = []
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    host_cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    common = ["-ccbin", host_cxx, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--expt-relaxed-constexpr"] + ARCH_FLAGS
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in sources():
        obj = os.path.join(build_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        extra = ["-x", "cu"] if src.endswith(".cpp") else []
        cmd = [_nvcc()] + common + extra + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed (see output above)")
    link = [_nvcc(), "-ccbin", host_cxx, "-shared", "-o", LIB] + objs + ["-lcudart"] + ARCH_FLAGS
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
