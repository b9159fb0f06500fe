"""Builds the native libraries in-tree.

  libb200dnn.so        CUDA kernels + C ABI (include/b200dnn.h), nvcc for sm_100a only
  libzendnnl_b200.so   C++ shims with the reference's LowOHA signatures over the C ABI (g++)

Run as `python -m zendnn_b200.build` or through __graft_entry__.build().  nvcc cross-compiles
without a GPU.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_CUDA = os.path.join(PKG, "libb200dnn.so")
LIB_HOST = os.path.join(PKG, "libzendnnl_b200.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources(exts):
    out = []
    for d in (CSRC, os.path.join(ROOT, "include"), os.path.join(ROOT, "include", "zendnnl_b200")):
        if os.path.isdir(d):
            out += [os.path.join(d, f) for f in sorted(os.listdir(d)) if f.endswith(exts)]
    return out


def nvcc_path():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def host_cxx():
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"


def build(force=False, verbose=False):
    deps = _sources((".cu", ".cuh", ".h", ".hpp", ".cpp"))
    if force or _newer(LIB_CUDA, deps):
        cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
               "-ccbin", host_cxx(), "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
               "-Xptxas", "-v" if verbose else "-O3",
               "-I", os.path.join(ROOT, "include"), "-o", LIB_CUDA] + \
              [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu")] + ["-lcudart"]
        subprocess.check_call(cmd)
    host_src = os.path.join(CSRC, "lowoha_host.cpp")
    if os.path.exists(host_src) and (force or _newer(LIB_HOST, deps)):
        cmd = [host_cxx(), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
               "-I", os.path.join(ROOT, "include"), "-o", LIB_HOST, host_src,
               "-L", PKG, "-lb200dnn", "-Wl,-rpath,$ORIGIN"]
        subprocess.check_call(cmd)
    return LIB_CUDA


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_CUDA)
