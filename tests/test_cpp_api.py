"""The C++ LowOHA interface (include/zendnnl_b200/lowoha.hpp, libzendnnl_b200.so): a caller-side C++
program is compiled against the reference-style include paths (CPU check) and run on a GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "zendnn_b200")
SRC = os.path.join(ROOT, "tests", "cpp", "test_lowoha_api.cpp")
OUT = os.path.join(ROOT, "tests", "cpp", "_build", "test_lowoha_api")


def _compile():
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cmd = [cxx, "-O1", "-std=c++17", "-ffp-contract=off", "-I", os.path.join(ROOT, "include"), SRC, "-o", OUT,
           "-L", PKG, "-lzendnnl_b200", "-lb200dnn", "-Wl,-rpath," + PKG]
    subprocess.check_call(cmd)
    return OUT


def test_cpp_caller_compiles_and_links():
    assert os.path.exists(os.path.join(PKG, "libzendnnl_b200.so")), "run python -m zendnn_b200.build"
    exe = _compile()
    assert os.path.exists(exe)
    # the shim library exports the reference's mangled C++ names
    syms = subprocess.check_output(["nm", "-DC", os.path.join(PKG, "libzendnnl_b200.so")], text=True)
    for name in ("zendnnl::lowoha::matmul::matmul_direct(", "zendnnl::lowoha::matmul::group_matmul_direct(",
                 "zendnnl::lowoha::reorder::reorder_direct(", "zendnnl::lowoha::reorder::weight_prepack_size(",
                 "zendnnl::lowoha::reorder::group_dynamic_quant("):
        assert name in syms, name


@pytest.mark.gpu
def test_cpp_caller_runs():
    exe = _compile()
    p = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-2000:]
    assert " 0 failures" in p.stdout
