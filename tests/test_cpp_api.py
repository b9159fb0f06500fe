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
                 "zendnnl::lowoha::reorder::group_dynamic_quant(", "zendnnl::lowoha::normalization::normalization_direct(", "zendnnl::lowoha::sdpa::sdpa_direct("):
        assert name in syms, name


def test_per_call_log_line_follows_the_reference_env_knobs():
    """ZENDNNL_API_LOG_LEVEL >= info prints one line per call, ZENDNNL_ENABLE_PROFILER + ZENDNNL_PROFILE_LOG_LEVEL=4 adds the
    timed line (reference: lowoha_operators/matmul/lowoha_matmul.cpp:468-506, common/config_manager.cpp:273-330); unset, the
    call prints nothing.  The call here is refused in the shim, so no device is needed."""
    exe = _compile()
    env = {k: v for k, v in os.environ.items() if not k.startswith("ZENDNNL_")}
    quiet = subprocess.run([exe, "--log-line"], capture_output=True, text=True, timeout=120, env=env)
    assert quiet.returncode == 0 and "LOWOHA matmul_direct" not in quiet.stderr
    api = subprocess.run([exe, "--log-line"], capture_output=True, text=True, timeout=120, env=dict(env, ZENDNNL_API_LOG_LEVEL="info"))
    lines = [l for l in api.stderr.splitlines() if "LOWOHA matmul_direct" in l]
    assert len(lines) == 1 and "M=2, N=2, K=4" in lines[0] and "transA=true" in lines[0] and "input_dtype=s8" in lines[0]
    assert "output_dtype=bf16" in lines[0] and "time=" not in lines[0]
    prof = subprocess.run([exe, "--log-line"], capture_output=True, text=True, timeout=120,
                          env=dict(env, ZENDNNL_ENABLE_PROFILER="1", ZENDNNL_PROFILE_LOG_LEVEL="4"))
    lines = [l for l in prof.stderr.splitlines() if "LOWOHA matmul_direct" in l]
    assert len(lines) == 1 and "time=" in lines[0] and " ms" in lines[0]
    # the profiler alone, at the default profile level, stays silent as the reference's does
    off = subprocess.run([exe, "--log-line"], capture_output=True, text=True, timeout=120, env=dict(env, ZENDNNL_ENABLE_PROFILER="1"))
    assert "LOWOHA matmul_direct" not in off.stderr


@pytest.mark.gpu
def test_cpp_caller_runs():
    exe = _compile()
    p = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-4000:] + p.stderr[-2000:]
    assert " 0 failures" in p.stdout
