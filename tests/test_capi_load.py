"""CPU-side checks of the boundary: the shared library loads and exports exactly what
include/b200dnn.h declares.  No compute entry point is called here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200dnn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200dnn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from zendnn_b200 import capi
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(capi.lib, n), "libb200dnn.so does not export " + n
    assert sorted(capi.EXPORTS) == names


def test_version_and_sizes():
    from zendnn_b200 import capi
    assert capi.lib.b200dnn_version() >= 100
    sz = capi.lib.b200dnn_prepack_size(4096, 4096, 0)
    assert sz % 64 == 0 and sz >= 4096 * 4096
    assert capi.lib.b200dnn_prepack_size(0, 16, 0) == 0
    # K and N are padded to 128 inside the packed form
    assert capi.lib.b200dnn_prepack_size(100, 100, 0) == 256 + 128 * 4 + 128 * 128


def test_struct_layout_matches_header():
    from zendnn_b200 import capi
    assert ctypes.sizeof(capi.Quant) == 24
    assert ctypes.sizeof(capi.PostOp) == 32
    assert ctypes.sizeof(capi.MatmulDesc) == 4 * 8 + 3 * 8 + 4 * 8 + 4 * 4 + 3 * 24 + 8 * 32 + 8 + 3 * 24 + 8
    assert ctypes.sizeof(capi.MoeExpert) == 136


def test_static_scratch_bound_is_host_arithmetic():
    """The no-allocation matmul's fixed array: decode shapes fit, shapes that are not split over K need nothing, and a
    split shape beyond 8 MiB of partial sums (only reachable on a device with far more SMs) is refused."""
    from zendnn_b200 import capi
    need = ctypes.c_size_t(0)
    q = lambda M, N, K, sm: capi.lib.b200dnn_static_scratch_query(M, N, K, sm, ctypes.byref(need))
    for M in (1, 4, 16):
        for K, N in ((4096, 4096), (4096, 11008), (11008, 4096)):
            assert q(M, N, K, 148) == capi.SUCCESS and 0 <= need.value <= (8 << 20) + 4096 * 4
    assert q(2048, 4096, 256, 148) == capi.SUCCESS and need.value == 0      # 16384 tiles, not split
    assert q(16, 200000, 256, 148) == capi.SUCCESS and need.value == 0
    assert q(16, 32768, 16384, 100000) == capi.FAILURE and need.value > (8 << 20)
    assert "static scratch" in capi.last_error()
    assert q(0, 16, 16, 148) == capi.FAILURE
