"""GPU test of b200dnn_matmul_static_scratch, the entry point for callers that may not allocate
device memory at call time (a serving process whose memory pool already owns the whole GPU, or a
latency-critical loop that cannot afford a blocking cudaMalloc).  It keeps its split-K scratch in a
fixed array inside the library and takes device pointers only.

The file name sorts last on purpose: if this addition ever fails, a run that stops at the first
failure has already exercised every other test.  The check itself needs nothing from the other
tests: outputs must equal those of the regular entry point (b200dnn_matmul) bit for bit, on two
calls in a row that share the scratch array, and shapes beyond the fixed scratch must be refused."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0
    return c


def _case(capi, torch, dev, M, K, N, seed, dst="bf16", u8=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = torch.randint(-127, 128, (K, N), dtype=torch.int8, generator=g).to(dev)
    if u8:
        A = torch.randint(0, 256, (M, K), dtype=torch.uint8, generator=g).to(dev)
    else:
        A = torch.randint(-127, 128, (M, K), dtype=torch.int8, generator=g).to(dev)
    # s8 source: per-token scales; u8 source: one scale and a zero-point (the combinations the API allows)
    sa = (torch.rand(1 if u8 else M, generator=g) * 0.05 + 0.01).to(dev)
    zp = torch.tensor([128], dtype=torch.int32, device=dev) if u8 else None
    sw = (torch.rand(N, generator=g) * 0.009 + 0.001).to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    packed = torch.empty(capi.lib.b200dnn_prepack_size(K, N, 0), dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    capi.check(capi.lib.b200dnn_prepack(W.data_ptr(), K, N, N, 0, 0, packed.data_ptr(), st))
    tdt = {"bf16": torch.bfloat16, "f32": torch.float32}[dst]
    outs = [torch.zeros(M, N, dtype=tdt, device=dev) for _ in range(2)]
    descs = [capi.make_matmul(M, N, K, A, packed, o, src_dt=capi.DT["u8" if u8 else "s8"], dst_dt=capi.DT[dst],
                              wei_format="r", src_scale=sa, wei_scale=sw, src_zp=zp, bias=bias, postops=["relu"], force_kernel=1)
             for o in outs]
    keep = (W, A, sa, sw, zp, bias, packed)
    return descs, outs, keep


def test_static_scratch_matches_regular_entry_twice_in_a_row(capi):
    import torch
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    # two different shapes back to back: the second call finds the first call's data in the scratch
    for (M, K, N, dst, u8) in [(16, 4096, 1024, "bf16", False), (5, 1000, 200, "f32", True)]:
        descs, outs, keep = _case(capi, torch, dev, M, K, N, seed=M + K, dst=dst, u8=u8)
        capi.check(capi.lib.b200dnn_matmul(descs[0], st))                   # regular entry point
        capi.check(capi.lib.b200dnn_matmul_static_scratch(descs[1], st))    # no-allocation entry point
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1]), "first call differs (M=%d K=%d N=%d)" % (M, K, N)
        outs[1].zero_()
        capi.check(capi.lib.b200dnn_matmul_static_scratch(descs[1], st))    # again, same scratch
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1]), "second call differs (M=%d K=%d N=%d)" % (M, K, N)
        assert float(outs[1].float().abs().sum()) > 1e-3


def test_static_scratch_rejects_what_it_cannot_hold(capi):
    import torch
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    descs, outs, keep = _case(capi, torch, dev, 4, 256, 64, seed=1)
    d = descs[1]
    d.wei_format = ord("n")                       # raw weights would need a packing buffer
    assert capi.lib.b200dnn_matmul_static_scratch(d, st) == capi.UNIMPLEMENTED
    d.wei_format = ord("r")
    d.dynamic_quant = 1                           # quantising the source would need workspace
    assert capi.lib.b200dnn_matmul_static_scratch(d, st) == capi.UNIMPLEMENTED
    d.dynamic_quant = 0
    # nothing is staged, so a host pointer must be refused, not handed to the kernel
    host_src = np.zeros((4, 256), dtype=np.int8)
    src_dev = d.src
    d.src = host_src.ctypes.data
    assert capi.lib.b200dnn_matmul_static_scratch(d, st) == capi.FAILURE
    assert "device pointers only" in capi.last_error()
    d.src = src_dev
    # a weight packed for another shape is refused (its header says K=256, N=64), not read out of bounds
    d.N, d.ldc, d.wei_scale.count = 128, 128, 128
    assert capi.lib.b200dnn_matmul_static_scratch(d, st) == capi.FAILURE
    assert "prepacked weight is" in capi.last_error()
    torch.cuda.synchronize()


def test_unsplit_shapes_need_no_scratch_and_steady_calls_allocate_nothing(capi):
    """A shape with more output tiles than the fixed array has counters for is not split over K, uses no scratch and
    must run (and equal the regular entry point); a steady-state call leaves the free device memory unchanged."""
    import ctypes as C
    import torch
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    M, K, N = 2048, 256, 4096                      # 128 x 128 = 16384 tiles, no split
    need = C.c_size_t(123)
    assert capi.lib.b200dnn_static_scratch_query(M, N, K, 0, C.byref(need)) == capi.SUCCESS and need.value == 0
    descs, outs, keep = _case(capi, torch, dev, M, K, N, seed=7)
    descs[0].force_kernel = 3                      # the same tiled streaming kernel through the regular entry point
    capi.check(capi.lib.b200dnn_matmul(descs[0], st))
    capi.check(capi.lib.b200dnn_matmul_static_scratch(descs[1], st))
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    # steady state: the first call on the device is the warm-up (module load, symbol address); later calls allocate nothing
    d2, o2, keep2 = _case(capi, torch, dev, 16, 4096, 1024, seed=3)
    capi.check(capi.lib.b200dnn_matmul_static_scratch(d2[1], st))
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        capi.check(capi.lib.b200dnn_matmul_static_scratch(d2[1], st))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
