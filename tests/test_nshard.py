"""N-column sharding of one matmul_direct over the GPUs of a node (b200dnn_nshard_* / b200dnn_matmul_nshard; no counterpart
in the reference).  Rank r computes a column block of C from its column block of the weight and the whole source; nothing
is reduced, so the assembled C equals the single-GPU C bit for bit."""
import ctypes as C
import os
import socket

import numpy as np
import pytest


def _ranges(capi, N, world):
    out = []
    for r in range(world):
        a, b, s = C.c_int64(), C.c_int64(), C.c_int32()
        assert capi.lib.b200dnn_nshard_range(N, world, r, C.byref(a), C.byref(b), C.byref(s)) == capi.SUCCESS
        out.append((a.value, b.value, s.value))
    return out


@pytest.mark.parametrize("N", [2048, 4096, 11008, 14336, 2050, 33000])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_column_blocks_tile_the_matrix(N, world):
    """Blocks are disjoint, ordered, cover [0, N), start on 128-column tile boundaries and differ by at most one tile."""
    from zendnn_b200 import capi
    rs = _ranges(capi, N, world)
    if world == 1:
        assert rs == [(0, N, 0)]
        return
    assert rs[0][0] == 0 and rs[-1][1] == N and all(s == 1 for _, _, s in rs)
    for (a0, b0, _), (a1, b1, _) in zip(rs, rs[1:]):
        assert b0 == a1 and a1 % 128 == 0
    widths = [b - a for a, b, _ in rs]
    assert max(widths) - min(widths) <= 128 + (128 - N % 128) % 128


def test_narrow_gemms_are_not_split():
    """north_star: single GEMMs shard by N-columns only when N >= 8 tiles; below that every rank computes the whole GEMM."""
    from zendnn_b200 import capi
    for N in (16, 1000, 2047):
        assert _ranges(capi, N, 4) == [(0, N, 0)] * 4
    assert capi.lib.b200dnn_nshard_range(0, 2, 0, C.byref(C.c_int64()), C.byref(C.c_int64()), None) == capi.FAILURE
    assert capi.lib.b200dnn_nshard_range(4096, 2, 2, C.byref(C.c_int64()), C.byref(C.c_int64()), None) == capi.FAILURE


def _problem(oracle, M, K, N, seed):
    rng = np.random.default_rng(seed)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (K, N), dtype=np.int8)
    sa = rng.uniform(0.01, 0.05, M).astype(np.float32)
    sw = rng.uniform(1e-4, 5e-4, N).astype(np.float32)
    bias = rng.normal(size=N).astype(np.float32)
    add = oracle.f32_to_bf16(rng.normal(size=(M, N)).astype(np.float32))
    return A, W, sa, sw, bias, add


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("transB", [False, True])
def test_ranks_in_one_process_assemble_the_single_gpu_result(oracle, world, transB):
    """Every rank's call, made in turn on one GPU without gathering, fills its column block of one shared C: the result
    equals one unsharded call bit for bit (per-channel scales, bias, a dense binary_add operand and gelu_tanh sliced by
    column) and the oracle within 1 bf16 ulp."""
    from zendnn_b200 import capi
    from helpers import assert_bf16_close
    M, K, N = 150, 512, 2304
    A, W, sa, sw, bias, add = _problem(oracle, M, K, N, 3)
    Wc = np.ascontiguousarray(W.T) if transB else W
    po = [dict(type="binary_add", buff=add), "gelu_tanh"]
    mk = lambda out: capi.make_matmul(M, N, K, A, Wc, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], transB=transB, bias=bias,
                                      src_scale=sa, wei_scale=sw, weights_const=False, postops=po)
    whole = np.zeros((M, N), dtype=np.uint16)
    capi.check(capi.matmul(mk(whole)))
    parts = np.zeros((M, N), dtype=np.uint16)
    d = mk(parts)
    for r in range(world):
        h = C.c_void_p()
        capi.check(capi.lib.b200dnn_nshard_create(world, r, None, None, C.byref(h)))
        capi.check(capi.lib.b200dnn_matmul_nshard(h, C.byref(d), 0, None))
        capi.check(capi.lib.b200dnn_nshard_destroy(h))
    assert (parts == whole).all()
    assert_bf16_close(whole, oracle.matmul_w8a8(A, W, "bf16", src_scale=sa, wei_scale=sw, bias=bias, postops=po), 1, "nshard", atol=1e-5)
    # gathering without a communicator is refused
    h = C.c_void_p()
    capi.check(capi.lib.b200dnn_nshard_create(world, 0, None, None, C.byref(h)))
    assert capi.lib.b200dnn_matmul_nshard(h, C.byref(d), 1, None) == capi.FAILURE
    capi.check(capi.lib.b200dnn_nshard_destroy(h))


def _gather_worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    from zendnn_b200 import capi
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, K, N = 96, 1024, 4352
    A, W, sa, sw, bias, add = _problem(O, M, K, N, 11)
    t = lambda a: torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).to(dev)
    Ad, Wd, sad, swd, bd = t(A), t(W), t(sa), t(sw), t(bias)
    box = [None]
    if rank == 0:
        ident = (C.c_uint8 * 128)()
        capi.check(capi.lib.b200dnn_ep_nccl_unique_id(ident))
        box[0] = bytes(ident)
    dist.broadcast_object_list(box, src=0)
    ident = (C.c_uint8 * 128).from_buffer_copy(box[0])
    h = C.c_void_p()
    capi.check(capi.lib.b200dnn_nshard_create(world, rank, ident, None, C.byref(h)))
    st = torch.cuda.current_stream().cuda_stream
    mk = lambda out: capi.make_matmul(M, N, K, Ad, Wd, out, src_dt=capi.DT["s8"], dst_dt=capi.DT["bf16"], bias=bd,
                                      src_scale=sad, wei_scale=swd, weights_const=True, postops=["relu"])
    whole = torch.zeros(M, N, dtype=torch.int16, device=dev)
    capi.check(capi.matmul(mk(whole), st))
    ok = True
    for _ in range(2):
        full = torch.zeros(M, N, dtype=torch.int16, device=dev)
        d = mk(full)
        capi.check(capi.lib.b200dnn_matmul_nshard(h, C.byref(d), 1, st))
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(full, whole))
    ret[rank] = ok
    dist.barrier()
    capi.check(capi.lib.b200dnn_nshard_destroy(h))
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_one_process_per_gpu_gathers_the_whole_result(world):
    """One process per GPU over NCCL: every rank ends with the whole C, equal to its own unsharded call bit for bit."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_gather_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)), dict(ret)
