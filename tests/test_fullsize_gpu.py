"""Full-size parity: the large configurations run whole on the device; the CPU oracle recomputes a
seeded sample of rows / tokens (every output row depends only on its own input row and the weights),
and size-independent identities cover the rest of the output."""

import numpy as np
import pytest

from helpers import assert_bf16_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from zendnn_b200 import capi as c
    assert c.lib.b200dnn_device_count() > 0
    return c


def _torch():
    import torch
    return torch


def _u16(t):
    torch = _torch()
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def test_prefill_config3_sampled_rows(capi, oracle):
    """M2048 K4096 N14336: bf16 activations -> per-token s8 inside the call -> GEMM -> bias + gelu_tanh -> bf16."""
    torch = _torch()
    M, K, N = 2048, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = torch.randint(-127, 128, (K, N), generator=g, device="cuda", dtype=torch.int8)
    ws = (torch.rand(N, generator=g, device="cuda") * 4e-4 + 1e-4).float()
    bias = torch.randn(N, generator=g, device="cuda")
    dst = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    d = capi.make_matmul(M, N, K, x, w, dst, src_dt=capi.DT["bf16"], dst_dt=capi.DT["bf16"], bias=bias,
                         dynamic_quant=True, src_scale=capi.quant(None, M, capi.DT["f32"]), wei_scale=ws,
                         postops=["gelu_tanh"])
    assert capi.matmul(d, torch.cuda.current_stream().cuda_stream) == capi.SUCCESS, capi.last_error()
    torch.cuda.synchronize()
    rows = np.random.default_rng(0).choice(M, 40, replace=False)
    rows.sort()
    xs = _u16(x[torch.from_numpy(rows).cuda()])
    q, s = oracle.quant_per_token(xs)
    ref = oracle.matmul_w8a8(q, w.cpu().numpy(), "bf16", src_scale=s, wei_scale=ws.cpu().numpy(),
                             bias=bias.cpu().numpy(), postops=["gelu_tanh"])
    assert_bf16_close(_u16(dst)[rows], ref, 1, "config 3 sampled rows", atol=1e-5)

    # identity over the whole output: all-ones s8 activations give the column sums of W in every row
    ones = torch.ones(M, K, device="cuda", dtype=torch.int8)
    out32 = torch.zeros(M, N, device="cuda", dtype=torch.int32)
    d = capi.make_matmul(M, N, K, ones, w, out32, src_dt=capi.DT["s8"], dst_dt=capi.DT["s32"])
    assert capi.matmul(d, torch.cuda.current_stream().cuda_stream) == capi.SUCCESS, capi.last_error()
    torch.cuda.synchronize()
    colsum = w.to(torch.int32).sum(0)
    assert bool((out32 == colsum[None, :]).all())
    capi.lib.b200dnn_clear_caches()


def _device_experts(torch, capi, g, n, H, I):
    ex, keep = (capi.MoeExpert * n)(), []
    for e in range(n):
        w13 = torch.randint(-127, 128, (H, 2 * I), generator=g, device="cuda", dtype=torch.int8)
        s13 = (torch.rand(2 * I, generator=g, device="cuda") * 4e-4 + 1e-4).float()
        w2 = torch.randint(-127, 128, (I, H), generator=g, device="cuda", dtype=torch.int8)
        s2 = (torch.rand(H, generator=g, device="cuda") * 4e-4 + 1e-4).float()
        keep.append((w13, s13, w2, s2))
        ex[e].w13, ex[e].ldb13, ex[e].w13_scale = w13.data_ptr(), 2 * I, s13.data_ptr()
        ex[e].w2, ex[e].ldb2, ex[e].w2_scale = w2.data_ptr(), H, s2.data_ptr()
    return ex, keep


@pytest.mark.parametrize("T,H,I,E,k,S,zipf", [(4096, 4096, 14336, 8, 2, 0, False), (16384, 2048, 1408, 64, 6, 2, True)])
def test_moe_full_size_sampled_tokens(capi, oracle, T, H, I, E, k, S, zipf):
    """Configurations 4 and 5 whole on the device; the oracle recomputes a sample of tokens end to end."""
    torch = _torch()
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device="cuda")
    if zipf:
        p = torch.arange(1, E + 1, device="cuda", dtype=torch.float64) ** -1.1
        logits = (logits + torch.log(p / p.sum())[torch.randperm(E, generator=g, device="cuda")].float()).contiguous()
    ex, keep = _device_experts(torch, capi, g, E + S, H, I)
    out = torch.zeros(T, H, device="cuda", dtype=torch.bfloat16)
    st = capi.lib.b200dnn_moe_layer(x.data_ptr(), H, logits.data_ptr(), T, E, S, k, ex, H, I, H, 0, capi.ACT["silu_and_mul"],
                                    out.data_ptr(), H, torch.cuda.current_stream().cuda_stream)
    assert st == capi.SUCCESS, capi.last_error()
    torch.cuda.synchronize()
    assert bool(torch.isfinite(out.float()).all())

    toks = np.sort(np.random.default_rng(2).choice(T, 24, replace=False))
    ti = torch.from_numpy(toks).cuda()
    ids, w = oracle.router_topk(logits[ti].cpu().numpy(), k)
    ids_all = np.concatenate([ids, np.tile(np.arange(E, E + S, dtype=np.int32), (len(toks), 1))], axis=1)
    w_all = np.concatenate([w, np.ones((len(toks), S), dtype=np.float32)], axis=1)
    need = set(int(e) for e in ids_all.reshape(-1))
    empty = np.zeros((1, 1), dtype=np.int8)
    w13 = [keep[e][0].cpu().numpy() if e in need else empty for e in range(E + S)]
    s13 = [keep[e][1].cpu().numpy() for e in range(E + S)]
    w2 = [keep[e][2].cpu().numpy() if e in need else empty for e in range(E + S)]
    s2 = [keep[e][3].cpu().numpy() for e in range(E + S)]
    ref, _ = oracle.fused_moe(_u16(x[ti]), ids_all, w_all, w13, s13, w2, s2)
    assert_bf16_close(_u16(out[ti]), ref, 1, "sampled tokens")
    capi.lib.b200dnn_clear_caches()
