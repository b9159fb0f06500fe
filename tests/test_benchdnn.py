"""The benchdnn-style driver (zendnn_b200/benchdnn.py): input-line parsing and the supported-subset decision on CPU,
a few lines end to end on the GPU.  Line format: benchdnn/doc/matmul.md of the reference."""
import numpy as np
import pytest

from zendnn_b200 import benchdnn as B


def test_parse_full_line():
    c = B.parse_line("64, 512, 256, 10, bf16:s8:bf16, true, f32, gelu_tanh, , aocl_dlp, true, false, false, 1.0, 0.0, "
                     "per-channel, , f32, 3, true, per-token, 0, f32")
    assert (c["m"], c["k"], c["n"], c["iters"]) == (64, 512, [256], 10)
    assert (c["sdt"], c["wdt"], c["ddt"]) == ("bf16", "s8", "bf16")
    assert c["bias"] and c["post_ops"] == ["gelu_tanh"] and c["dyn"] and c["sgran"] == "per-token" and c["warmup"] == 3
    assert B.unsupported_reason(c) is None


def test_parse_defaults_comments_and_pipeline():
    assert B.parse_line("# a comment") is None and B.parse_line("   ") is None
    c = B.parse_line("16, 128, 64:32, 5, u8:s8:bf16")
    assert c["n"] == [64, 32] and c["is_weights_const"] and not c["bias"] and c["wgran"] == "per-channel"
    assert c["alpha"] == 1.0 and c["beta"] == 0.0 and not c["dyn"]
    assert B.parse_line("16, 128, 64, 5, u8:s8:bf16   # a trailing comment")["n"] == [64]
    with pytest.raises(ValueError):
        B.parse_line("16, 128")
    with pytest.raises(ValueError):
        B.parse_line("16, 128, 64, 5, f32:f32")
    with pytest.raises(ValueError):
        B.parse_line("0, 128, 64, 5, u8:s8:bf16")


@pytest.mark.parametrize("line,why", [
    ("128, 256, 64, 1, f32:f32:f32, true, f32, relu", "weights f32"),
    ("128, 256, 64, 1, bf16:s4:bf16, true, f32, , , x, true, false, false, 1.0, 0.0, per-group, 128, bf16", "weights s4"),
    ("128, 256, 64, 1, bf16:s8:bf16, false, f32, , , x, true, false, false, 1.0, 0.0, per-channel, , f32, 0, true, per-group, 128, bf16",
     "per-group source"),
    ("128, 256, 64, 1, u8:s8:bf16, false, f32, , , x, true, false, false, 2.0, 0.0", "alpha"),
    ("128, 256, 64, 1, bf16:s8:bf16", "without src_dynamic_quant"),
])
def test_unsupported_lines_are_reported(line, why):
    r = B.unsupported_reason(B.parse_line(line))
    assert r is not None and why.split()[0] in r
    assert "unimplemented" in B.run_config(B.parse_line(line))[1]


def test_result_row_has_the_reference_columns():
    c = B.parse_line("16, 128, 64, 4, u8:s8:bf16")
    cols = B.row(c, 2.0, "success").split(", ")
    assert len(cols) == len(B.HEADER.split(", "))
    assert cols[0] == "16" and cols[-1] == "success" and float(cols[-3]) == 0.5


@pytest.mark.gpu
def test_lines_run_on_the_gpu(tmp_path):
    p = tmp_path / "inputs.txt"
    p.write_text("# decode, prefill, pipeline, unsupported\n"
                 "4, 512, 256, 3, bf16:s8:bf16, false, f32, , , aocl_dlp, true, false, false, 1.0, 0.0, per-channel, , f32, 1, true, per-token, 0, f32\n"
                 "200, 256, 384, 3, u8:s8:bf16, true, f32, relu\n"
                 "64, 256, 128:64, 2, bf16:s8:bf16, true, f32, gelu_tanh, , , true, false, true, 1.0, 0.0, per-channel, , f32, 0, true, per-token\n"
                 "64, 256, 128, 2, f32:f32:f32\n")
    cfgs = B.parse_file(str(p))
    assert len(cfgs) == 4
    results = [B.run_config(c, "warm", 2) for c in cfgs]
    assert [r[1] for r in results[:3]] == ["success"] * 3, results
    assert all(r[0] > 0 for r in results[:3])
    assert results[3][1].startswith("unimplemented")


def _u16(a):
    return a.view(np.uint16) if a.dtype == np.int16 else a


@pytest.mark.gpu
def test_matmul_lines_compute_what_the_oracle_computes(oracle):
    """The driver's operands and results of each line against the oracle's statement of the same matmul_direct call:
    static u8 + zero point with bias and relu; dynamic per-token bf16 source with gelu_tanh; a transposed weight with a
    dense binary_add operand; a two-layer pipeline whose second layer quantises the first layer's bf16 output."""
    from helpers import assert_bf16_close
    lines = ["200, 256, 384, 2, u8:s8:bf16, true, f32, relu",
             "37, 512, 256, 2, bf16:s8:bf16, true, f32, gelu_tanh, , , true, false, true, 1.0, 0.0, per-channel, , f32, 0, true, per-token",
             "64, 256, 128, 2, s8:s8:f32, false, f32, binary_add, , , true, false, true",
             "64, 256, 128:64, 2, bf16:s8:bf16, true, f32, gelu_tanh, , , true, false, true, 1.0, 0.0, per-channel, , f32, 0, true, per-token"]
    lines.append("70, 256, 128:64, 2, bf16:bf16:bf16, true, f32, gelu_tanh")
    lines.append("96, 256, 128, 2, u8:s8:bf16, true, f32, relu, , , true, true, false")           # transposed source
    for line in lines:
        cfg, cap = B.parse_line(line), {}
        total, status = B.run_config(cfg, capture=cap)
        assert status == "success" and total > 0, (line, status)
        src = _u16(cap["x"])
        if cfg["transA"]:
            src = np.ascontiguousarray(src.T)
        for li, L in enumerate(cap["layers"]):
            w = L["w"].T if cfg["transB"] else L["w"]
            if cfg["wdt"] == "bf16":
                ref = oracle.matmul_bf16(src, np.ascontiguousarray(_u16(w)), "bf16", bias=L["bias"], postops=L["pos"])
                src = _u16(L["out"])
                assert_bf16_close(src, ref, 1, "%s (layer %d)" % (line, li), atol=1e-4)
                continue
            if cfg["dyn"] or li > 0:
                qa, sa = oracle.quant_per_token(src if src.dtype != np.float32 else src)
                kw = dict(src_scale=sa)
            else:
                qa, kw = src, dict(src_scale=cap["sscale"], src_zp=cap["szp"] or 0)
            pos = [dict(p, buff=_u16(p["buff"])) if isinstance(p, dict) else p for p in L["pos"]]
            ws = _u16(L["wscale"])
            ws = oracle.bf16_to_f32(ws) if ws.dtype == np.uint16 else ws
            bias = None if L["bias"] is None else _u16(L["bias"])
            bias = oracle.bf16_to_f32(bias) if bias is not None and bias.dtype == np.uint16 else bias
            ref = oracle.matmul_w8a8(qa, np.ascontiguousarray(w), L["ddt"], wei_scale=ws, bias=bias, postops=pos, **kw)
            got = _u16(L["out"])
            if L["ddt"] == "bf16":
                assert_bf16_close(got, ref, 1, "%s (layer %d)" % (line, li), atol=1e-5)
            else:
                assert np.allclose(got, ref, rtol=1e-5, atol=1e-5), line
            src = got          # the next layer of a pipeline reads this layer's output


def test_parse_grp_lines():
    c = B.parse_grp_line("8, 14:5:6:7:4:22:2:4, 4096, 28672, 200, bf16:bf16:bf16, true, 50, 2, 1, 4096")
    assert c["ops"] == 8 and c["M"] == [14, 5, 6, 7, 4, 22, 2, 4] and (c["topk"], c["act"], c["n_down"]) == (2, 1, 4096)
    assert B.grp_unsupported_reason(c) is None            # the reference's shipped traces run as written
    c["wdt"] = "f32"
    assert "weights f32" in B.grp_unsupported_reason(c)
    c["wdt"] = "s8"
    assert B.grp_unsupported_reason(c) is None
    u = B.parse_grp_line("4, 32, 2880, 5760, 200, bf16:s8:bf16, true, 50, 4, 3, 2880, 1, 32")
    assert u["M"] == [32] * 4 and u["total_experts"] == 32 and B.grp_unsupported_reason(u) is None
    t = B.parse_grp_line("9, 9:32:1:1:18:5:32:12:18, 2880, 5760, 100, bf16:bf16:bf16, true, 20, 4, 3, 2880, 1, 32  # freq=4")
    assert t["total_experts"] == 32 and t["M"][1] == 32 and B.grp_unsupported_reason(t) is None     # trailing comment of the shipped traces
    plain = B.parse_grp_line("8, 4, 4096, 14336, 200, bf16:s8:bf16, true, 50")
    assert "fused" in B.grp_unsupported_reason(plain)
    assert B.parse_grp_line("# comment") is None
    with pytest.raises(ValueError):
        B.parse_grp_line("8, 1:2:3, 4096, 28672, 200, bf16:s8:bf16, true, 50")
    assert len(B.grp_row(c, 3.0, "success").split(", ")) == len(B.GRP_HEADER.split(", "))


@pytest.mark.gpu
def test_grp_lines_run_on_the_gpu():
    for line in ("4, 10:0:7:3, 256, 512, 2, bf16:s8:bf16, true, 1, 2, 1, 256",
                 "3, 8, 128, 256, 2, bf16:s8:bf16, true, 0, 0, 3, 128",
                 "4, 10:0:7:3, 256, 512, 2, bf16:bf16:bf16, true, 1, 2, 1, 256",
                 "3, 8, 128, 256, 2, bf16:bf16:bf16, true, 0, 0, 3, 128"):
        total, status = B.run_grp_config(B.parse_grp_line(line))
        assert status == "success" and total > 0, (line, status)


def test_parse_reorder_lines():
    c = B.parse_reorder_line("1, 2048, 512, 50, bf16, s8, reference, per_channel_row, 0, true, 0, 10")
    assert (c["rows"], c["cols"], c["sdt"], c["ddt"], c["gran"], c["dyn"], c["warmup"]) == (2048, 512, "bf16", "s8", "per_channel_row", True, 10)
    assert B.reorder_unsupported_reason(c) is None
    assert B.parse_reorder_line("1, 64, 64, 10, f32, s8, reference, per_tensor, 0, false")["warmup"] == 2
    for line, why in (("4, 1024, 768, 100, f32, u8, reference, per_group_col, 128, false, 8, 20", "batched"),
                      ("1, 1024, 768, 100, f32, u8, reference, per_group_col, 128, false, 8, 20", "granularity"),
                      ("1, 2048, 1024, 100, f16, s8, native, per_channel_row, 0, true, 0, 20", "f16"),
                      ("1, 4096, 4096, 50, f32, u8, reference, per_channel_col, 0, true, 0, 10", "dynamic")):
        r = B.reorder_unsupported_reason(B.parse_reorder_line(line))
        assert r is not None and why in r, (line, r)
    with pytest.raises(ValueError):
        B.parse_reorder_line("1, 64, 64")
    assert len(B.reorder_row(c, 1.0, "success").split(", ")) == len(B.REORDER_HEADER.split(", "))


@pytest.mark.gpu
def test_reorder_lines_run_on_the_gpu():
    for line in ("1, 300, 520, 3, bf16, s8, reference, per_channel_row, 0, true, 0, 1",
                 "1, 256, 384, 3, f32, s8, reference, per_channel_col, 0, true, 0, 1",
                 "1, 256, 384, 3, f32, s8, reference, per_tensor, 0, true, 0, 1",
                 "1, 128, 256, 3, f32, u8, reference, per_tensor, 0, false, 0, 1",
                 "1, 128, 256, 3, s8, bf16, native, per_channel_col, 0, false, 0, 1"):
        total, status = B.run_reorder_config(B.parse_reorder_line(line))
        assert status == "success" and total > 0, (line, status)
