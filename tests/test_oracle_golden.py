"""The CPU oracle against fixtures produced by the reference's own functions, and known-answer properties."""
import os

import numpy as np
import pytest
import torch

import tb_oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", ["w_small", "w_ragged", "w_wide", "w_tiny_scale"])
def test_quantize_matches_reference_fixture(name):
    z = np.load(os.path.join(GOLDEN, "nvfp4_quantize.npz"))
    w = torch.from_numpy(z[f"{name}.w_bf16_bits"]).view(torch.bfloat16)
    packed, scale, gs = orc.quantize_nvfp4(w)
    assert np.array_equal(packed, z[f"{name}.packed"])
    assert np.array_equal(scale, z[f"{name}.scale"])
    assert np.array_equal(gs.view(np.uint32), z[f"{name}.global_scale"].view(np.uint32))


def test_prefold_exact_matches_reference_fixture():
    z = np.load(os.path.join(GOLDEN, "prefold_exact.npz"))
    assert np.array_equal(orc.prefold(z["raw"], "exact"), z["prefolded"])


def test_recode_snc_matches_reference_fixture():
    z = np.load(os.path.join(GOLDEN, "recode_snc.npz"))
    p = z["packed"]
    got = orc.recode_snc(p & 0xF) | (orc.recode_snc(p >> 4) << 4)
    assert np.array_equal(got, z["recoded"])


def test_share_global_scale_matches_reference_fixture():
    z = np.load(os.path.join(GOLDEN, "share_global_scale.npz"))
    out, shared = orc.share_global_scale(z["weight_scale"], z["global_scales"], z["shard_sizes"])
    assert np.array_equal(out, z["out_scale"])
    assert np.array_equal(shared, z["shared"])


def _all_code_scale_pairs():
    raws = np.arange(0x1C, 0x7F, dtype=np.int16)
    codes = np.tile(np.arange(16, dtype=np.uint8), (raws.size, 1))  # one group of 16 = all 16 codes
    return codes, raws.reshape(-1, 1)


@pytest.mark.parametrize("bridge", ["exact", "fpma"])
def test_closed_form_equals_device_table_lookup(bridge):
    codes, raw = _all_code_scale_pairs()
    assert np.array_equal(orc.bridge_bytes(codes, raw, bridge), orc.bridge_bytes_lut(codes, raw, bridge))
    assert np.array_equal(orc.bridge_bytes(codes, raw, bridge), orc.bridge_bytes_by_table(codes, raw, bridge))


def test_exact_bridge_is_rne_of_code_times_scale_over_six():
    """Known-answer property: for raw 0x23..0x7E the exact bridge byte is RNE_E4M3(code * scale / 6); below that
    only the +-0.5 codes (E4M3 subnormal results) may differ."""
    codes, raw = _all_code_scale_pairs()
    got = orc.bridge_bytes(codes, raw, "exact")
    val = orc.E2M1_VALUES[codes & 7] * np.where(codes & 8, -1.0, 1.0)
    want = orc.e4m3_encode_rne_sat((val * orc.e4m3_decode(raw.astype(np.uint8)) / 6.0).astype(np.float32))
    want = np.where((codes & 7) == 0, 0, want)  # the bridge drops the sign of zero
    diff = got != want
    assert not diff[raw[:, 0] >= 0x23].any()
    assert set((codes[diff] & 7).tolist()) <= {1}
    assert diff.sum() == 14  # 7 scales x the two signs of 0.5


def test_fpma_bridge_constants():
    """fpma byte = raw - 28 + {0.5:0, 1:8, 1.5:12, 2:16, 3:20, 4:24, 6:28}."""
    codes, raw = _all_code_scale_pairs()
    got = orc.bridge_bytes(codes, raw, "fpma")[:, :8].astype(np.int32)
    off = np.array([0, 0, 8, 12, 16, 20, 24, 28])
    want = raw.astype(np.int32) - 28 + off[None, :]
    want[:, 0] = 0
    assert np.array_equal(got, want)


def test_checkpoint_rules():
    packed = np.full((8, 16), 0x77, np.uint8)  # K = 32: two groups per row
    raw = np.full((8, 2), 0x40, np.uint8)
    raw[0, 0] = 0x1B  # below range: zeroed
    codes, r = orc.checkpoint_to_padded(packed, raw)
    assert codes.shape == (128, 128) and r.shape == (128, 8)
    assert (codes[0, :16] == 0).all() and r[0, 0] == 0 and (codes[0, 16:32] == 7).all()
    assert (codes[8:] == 0).all() and (codes[:, 32:] == 0).all() and (r[8:] == 0).all()
    fp8 = orc.bridge_bytes(codes, r, "exact")
    assert (fp8[8:] == 0).all() and (fp8[0, :16] == 0).all()
    raw[1, 1] = 0x7F
    with pytest.raises(ValueError):
        orc.checkpoint_to_padded(packed, raw)
    _, r2 = orc.checkpoint_to_padded(packed, raw, clamp_scale=True)
    assert r2[1, 1] == 0x7E
    with pytest.raises(ValueError):
        orc.checkpoint_to_padded(np.zeros((4, 8), np.uint8), np.zeros((4, 1), np.uint8))  # N % 8


def test_e4m3_codec_roundtrip():
    b = np.arange(256, dtype=np.uint8)
    b = b[(b & 0x7F) != 0x7F]
    v = orc.e4m3_decode(b)
    assert np.array_equal(orc.e4m3_encode_rne_sat(v), b)
    assert orc.e4m3_encode_rne_sat(np.array([1e9, -1e9], np.float32)).tolist() == [0x7E, 0xFE]
    t = torch.from_numpy(b.copy()).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(t, v)


def test_activation_quantizers():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 300, generator=g).bfloat16()
    x[2] = 0
    q, s = orc.quantize_fp8_per_token(x)
    assert q.shape == (5, 300) and s.shape == (5, 1)
    assert s[2, 0] == np.float32(1e-30) / np.float32(448) and (q[2] == 0).all()
    assert (q[0] & 0x7F).max() == 0x7E  # the row maximum maps to 448
    back = orc.e4m3_decode(q) * s
    assert np.abs(back - x.float().numpy()).max() <= np.abs(x.float().numpy()).max() * 2 ** -4
    qg, sg = orc.quantize_fp8_group128(x)
    assert sg.shape == (5, 3)
    assert (qg[0, 256:] & 0x7F).max() == 0x7E  # ragged last group has its own scale


def test_grouped_semantics_agree_with_dense():
    g = torch.Generator().manual_seed(1)
    e, n, k = 3, 128, 128
    w_fp8, gs6 = [], []
    for i in range(e):
        p, s, gs = orc.quantize_nvfp4((torch.randn(n, k, generator=g) * 0.02).bfloat16())
        v = orc.prepare_reference_view(p, s, gs)
        w_fp8.append(v["fp8"]); gs6.append(v["global_scale6"][0])
    x = torch.randn(10, k, generator=g).bfloat16()
    q, s = orc.quantize_fp8_per_token(x)
    offsets = np.array([0, 4, 4, 10])
    out = orc.gemm_contiguous(q, s, w_fp8, gs6, offsets, n, k)
    assert torch.equal(out[:4], orc.gemm_dense(q[:4], s[:4], w_fp8[0], gs6[0], n, k))
    assert torch.equal(out[4:], orc.gemm_dense(q[4:], s[4:], w_fp8[2], gs6[2], n, k))
    # indexed: 5 tokens, top-2
    topk = np.array([[0, 2], [1, 2], [0, 1], [2, 0], [1, 0]])
    sid, eid, npad = orc.align_routes(topk, e, 4)
    assert npad[0] == sid.size and sid.size % 4 == 0 and eid.size == sid.size // 4
    out_i, valid = orc.gemm_indexed(q[:5], s[:5], w_fp8, gs6, sid, eid, npad[0], 4, 2, n, k)
    assert valid.all()
    for r in range(10):
        ex = topk.reshape(-1)[r]
        assert torch.equal(out_i[r], orc.gemm_dense(q[r // 2:r // 2 + 1], s[r // 2:r // 2 + 1], w_fp8[ex], gs6[ex], n, k)[0])
    # group scales with all-equal scales reduce to the per-token result up to fp32 summation order
    qg, sg = orc.quantize_fp8_group128(x)
    o1 = orc.gemm_dense_group_scales(qg, sg, w_fp8[0], gs6[0], n, k)
    o2 = orc.gemm_dense(qg, sg[:, :1], w_fp8[0], gs6[0], n, k)
    assert torch.equal(o1, o2)  # K = 128: one group


def test_table_dequant_equals_closed_form():
    g = torch.Generator().manual_seed(5)
    p, sc, gs = orc.quantize_nvfp4((torch.randn(72, 208, generator=g) * 0.02).bfloat16())
    for bridge in ("exact", "fpma"):
        v = orc.prepare_reference_view(p, sc, gs, bridge=bridge)
        fast = orc.dequant_weight_f32(v["codes"], v["raw"], bridge).numpy()
        assert np.array_equal(fast, orc.e4m3_decode(v["fp8"]))
        assert np.array_equal(v["fp8"], orc.bridge_bytes(v["codes"], v["raw"], bridge))  # the view's gather == closed form
