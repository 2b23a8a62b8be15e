"""GPU parity, part 4: the fused MoE producers (masked / bounded / scattered quantisers, SiLU-mul quantiser, FP8 scatter)
and the `moe_forward_*` orchestrators, each stage checked against the oracle fed with the stage's own GPU input so a
one-step BF16 rounding difference in a GEMM cannot cascade into the next comparison."""
import numpy as np
import pytest
import torch

import tb_oracle as orc
from helpers import seeded_activations, seeded_weight

pytestmark = pytest.mark.gpu

SENTINEL_Q = 0x55
SENTINEL_S = -7.0


def _out(rows, width, groups):
    q = torch.full((rows, width), SENTINEL_Q, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    s = torch.full((rows, groups), SENTINEL_S, dtype=torch.float32, device="cuda")
    return q, s


def _bytes(q):
    return q.view(torch.uint8).cpu().numpy()


def _check_rows(q, s, want_q, want_s, valid, exact=True):
    got_q, got_s = _bytes(q), s.cpu().numpy()
    if exact:
        assert np.array_equal(got_q[valid], want_q[valid])
        assert np.array_equal(got_s[valid], want_s[valid])
    else:  # expf may differ from the host's exp in the last place: a handful of BF16 values, hence codes, may move
        assert np.mean(got_q[valid] != want_q[valid]) <= 2e-3
        np.testing.assert_allclose(got_s[valid], want_s[valid], rtol=2 ** -7)
    assert (got_q[~valid] == SENTINEL_Q).all() and (got_s[~valid] == SENTINEL_S).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("mode", ["per_token", "group_128"])
@pytest.mark.parametrize("width", [128, 384, 1000, 7168])
def test_quantize_moe_masked(mode, width, dtype):
    from tensorbridge.quant import fp8
    counts = [3, 0, 6, 1]
    capacity = 5  # count 6 exceeds the capacity: every row of that block is valid, none beyond it
    x = seeded_activations(len(counts) * capacity, width, seed=11).to(dtype)
    groups = -(-width // 128) if mode == "group_128" else 1
    out = _out(x.size(0), width, groups)
    fp8.quantize_moe(x.cuda(), mode, expert_counts=torch.tensor(counts, dtype=torch.int32, device="cuda"), out=out)
    want_q, want_s = orc.quantize_rows(x.float().numpy(), mode == "group_128", use_division=True)
    valid = np.concatenate([np.arange(capacity) < c for c in counts])
    _check_rows(*out, want_q, want_s, valid)


@pytest.mark.parametrize("bound_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("mode", ["per_token", "group_128"])
def test_quantize_moe_bounded_and_strided(mode, bound_dtype):
    from tensorbridge.quant import fp8
    rows, width = 37, 512
    wide = seeded_activations(rows, width + 64, seed=12)
    x = wide.cuda()[:, 8:8 + width]  # row stride != width, rows 16-byte aligned
    groups = width // 128 if mode == "group_128" else 1
    out = _out(rows, width, groups)
    fp8.quantize_moe(x, mode, num_valid_rows=torch.tensor([21], dtype=bound_dtype, device="cuda"), out=out)
    want_q, want_s = orc.quantize_rows(wide[:, 8:8 + width].float().numpy(), mode == "group_128", use_division=True)
    _check_rows(*out, want_q, want_s, np.arange(rows) < 21)
    odd = wide.cuda()[:, 3:3 + width]  # rows that are not 16-byte aligned take the scalar loads
    out = _out(rows, width, groups)
    fp8.quantize_moe(odd, mode, out=out)
    want_q, want_s = orc.quantize_rows(wide[:, 3:3 + width].float().numpy(), mode == "group_128", use_division=True)
    _check_rows(*out, want_q, want_s, np.ones(rows, bool))


def _gate_up(rows, inter, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, 2 * inter, generator=g) * 2.5).bfloat16()


@pytest.mark.parametrize("inter", [128, 200, 2048])
def test_silu_mul_quantize(inter):
    from tensorbridge.quant import fp8
    rows = 19
    gu = _gate_up(rows, inter, seed=13)
    want_q, want_s = orc.quantize_rows(orc.silu_mul_bf16(gu), False, use_division=False)
    q, s = fp8.silu_mul_quantize(gu.cuda())
    assert tuple(q.shape) == (rows, inter) and tuple(s.shape) == (rows, 1)
    got_q, got_s = _bytes(q), s.cpu().numpy()
    assert np.mean(got_q != want_q) <= 2e-3
    np.testing.assert_allclose(got_s, want_s, rtol=2 ** -7)
    # against torch's own BF16 ops on the same device the scale (a pure max) must agree exactly
    gpu = gu.cuda()
    act = torch.nn.functional.silu(gpu[:, :inter]) * gpu[:, inter:]
    amax = act.float().abs().amax(dim=1, keepdim=True).cpu().numpy()
    assert np.array_equal(s.cpu().numpy(), np.maximum(amax, np.float32(1e-30)) / np.float32(448.0))
    for dtype in (torch.int32, torch.int64):
        out = _out(rows, inter, 1)
        fp8.silu_mul_quantize(gu.cuda(), torch.tensor([7], dtype=dtype, device="cuda"), out=out)
        _check_rows(*out, want_q, want_s, np.arange(rows) < 7, exact=False)


@pytest.mark.parametrize("mode", ["per_token", "group_128"])
def test_quantize_moe_activation_masked(mode):
    from tensorbridge.quant import fp8
    counts, capacity, inter = [2, 4, 0], 4, 384
    gu = _gate_up(len(counts) * capacity, inter, seed=14)
    groups = inter // 128 if mode == "group_128" else 1
    out = _out(gu.size(0), inter, groups)
    fp8.quantize_moe(gu.cuda(), mode, activation=True,
                     expert_counts=torch.tensor(counts, dtype=torch.int32, device="cuda"), out=out)
    want_q, want_s = orc.quantize_rows(orc.silu_mul_bf16(gu), mode == "group_128", use_division=True)
    valid = np.concatenate([np.arange(capacity) < c for c in counts])
    _check_rows(*out, want_q, want_s, valid, exact=False)
    with pytest.raises(ValueError):
        fp8.quantize_moe(gu.cuda().float(), mode, activation=True, out=out)


def _scatter_case(tokens, top_k, out_rows, seed):
    """Distinct targets per route; about a quarter fall outside [0, out_rows) as routes to other ranks' experts do."""
    rng = np.random.default_rng(seed)
    targets = rng.permutation(out_rows + out_rows // 2)[:tokens * top_k].astype(np.int32)
    targets[targets >= out_rows] = np.where(rng.random(int((targets >= out_rows).sum())) < 0.5, -1, out_rows + 3)
    return targets.reshape(tokens, top_k)


@pytest.mark.parametrize("tokens,top_k,width", [(1, 1, 128), (13, 2, 256), (40, 4, 7168)])
def test_scatter_quantize(tokens, top_k, width):
    from tensorbridge.quant import fp8
    out_rows = tokens * top_k
    idx = _scatter_case(tokens, top_k, out_rows, seed=tokens)
    x = seeded_activations(tokens, width, seed=15)
    out = _out(out_rows, width, 1)
    fp8.scatter_quantize(x.cuda(), torch.from_numpy(idx).cuda(), out_rows, out=out)
    tok_q, tok_s = orc.quantize_fp8_per_token(x)
    want_q = np.zeros((out_rows, width), np.uint8)
    want_s = np.zeros((out_rows, 1), np.float32)
    valid = np.zeros(out_rows, bool)
    for t in range(tokens):
        for j in range(top_k):
            r = idx[t, j]
            if 0 <= r < out_rows:
                want_q[r], want_s[r], valid[r] = tok_q[t], tok_s[t], True
    _check_rows(*out, want_q, want_s, valid)


@pytest.mark.parametrize("groups", [1, 4])
def test_scatter_fp8_and_group_scatter(groups):
    from tensorbridge.quant import fp8
    tokens, top_k, width = 21, 3, 512
    out_rows = tokens * top_k
    idx = _scatter_case(tokens, top_k, out_rows, seed=99)
    x = seeded_activations(tokens, width, seed=16)
    if groups == 1:
        q_in, s_in = fp8.quantize(x.cuda())
    else:
        q_in, s_in = fp8.quantize_group_128(x.cuda())  # M-major scales: strides are honoured
    out = _out(out_rows, width, groups)
    fp8.scatter_fp8(q_in, s_in, torch.from_numpy(idx).cuda(), out=out)
    want_q = np.zeros((out_rows, width), np.uint8)
    want_s = np.zeros((out_rows, groups), np.float32)
    valid = np.zeros(out_rows, bool)
    src_q, src_s = _bytes(q_in), s_in.cpu().numpy()
    for t in range(tokens):
        for r in idx[t]:
            if 0 <= r < out_rows:
                want_q[r], want_s[r], valid[r] = src_q[t], src_s[t], True
    _check_rows(*out, want_q, want_s, valid)
    if groups == 4:  # the fused group-128 quantise + scatter writes the same rows with division rounding
        out2 = _out(out_rows, width, groups)
        fp8.quantize_moe(x.cuda(), "group_128", scatter_idx=torch.from_numpy(idx).cuda(), out=out2)
        tok_q, tok_s = orc.quantize_rows(x.float().numpy(), True, use_division=True)
        for t in range(tokens):
            for r in idx[t]:
                if 0 <= r < out_rows:
                    want_q[r], want_s[r] = tok_q[t], tok_s[t]
        _check_rows(*out2, want_q, want_s, valid)


# ---- moe_forward_* ------------------------------------------------------------------------------------------

E, H, I, TOP_K = 4, 256, 128, 2


def _layer(layout, quant, bridge="exact"):
    """A gated layer quantised by the oracle; gate and up halves carry different global scales, so preparing it
    exercises the shared-scale rewrite.  Returns the prepared layer and the oracle's operand views per expert."""
    from tensorbridge import serving
    p13, s13, g13, p2, s2, g2, views13, views2 = [], [], [], [], [], [], [], []
    for e in range(E):
        gate = orc.quantize_nvfp4(seeded_weight(I, H, seed=700 + e, std=0.05))
        up = orc.quantize_nvfp4(seeded_weight(I, H, seed=800 + e, std=0.02))
        down = orc.quantize_nvfp4(seeded_weight(H, I, seed=900 + e, std=0.05))
        packed = np.concatenate([gate[0], up[0]])
        scale = np.concatenate([gate[1], up[1]])
        gs = np.array([gate[2][0], up[2][0]], np.float32)
        shared_scale, shared_gs = orc.share_global_scale(scale, gs, [I, I])
        views13.append(orc.prepare_reference_view(packed, shared_scale, np.asarray(shared_gs, np.float32).reshape(1), bridge=bridge))
        views2.append(orc.prepare_reference_view(down[0], down[1], down[2], bridge=bridge))
        p13.append(packed), s13.append(scale), g13.append(gs), p2.append(down[0]), s2.append(down[1]), g2.append(down[2][0])
    cuda = lambda xs, dt=None: torch.from_numpy(np.stack(xs)).cuda() if dt is None else torch.from_numpy(np.stack(xs)).cuda().view(dt)
    moe = serving.prepare_moe(cuda(p13), cuda(s13, torch.float8_e4m3fn), cuda(g13), cuda(p2), cuda(s2, torch.float8_e4m3fn),
                              torch.tensor(g2, dtype=torch.float32, device="cuda"), TOP_K, bridge=bridge, layout=layout,
                              scale_convention="multiplier", gate_up_quant=quant, down_quant=quant)
    return moe, views13, views2


def _buffers(moe, tokens):
    from tensorbridge import serving
    bufs = {}
    for name, (shape, dtype) in serving.moe_buffer_specs(moe, tokens).items():
        if dtype == torch.float8_e4m3fn:
            bufs[name] = torch.full(shape, SENTINEL_Q, dtype=torch.uint8, device="cuda").view(dtype)
        else:
            bufs[name] = torch.full(shape, SENTINEL_S, dtype=dtype, device="cuda")
    return bufs


def _close(got, want, valid):
    g = got.float().cpu()[torch.from_numpy(valid)]
    w = want.float()[torch.from_numpy(valid)]
    if w.numel():
        assert float((g - w).norm() / w.norm().clamp_min(1e-30)) <= 2e-3
        assert float((g - w).abs().max()) <= float(w.abs().max()) * 2 ** -6


def _stagewise(bufs, views13, views2, group, grouped_oracle, valid, act_division):
    """gate_up against the oracle GEMM of the GPU's quantised input; intermediate against the oracle activation of the
    GPU's gate_up; output against the oracle GEMM of the GPU's intermediate."""
    fp8_13, gs13 = [v["fp8"] for v in views13], [v["global_scale6"][0] for v in views13]
    fp8_2, gs2 = [v["fp8"] for v in views2], [v["global_scale6"][0] for v in views2]
    want_gu = grouped_oracle(_bytes(bufs["input"]), bufs["input_scale"].cpu().numpy(), fp8_13, gs13, 2 * I, H)
    _close(bufs["gate_up"], want_gu, valid)
    gu = bufs["gate_up"].cpu()
    gu[torch.from_numpy(~valid)] = 0  # unwritten rows hold the sentinel
    want_q, want_s = orc.quantize_rows(orc.silu_mul_bf16(gu), group, use_division=act_division)
    got_q, got_s = _bytes(bufs["intermediate"]), bufs["intermediate_scale"].cpu().numpy()
    assert np.mean(got_q[valid] != want_q[valid]) <= 2e-3
    np.testing.assert_allclose(got_s[valid], want_s[valid], rtol=2 ** -7)
    assert (got_q[~valid] == SENTINEL_Q).all()
    inter_q = np.where(valid[:, None], got_q, 0)
    inter_s = np.where(valid[:, None], got_s, 0).astype(np.float32)
    want_out = grouped_oracle(inter_q, inter_s, fp8_2, gs2, H, I)
    _close(bufs["output"], want_out, valid)


@pytest.mark.parametrize("quant", ["per_token", "group_128"])
def test_moe_forward_masked(quant):
    import tensorbridge as tb
    from tensorbridge import serving
    moe, v13, v2 = _layer("masked", quant)
    capacity, counts = 12, [5, 12, 0, 1]
    x = seeded_activations(E * capacity, H, seed=21)
    bufs = _buffers(moe, capacity)
    routing = tb.MaskedRouting(torch.tensor(counts, dtype=torch.int32, device="cuda"))
    out = serving.moe_forward_masked(moe, x.cuda(), routing, bufs, num_routes=sum(counts))
    tb.check_status()
    assert out.data_ptr() == bufs["output"].data_ptr()
    valid = np.concatenate([np.arange(capacity) < c for c in counts])
    want_q, want_s = orc.quantize_rows(x.float().numpy(), quant == "group_128", use_division=True)
    assert np.array_equal(_bytes(bufs["input"])[valid], want_q[valid])
    assert np.array_equal(bufs["input_scale"].cpu().numpy()[valid], want_s[valid])
    group = quant == "group_128"
    oracle = lambda q, s, w, g, n, k: orc.gemm_masked(np.where(valid[:, None], q, 0), np.where(valid[:, None], s, 0).astype(np.float32),
                                                      w, g, counts, n, k, group)[0]
    _stagewise(bufs, v13, v2, group, oracle, valid, act_division=True)
    assert bool((bufs["output"].float().cpu()[torch.from_numpy(~valid)] == SENTINEL_S).all())


@pytest.mark.parametrize("prequantised", [False, True])
@pytest.mark.parametrize("quant", ["per_token", "group_128"])
def test_moe_forward_contiguous(quant, prequantised):
    import tensorbridge as tb
    from tensorbridge import serving
    from tensorbridge.quant import fp8
    moe, v13, v2 = _layer("contiguous", quant)
    tokens = 11
    rng = np.random.default_rng(5)
    topk = np.stack([rng.choice(E + 2, size=TOP_K, replace=False) for _ in range(tokens)])  # experts E, E+1: other ranks
    local = topk < E
    order = np.argsort(np.where(local, topk, E).reshape(-1), kind="stable")
    rows = int(local.sum())
    scatter = np.full(tokens * TOP_K, -1, np.int32)
    scatter[order[:rows]] = np.arange(rows, dtype=np.int32)
    scatter = scatter.reshape(tokens, TOP_K)
    counts = np.bincount(topk[local], minlength=E)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    x = seeded_activations(tokens, H, seed=22)
    bufs = _buffers(moe, tokens)
    routing = tb.ContiguousRouting(torch.from_numpy(offsets).cuda())
    group = quant == "group_128"
    if prequantised:
        q_in, s_in = (fp8.quantize_group_128 if group else fp8.quantize)(x.cuda())
        out = serving.moe_forward_contiguous(moe, q_in, torch.from_numpy(scatter).cuda(), routing, bufs, input_scale=s_in)
        tok_q, tok_s = _bytes(q_in), s_in.cpu().numpy()
    else:
        out = serving.moe_forward_contiguous(moe, x.cuda(), torch.from_numpy(scatter).cuda(), routing, bufs)
        tok_q, tok_s = orc.quantize_rows(x.float().numpy(), group, use_division=group)
    tb.check_status()
    capacity = tokens * TOP_K
    valid = np.arange(capacity) < rows
    for t in range(tokens):
        for j in range(TOP_K):
            if scatter[t, j] >= 0:
                assert np.array_equal(_bytes(bufs["input"])[scatter[t, j]], tok_q[t])
                assert np.array_equal(bufs["input_scale"].cpu().numpy()[scatter[t, j]], tok_s[t])
    def oracle(q, s, w, g, n, k):
        full = torch.zeros((capacity, n), dtype=torch.bfloat16)
        full[:rows] = orc.gemm_contiguous(q[:rows], s[:rows], w, g, offsets, n, k, group)
        return full
    _stagewise(bufs, v13, v2, group, oracle, valid, act_division=group)
    assert out.data_ptr() == bufs["output"].data_ptr()


@pytest.mark.parametrize("quant", ["per_token", "group_128"])
def test_moe_forward_indexed(quant):
    import tensorbridge as tb
    from tensorbridge import routing as tb_routing
    from tensorbridge import serving
    moe, v13, v2 = _layer("indexed", quant)
    tokens, block_m = 23, 16
    rng = np.random.default_rng(6)
    topk = np.stack([rng.choice(E, size=TOP_K, replace=False) for _ in range(tokens)])
    sid, eid, npad = orc.align_routes(topk, E, block_m)
    dev = lambda a: torch.from_numpy(a).cuda()
    routing13 = tb.IndexedRouting(dev(sid), dev(eid), dev(npad), block_m, TOP_K)
    routing2 = tb.IndexedRouting(dev(sid), dev(eid), dev(npad), block_m, 1)
    x = seeded_activations(tokens, H, seed=23)
    bufs = _buffers(moe, tokens)
    import dataclasses
    cfg = tb.GemmConfig(block_m=block_m, num_stages=4, stream_k_aligned=3)
    moe = dataclasses.replace(moe, configs=(cfg, cfg))
    out = serving.moe_forward_indexed(moe, x.cuda(), routing13, routing2, bufs)
    tb.check_status()
    group = quant == "group_128"
    want_q, want_s = orc.quantize_rows(x.float().numpy(), group, use_division=group)
    assert np.array_equal(_bytes(bufs["input"]), want_q)
    assert np.array_equal(bufs["input_scale"].cpu().numpy(), want_s)
    routes = tokens * TOP_K
    valid = np.ones(routes, bool)
    fp8_13, gs13 = [v["fp8"] for v in v13], [v["global_scale6"][0] for v in v13]
    want_gu, written = orc.gemm_indexed(want_q, want_s, fp8_13, gs13, sid, eid, int(npad[0]), block_m, TOP_K, 2 * I, H, group)
    assert written.all()
    _close(bufs["gate_up"], want_gu, valid)
    iq, isc = orc.quantize_rows(orc.silu_mul_bf16(bufs["gate_up"].cpu()), group, use_division=group)
    got_q, got_s = _bytes(bufs["intermediate"]), bufs["intermediate_scale"].cpu().numpy()
    assert np.mean(got_q != iq) <= 2e-3
    np.testing.assert_allclose(got_s, isc, rtol=2 ** -7)
    fp8_2, gs2 = [v["fp8"] for v in v2], [v["global_scale6"][0] for v in v2]
    want_out, _ = orc.gemm_indexed(got_q, got_s, fp8_2, gs2, sid, eid, int(npad[0]), block_m, 1, H, I, group)
    _close(out, want_out, valid)
    # weighting and summing the top-k outputs is the caller's step; against a float reference of the whole layer the
    # result must agree to quantisation accuracy
    w13 = [orc.e4m3_decode(v["fp8"][:2 * I, :H]) * v["global_scale6"][0] for v in v13]
    w2 = [orc.e4m3_decode(v["fp8"][:H, :I]) * v["global_scale6"][0] for v in v2]
    xf = x.float().numpy()
    ref = np.zeros((routes, H), np.float32)
    for t in range(tokens):
        for j in range(TOP_K):
            e = topk[t, j]
            gu = xf[t] @ w13[e].T
            act = gu[:I] / (1 + np.exp(-gu[:I])) * gu[I:]
            ref[t * TOP_K + j] = act @ w2[e].T
    err = np.linalg.norm(out.float().cpu().numpy() - ref) / np.linalg.norm(ref)
    assert err <= 0.08, err
    assert tb_routing.padded_capacity(routes, E, block_m) >= int(npad[0])


def test_moe_forward_errors():
    import tensorbridge as tb
    from tensorbridge import serving
    moe, _, _ = _layer("masked", "per_token")
    bufs = _buffers(moe, 4)
    x = seeded_activations(E * 4, H, seed=1).cuda()
    offsets = torch.zeros(E + 1, dtype=torch.int64, device="cuda")
    with pytest.raises(ValueError):
        serving.moe_forward_contiguous(moe, x, torch.zeros((4, TOP_K), dtype=torch.int32, device="cuda"),
                                       tb.ContiguousRouting(offsets), bufs)
    import dataclasses
    ungated = dataclasses.replace(moe, is_gated=False)
    with pytest.raises(ValueError):
        serving.moe_forward_masked(ungated, x, tb.MaskedRouting(torch.zeros(E, dtype=torch.int32, device="cuda")), bufs)
    specs = serving.moe_buffer_specs(moe, 4, unfused_activation=True)
    assert specs["activated"] == ((E * 4, I), torch.bfloat16) and specs["input"][0] == (E * 4, H)
    assert serving.moe_rows(dataclasses.replace(moe, num_global_experts=8), 64) == 32


def test_moe_forward_custom_activation():
    """`activation_fn` replaces the fused SiLU-mul: with the same function the result must match the fused path's."""
    import tensorbridge as tb
    from tensorbridge import serving
    moe, _, _ = _layer("masked", "per_token")
    capacity, counts = 8, [8, 3, 0, 5]
    x = seeded_activations(E * capacity, H, seed=24).cuda()
    routing = tb.MaskedRouting(torch.tensor(counts, dtype=torch.int32, device="cuda"))
    fused = _buffers(moe, capacity)
    serving.moe_forward_masked(moe, x, routing, fused)
    custom = _buffers(moe, capacity)
    custom["gate_up"].zero_()

    def act(out, gate_up):
        assert out.dim() == 3 and gate_up.dim() == 3
        torch.mul(torch.nn.functional.silu(gate_up[..., :I]), gate_up[..., I:], out=out)

    serving.moe_forward_masked(moe, x, routing, custom, activation_fn=act)
    tb.check_status()
    valid = torch.from_numpy(np.concatenate([np.arange(capacity) < c for c in counts]))
    a, b = fused["output"].float().cpu()[valid], custom["output"].float().cpu()[valid]
    assert float((a - b).norm() / a.norm()) <= 5e-3


@pytest.mark.parametrize("tokens,top_k,width,indexed", [(1, 1, 8, False), (37, 4, 2048, False), (300, 8, 1536, True),
                                                       (64, 2, 136, True)])
def test_combine_routes_kernel(tokens, top_k, width, indexed):
    """`tb_moe_combine` against the same sum in torch: FP32 multiply-adds in slot order, one BF16 rounding at the end;
    routes with a negative index add nothing."""
    from tensorbridge import vllm_moe
    g = torch.Generator().manual_seed(tokens + width)
    rows = torch.randn((tokens * top_k + 5, width), generator=g).bfloat16().cuda()
    weights = torch.rand((tokens, top_k), generator=g).cuda()
    index = None
    if indexed:
        index = torch.randint(-1, rows.size(0), (tokens, top_k), generator=g, dtype=torch.int32).cuda()
    got = vllm_moe.combine_routes(rows, weights, None if index is None else index.reshape(-1))
    source = rows[:tokens * top_k].view(tokens, top_k, width) if index is None else rows[index.clamp(min=0).long()]
    want = torch.zeros((tokens, width), dtype=torch.float32, device="cuda")
    for j in range(top_k):
        term = torch.addcmul(want, source[:, j].float(), weights[:, j:j + 1])  # fused multiply-add, like the kernel
        want = term if index is None else torch.where((index[:, j] >= 0).unsqueeze(1), term, want)
    close = (got.float() - want.bfloat16().float()).abs() <= want.abs() * 2 ** -7 + 1e-30
    assert bool(close.all())
    assert float((got != want.bfloat16()).float().mean()) < 1e-3  # addcmul may not fuse exactly like fmaf


@pytest.mark.parametrize("layout", ["indexed", "contiguous"])
def test_vllm_style_moe_method_without_vllm(layout):
    """The layer-level adapter: checkpoint tensors on a module -> `process_weights_after_loading` -> `apply(x, topk_weights,
    topk_ids)`.  Its output is the weighted sum of what `moe_forward_*` returns for each route (checked against those
    functions driven by hand), and agrees with a float reference of the whole layer to quantisation accuracy; with an
    `expert_map` that hides half of the experts, the hidden routes add nothing."""
    import tensorbridge as tb
    from tensorbridge import serving, vllm_moe
    _, v13, v2 = _layer(layout, "per_token")
    p13, s13, g13, p2, s2, g2 = [], [], [], [], [], []
    for e in range(E):
        gate = orc.quantize_nvfp4(seeded_weight(I, H, seed=700 + e, std=0.05))
        up = orc.quantize_nvfp4(seeded_weight(I, H, seed=800 + e, std=0.02))
        down = orc.quantize_nvfp4(seeded_weight(H, I, seed=900 + e, std=0.05))
        p13.append(np.concatenate([gate[0], up[0]])), s13.append(np.concatenate([gate[1], up[1]]))
        g13.append(np.array([gate[2][0], up[2][0]], np.float32))
        p2.append(down[0]), s2.append(down[1]), g2.append(down[2][0])
    cuda = lambda xs, dt=None: torch.from_numpy(np.stack(xs)).cuda() if dt is None else torch.from_numpy(np.stack(xs)).cuda().view(dt)
    layer = torch.nn.Module()
    layer.w13_weight, layer.w13_weight_scale, layer.w13_weight_scale_2 = cuda(p13), cuda(s13, torch.float8_e4m3fn), cuda(g13)
    layer.w2_weight, layer.w2_weight_scale = cuda(p2), cuda(s2, torch.float8_e4m3fn)
    layer.w2_weight_scale_2 = torch.tensor(g2, dtype=torch.float32, device="cuda")
    layer.w13_input_scale = torch.ones(1, device="cuda")
    method = vllm_moe.TensorBridgeMoEMethod(TOP_K, E, layout=layout, checkpoint="modelopt", layer_name="layers.0.mlp")
    method.process_weights_after_loading(layer)
    assert not hasattr(layer, "w13_weight_scale_2") and not hasattr(layer, "w13_input_scale")
    assert layer.w13_weight.dtype == torch.int32 and layer.tensorbridge_w2_locks.numel() == 1024

    tokens = 29
    rng = np.random.default_rng(8)
    topk = np.stack([rng.choice(E, size=TOP_K, replace=False) for _ in range(tokens)])
    ids = torch.from_numpy(topk).cuda()
    weights = torch.from_numpy(rng.random((tokens, TOP_K), np.float32)).cuda()
    x = seeded_activations(tokens, H, seed=31)
    out = method.apply(layer, x.cuda(), weights, ids)
    tb.check_status()
    assert out.shape == (tokens, H) and out.dtype == torch.bfloat16

    w13 = [orc.e4m3_decode(v["fp8"][:2 * I, :H]) * v["global_scale6"][0] for v in v13]
    w2 = [orc.e4m3_decode(v["fp8"][:H, :I]) * v["global_scale6"][0] for v in v2]
    xf = x.float().numpy()

    def reference(keep):
        ref = np.zeros((tokens, H), np.float32)
        for t in range(tokens):
            for j in range(TOP_K):
                e = topk[t, j]
                if keep(e):
                    gu = xf[t] @ w13[e].T
                    ref[t] += float(weights[t, j]) * ((gu[:I] / (1 + np.exp(-gu[:I])) * gu[I:]) @ w2[e].T)
        return ref

    ref = reference(lambda e: True)
    assert np.linalg.norm(out.float().cpu().numpy() - ref) / np.linalg.norm(ref) <= 0.08
    again = method.apply(layer, x.cuda(), weights, ids)
    assert torch.equal(out, again)

    # the same experts object serves a rank that holds only the even experts: ids go through expert_map, the others drop out
    if layout == "indexed":
        half = vllm_moe.make_experts(serving.NVFP4MoE(
            w13=_take(method.experts.prepared.w13, slice(0, E, 2)), w2=_take(method.experts.prepared.w2, slice(0, E, 2)),
            top_k=TOP_K, num_global_experts=E, dispatch_ranks=1, layout="indexed", configs=None))
        expert_map = torch.full((E,), -1, dtype=torch.int64, device="cuda")
        expert_map[0::2] = torch.arange(E // 2, device="cuda")
        part = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
        half.apply(part, x.cuda(), weights, ids, expert_map=expert_map)
        tb.check_status()
        ref_half = reference(lambda e: e % 2 == 0)
        assert np.linalg.norm(part.float().cpu().numpy() - ref_half) / np.linalg.norm(ref_half) <= 0.08


def _take(experts, which):
    """A subset of prepared experts (weights, scales and global scales sliced along the expert axis)."""
    import dataclasses
    return dataclasses.replace(experts, weight=experts.weight[which].contiguous(), scale=experts.scale[which].contiguous(),
                               global_scale=experts.global_scale[which].contiguous())


def test_vllm_style_linear_method_without_vllm():
    """`TensorBridgeLinearMethod` on a plain module: the loader's parameters are swapped for the kernel layout, a fused
    layer of two shards with different global scales is brought to a shared one, bias is added, leading dimensions kept."""
    import tensorbridge as tb
    from tensorbridge import vllm_plugin
    from tensorbridge.quant import nvfp4
    shards, k = [128, 256], 512
    layer = torch.nn.Module()
    method = vllm_plugin.TensorBridgeLinearMethod(bridge="exact")
    method.create_weights(layer, k, shards, k, sum(shards), torch.bfloat16)
    weights = [seeded_weight(n, k, seed=40 + i, std=0.02 * (i + 1)) for i, n in enumerate(shards)]
    packed, scales, multipliers = zip(*(nvfp4.quantize(w) for w in weights))
    layer.weight.data = torch.cat(packed).cuda()
    layer.weight_scale.data = torch.cat(scales).cuda()
    layer.weight_scale_2.data = torch.cat(multipliers).cuda()
    assert vllm_plugin.unsupported_linear_reason(layer) is None
    method.process_weights_after_loading(layer)
    assert not hasattr(layer, "weight") and layer.tensorbridge_weight.dtype == torch.int32
    x = seeded_activations(6, k, seed=50).cuda().view(2, 3, k)
    bias = torch.full((sum(shards),), 0.5, dtype=torch.bfloat16, device="cuda")
    out = method.apply(layer, x, bias)
    tb.check_status()
    assert out.shape == (2, 3, sum(shards))
    # reference: each shard's own dequantised weight (the shared global scale only re-rounds the smaller shard's group
    # scales to E4M3, a relative step of at most 2^-4 on single groups)
    ref = torch.cat([orc_dequant(w).cuda() for w in weights]).float()
    want = x.float().view(6, k) @ ref.T + 0.5
    err = float((out.float().view(6, -1) - want).norm() / want.norm())
    assert err < 0.2, err  # a sanity bound: FP8 activations and 4-bit weights against the unquantised product (about 0.1)
    with pytest.raises(ValueError):
        method.apply(layer, x.float(), None)
    with pytest.raises(ValueError):
        vllm_plugin.TensorBridgeLinearMethod().create_weights(torch.nn.Module(), 24, [8], 24, 8, torch.bfloat16)


def orc_dequant(w):
    """The BF16 weight itself (what quantisation approximates)."""
    return w.float()
