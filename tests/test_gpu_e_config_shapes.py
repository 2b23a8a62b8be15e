"""GPU parity, part 5: the benchmark's own shapes at full size.

The small cases of the other files cannot reach what only production shapes exercise (deep K loops, every ring depth
and team count the selection rule really serves, 32 to 128 experts, profile hits, launches chained by programmatic
dependent launch, CUDA-graph replays).  Every case here runs at a size the benchmark times and is checked three ways:

* bridged weight bytes bit for bit against the oracle (whole weight for the dense shape; a 256-channel slice of every
  expert plus a few experts in full for the grouped shapes);
* output values against the oracle on a seeded sample of at least 64 rows per case (all rows when there are fewer):
  normwise relative error <= 2e-3 against the FP32 product of the same operands -- the plain bar, no allowance --
  plus the tighter pins of `helpers.assert_close_to_oracle`;
* the whole output against an FP32 matmul of the same bridged bytes on the GPU (the size-independent form of the same
  check) and bit identity from run to run and across launch modes.
"""
import dataclasses

import numpy as np
import pytest
import torch

import tb_oracle as orc
from helpers import assert_close_to_oracle, oracle_weight, seeded_activations, seeded_weight, to_cuda_checkpoint

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _sample_rows(rows: int, count: int = 64, seed: int = 0) -> np.ndarray:
    if rows <= count:
        return np.arange(rows)
    picked = np.random.default_rng(seed).choice(rows, size=count - 2, replace=False)
    return np.unique(np.concatenate([picked, [0, rows - 1]]))


def _gpu_reference(q, s, w_bytes, gs6, n, k):
    """FP32 on the GPU: (decode(q) @ decode(bridged bytes).T) * (s * gs6).  FP8 x FP8 products are exact in FP32."""
    w = w_bytes[:n, :k].view(torch.float8_e4m3fn).float()
    return (q.float() @ w.T) * (s.reshape(-1, 1) * gs6)


def _normwise(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).norm() / want.double().norm().clamp_min(1e-300))


# ---------------------------------------------------------------------------------------------------------------------
# Config 2: dense N = 6144, K = 7168, both bridges, the launch modes the library's layers use.
# ---------------------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module", params=["exact", "fpma"])
def c2_weight(request):
    from tensorbridge.quant import nvfp4
    bridge = request.param
    n, k = 6144, 7168
    view = oracle_weight(seeded_weight(n, k, seed=0), bridge)
    weight = nvfp4.prepare(*to_cuda_checkpoint(view), bridge=bridge)
    bridged = nvfp4.bridged_fp8(weight)
    assert np.array_equal(bridged.cpu().numpy(), view["fp8"]), "bridged weight bytes differ from the oracle's"
    assert np.array_equal(weight.scale.view(torch.uint8).cpu().numpy(), view["scale_t"])
    decoded = orc.decoded_weight(view["fp8"], n, k)
    return bridge, n, k, view, weight, bridged, decoded


@pytest.mark.parametrize("m", [1, 16, 64, 512, 2048, 8192])
def test_c2_dense_sweep_shape(c2_weight, m):
    import tensorbridge as tb
    from tensorbridge.quant import fp8
    bridge, n, k, view, weight, bridged, decoded = c2_weight
    x = seeded_activations(m, k, seed=100 + m)
    q, s = fp8.quantize(x.cuda())
    wq, ws = orc.quantize_fp8_per_token(x)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), wq) and np.array_equal(s.cpu().numpy(), ws)
    served = tb.select_config(m, n, k, bridge=bridge)
    outs = [tb.fp8_nvfp4_gemm(q, s, weight, enable_pdl=mode) for mode in (False, True, tb.PDL_STATIC_WEIGHTS, False)]
    # behind the quantiser, as NVFP4Linear launches it
    q2, s2 = fp8.quantize(x.cuda())
    outs.append(tb.fp8_nvfp4_gemm(q2, s2, weight, enable_pdl=tb.PDL_STATIC_WEIGHTS))
    tb.check_status()
    for other in outs[1:]:
        assert torch.equal(outs[0], other), f"launch modes disagree at M = {m} ({served})"
    gs6 = float(view["global_scale6"][0])
    rows = _sample_rows(m, seed=m)
    fp32 = orc.gemm_fp32(wq[rows], decoded, n, k).astype(np.float64) * (ws[rows].astype(np.float64) * gs6)
    want = orc.gemm_dense(wq[rows], ws[rows], decoded, gs6, n, k)
    got = outs[0][torch.from_numpy(rows).cuda()]
    err = orc.normwise_rel_err(got, fp32)
    assert err <= TOL, f"M = {m}: normwise relative error {err:.3e} on {rows.size} sampled rows"
    if rows.size >= 16:
        assert_close_to_oracle(got, want, fp32)
    # every row, against the FP32 product of the same bridged bytes computed on the GPU
    ref = _gpu_reference(q, s, bridged, gs6, n, k)
    assert _normwise(outs[0].float(), ref) <= TOL
    assert _normwise(outs[0].float(), ref.to(torch.bfloat16).float()) <= 5e-4


# ---------------------------------------------------------------------------------------------------------------------
# Grouped shapes: experts are generated and quantised on the GPU (as the benchmark does); the oracle prepares the same
# checkpoint bytes on the CPU.
# ---------------------------------------------------------------------------------------------------------------------
def _gpu_experts(count: int, n: int, k: int, seed: int, group: bool):
    from tensorbridge.quant import nvfp4
    gen = torch.Generator(device="cuda")
    packed, scales, gss = [], [], []
    for e in range(count):
        gen.manual_seed(seed + e)
        w = (torch.randn((n, k), generator=gen, device="cuda") * 0.02).bfloat16()
        pk, sc, gs = nvfp4.quantize(w)
        packed.append(pk); scales.append(sc); gss.append(gs)
    packed, scales, gss = torch.stack(packed), torch.stack(scales), torch.cat(gss)
    ex = nvfp4.prepare_experts(packed, scales, gss, bridge="exact")
    if group:
        sc = ex.scale.view(torch.uint8).view(count, k // 128, 8, n).permute(0, 1, 3, 2).contiguous()
        ex = dataclasses.replace(ex, scale=sc.view(torch.float8_e4m3fn))
    return ex, packed, scales, gss


def _check_expert_bytes(ex, packed, scales, gss, full_experts):
    """Bridged bytes: a 256-channel slice of every expert, and `full_experts` whole; returns their oracle views."""
    from tensorbridge.quant import nvfp4
    bridged = nvfp4.bridged_fp8(ex)
    raw = scales.view(torch.uint8)
    for e in range(packed.size(0)):
        view = orc.prepare_reference_view(packed[e, :256].cpu().numpy(), raw[e, :256].cpu().numpy(), gss[e:e + 1].cpu().numpy())
        assert np.array_equal(bridged[e, :256].cpu().numpy(), view["fp8"]), f"expert {e}: bridged bytes differ"
    views = {}
    for e in full_experts:
        views[e] = orc.prepare_reference_view(packed[e].cpu().numpy(), raw[e].cpu().numpy(), gss[e:e + 1].cpu().numpy())
        assert np.array_equal(bridged[e].cpu().numpy(), views[e]["fp8"]), f"expert {e}: bridged bytes differ"
        assert abs(float(ex.global_scale[e]) - float(views[e]["global_scale6"][0])) == 0.0
    return bridged, views


def _check_rows_against_oracle(out_rows, wq, ws, view, n, k, group, what):
    gs6 = float(view["global_scale6"][0])
    decoded = orc.decoded_weight(view["fp8"], n, k)
    if group:
        want = orc.gemm_dense_group_scales(wq, ws, decoded, gs6, n, k)
        a = orc.e4m3_decode(wq).astype(np.float64)
        fp32 = np.zeros((wq.shape[0], n))
        for kb in range(k // 128):
            fp32 += (a[:, kb * 128:(kb + 1) * 128] @ decoded[:, kb * 128:(kb + 1) * 128].T.astype(np.float64)) * ws[:, kb:kb + 1]
        fp32 *= gs6
    else:
        want = orc.gemm_dense(wq, ws, decoded, gs6, n, k)
        fp32 = orc.gemm_fp32(wq, decoded, n, k).astype(np.float64) * (ws.astype(np.float64).reshape(-1, 1) * gs6)
    err = orc.normwise_rel_err(out_rows, fp32)
    assert err <= TOL, f"{what}: normwise relative error {err:.3e} on {wq.shape[0]} rows"
    if wq.shape[0] >= 16:
        assert_close_to_oracle(out_rows, want, fp32)


@pytest.fixture(scope="module")
def c3_experts():
    ex, packed, scales, gss = _gpu_experts(32, 4096, 7168, seed=3_000_000, group=False)
    bridged, views = _check_expert_bytes(ex, packed, scales, gss, full_experts=(0, 13))
    return ex, bridged, views


@pytest.mark.parametrize("tokens", [64, 512, 4096])
def test_c3_masked_moe_shape(c3_experts, tokens):
    """Config 3 as one rank of eight sees it: 32 of 256 experts, N = 4096, K = 7168, capacity 2 * T * 8 / 256, counts
    from Zipf(1.1)-skewed softmax routing clamped to the capacity."""
    import tensorbridge as tb
    from tensorbridge.quant import fp8
    ex, bridged, views = c3_experts
    experts_global, local, n, k, top_k = 256, 32, 4096, 7168, 8
    logits = torch.randn((tokens, experts_global), generator=torch.Generator().manual_seed(11 + tokens))
    logits += torch.log(torch.arange(1, experts_global + 1, dtype=torch.float32) ** -1.1)
    top = torch.topk(torch.softmax(logits, -1), top_k, -1).indices
    capacity = max(2 * tokens * top_k // experts_global, 1)
    counts = torch.bincount(top.reshape(-1), minlength=experts_global)[:local].clamp(max=capacity).to(torch.int32)
    rows = local * capacity
    x = seeded_activations(rows, k, seed=300 + tokens)
    q, s = fp8.quantize(x.cuda())
    route = tb.MaskedRouting(counts.cuda())
    outs = []
    for pdl in (False, True):
        out = torch.full((rows, n), 123.0, dtype=torch.bfloat16, device="cuda")
        tb.fp8_nvfp4_grouped_gemm(q, s, ex, route, int(counts.sum()), out=out, enable_pdl=pdl)
        outs.append(out)
    tb.check_status()
    assert torch.equal(outs[0], outs[1])
    out = outs[0]
    wq, ws = orc.quantize_fp8_per_token(x)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), wq)
    for e in range(local):
        c, lo = int(counts[e]), e * capacity
        assert bool((out[lo + c:lo + capacity] == 123.0).all()), f"expert {e}: rows past its count were written"
        if c == 0:
            continue
        ref = _gpu_reference(q[lo:lo + c], s[lo:lo + c], bridged[e], ex.global_scale[e], n, k)
        assert _normwise(out[lo:lo + c].float(), ref) <= TOL, f"expert {e}"
        assert _normwise(out[lo:lo + c].float(), ref.to(torch.bfloat16).float()) <= 5e-4, f"expert {e}"
        if e in views:
            pick = _sample_rows(c, seed=e)
            _check_rows_against_oracle(out[lo:lo + c][torch.from_numpy(pick).cuda()], wq[lo:lo + c][pick], ws[lo:lo + c][pick],
                                       views[e], n, k, False, f"T = {tokens}, expert {e}")


@pytest.fixture(scope="module")
def c4_experts():
    ex, packed, scales, gss = _gpu_experts(128, 7168, 2048, seed=4_000_000, group=True)
    bridged, views = _check_expert_bytes(ex, packed, scales, gss, full_experts=(5, 77))
    return ex, bridged, views


@pytest.mark.parametrize("total_rows", [256, 2048, 16384])
def test_c4_contiguous_group_scale_shape(c4_experts, total_rows):
    """Config 4: 128 experts, N = 7168, K = 2048, [1,128] activation scales, rows per expert from a multinomial over
    Dirichlet(0.3) weights."""
    import tensorbridge as tb
    from tensorbridge.quant import fp8
    ex, bridged, views = c4_experts
    experts, n, k = 128, 7168, 2048
    gen = torch.Generator().manual_seed(40 + total_rows)
    torch.manual_seed(40 + total_rows)
    probs = torch.distributions.Dirichlet(torch.full((experts,), 0.3)).sample()
    choice = torch.multinomial(probs, total_rows, replacement=True, generator=gen)
    counts = torch.bincount(choice, minlength=experts)
    for e in views:  # the experts checked in full must own rows
        counts[e] = max(int(counts[e]), 3)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)])
    rows = int(offsets[-1])
    x = seeded_activations(rows, k, seed=400 + total_rows)
    q, s = fp8.quantize_group_128(x.cuda())
    s = s.contiguous()
    wq, ws = orc.quantize_fp8_group128(x)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), wq) and np.array_equal(s.cpu().numpy(), ws)
    route = tb.ContiguousRouting(offsets.cuda())
    outs = [tb.fp8_nvfp4_grouped_gemm(q, s, ex, route, rows, group_scales=True, enable_pdl=pdl) for pdl in (False, True)]
    tb.check_status()
    assert torch.equal(outs[0], outs[1])
    out = outs[0]
    scale_rows = s.float()
    for e in range(experts):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi == lo:
            continue
        w = bridged[e, :n, :k].view(torch.float8_e4m3fn).float()
        a = q[lo:hi].float()
        ref = torch.zeros((hi - lo, n), dtype=torch.float32, device="cuda")
        for kb in range(k // 128):
            ref += (a[:, kb * 128:(kb + 1) * 128] @ w[:, kb * 128:(kb + 1) * 128].T) * scale_rows[lo:hi, kb:kb + 1]
        ref *= ex.global_scale[e]
        assert _normwise(out[lo:hi].float(), ref) <= TOL, f"expert {e}"
        assert _normwise(out[lo:hi].float(), ref.to(torch.bfloat16).float()) <= 5e-4, f"expert {e}"
        if e in views:
            pick = _sample_rows(hi - lo, seed=e)
            _check_rows_against_oracle(out[lo:hi][torch.from_numpy(pick).cuda()], wq[lo:hi][pick], ws[lo:hi][pick], views[e],
                                       n, k, True, f"{total_rows} rows, expert {e}")


@pytest.fixture(scope="module")
def c5_experts():
    ex, packed, scales, gss = _gpu_experts(128, 1536, 2048, seed=5_000_000, group=False)
    bridged, views = _check_expert_bytes(ex, packed, scales, gss, full_experts=(0, 64, 127))
    return ex, bridged, views


@pytest.mark.parametrize("tokens", [1, 64, 4096])
def test_c5_indexed_moe_shape_in_a_cuda_graph(c5_experts, tokens):
    """Config 5: 128 experts, N = 1536, K = 2048, top_k = 8, uniform routing, routes sorted and padded to the selected
    block_m; fp8.quantize and the grouped GEMM (chained by programmatic dependent launch) captured in one CUDA graph and
    replayed with two different routings and activations."""
    import tensorbridge as tb
    from tensorbridge import routing
    from tensorbridge.quant import fp8
    ex, bridged, views = c5_experts
    experts, n, k, top_k = 128, 1536, 2048, 8
    config = tb.select_config(tokens * top_k, n, k, experts, "indexed", top_k=top_k)
    capacity = routing.padded_capacity(tokens * top_k, experts, config.block_m)
    x = torch.empty((tokens, k), dtype=torch.bfloat16, device="cuda")
    q = torch.empty((tokens, k), dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.empty((tokens, 1), dtype=torch.float32, device="cuda")
    sorted_ids = torch.zeros(capacity, dtype=torch.int32, device="cuda")
    expert_ids = torch.zeros(capacity // config.block_m, dtype=torch.int32, device="cuda")
    padded = torch.zeros(1, dtype=torch.int32, device="cuda")
    route = tb.IndexedRouting(sorted_ids, expert_ids, padded, config.block_m, top_k)
    out = torch.zeros((tokens * top_k, n), dtype=torch.bfloat16, device="cuda")

    def load(case: int) -> np.ndarray:
        rng = np.random.default_rng(1000 * case + tokens)
        topk = np.stack([rng.permutation(experts)[:top_k] for _ in range(tokens)])
        topk[0, 0] = (0, 64, 127)[case % 3]  # one of the experts the oracle holds in full always has a route
        topk[0, 1:] = [e for e in rng.permutation(experts) if e != topk[0, 0]][:top_k - 1]
        fresh = routing.align_routes(torch.from_numpy(topk).cuda(), experts, config.block_m)
        sorted_ids.copy_(fresh.sorted_ids); expert_ids.copy_(fresh.expert_ids); padded.copy_(fresh.num_tokens_padded)
        x.copy_(seeded_activations(tokens, k, seed=500 + case + tokens))
        return topk

    def step():
        fp8.quantize(x, out=(q, s))
        tb.fp8_nvfp4_grouped_gemm(q, s, ex, route, tokens * top_k, out=out, config=config, enable_pdl=True)

    load(0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # lets the stream allocate its gather scratch before the capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
    tb.check_status()
    for case in (1, 2):
        topk = load(case)
        out.fill_(55.0)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        tb.check_status()
        first = out.clone()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(first, out), "replays differ"
        wq, ws = orc.quantize_fp8_per_token(x.cpu())
        assert np.array_equal(q.view(torch.uint8).cpu().numpy(), wq)
        flat = torch.from_numpy(topk.reshape(-1)).cuda()
        token_of = torch.arange(tokens * top_k, device="cuda") // top_k
        for e in torch.unique(flat).tolist():
            routes = (flat == e).nonzero().flatten()
            if routes.numel() == 0:
                continue
            src = token_of[routes]
            ref = _gpu_reference(q[src], s[src], bridged[e], ex.global_scale[e], n, k)
            assert _normwise(first[routes].float(), ref) <= TOL, f"expert {e}"
            assert _normwise(first[routes].float(), ref.to(torch.bfloat16).float()) <= 5e-4, f"expert {e}"
            if e in views:
                pick = _sample_rows(routes.numel(), seed=e)
                rows = src.cpu().numpy()[pick]
                _check_rows_against_oracle(first[routes][torch.from_numpy(pick).cuda()], wq[rows], ws[rows], views[e], n, k, False,
                                           f"T = {tokens}, case {case}, expert {e}")
