"""GPU parity, part 6: the expert-parallel dispatch kernels (`tb_ep_plan`, `tb_ep_pack`, `tb_ep_layout`, `tb_ep_place`,
`tb_gather_rows`) against the torch-op restatement of the same plan that the two-rank gloo test runs on CPU.

One GPU stands in for all ranks: every rank's plan is made in turn, the all-to-all is emulated by slicing the send
buffers, and every rank's received rows are placed.  Integer work: every count, position and byte must be equal.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank_inputs(rank, tokens, width, groups, experts, top_k, seed, dtype):
    g = torch.Generator().manual_seed(seed * 100 + rank)
    x = torch.randint(0, 255, (tokens, width), generator=g, dtype=torch.int32).to(torch.uint8).cuda().view(torch.float8_e4m3fn)
    s = torch.rand((tokens, groups), generator=g).cuda()
    ids = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)]).to(dtype)
    if tokens > 3:
        ids[1, 0] = -1          # routes of experts nobody owns are not sent
        ids[2, top_k - 1] = experts
    return x, s, ids.cuda()


@pytest.mark.parametrize("ids_dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("world,experts,tokens,top_k,width,groups,capacity,placement", [
    (2, 4, 6, 2, 16, 1, 4, "contiguous"),
    (4, 32, 40, 4, 256, 2, 8, "interleaved"),
    (8, 256, 512, 8, 7168, 1, 32, "interleaved"),
    (1, 256, 1500, 8, 512, 1, 20, "contiguous"),     # more than one tile of 1024 routes, one rank
    (2, 1024, 300, 8, 128, 4, 2, "interleaved"),     # the largest expert count the plan kernel takes
])
def test_dispatch_kernels_match_the_torch_plan(world, experts, tokens, top_k, width, groups, capacity, placement, ids_dtype):
    from tensorbridge import parallel
    e_local = experts // world
    row_bytes = parallel.packed_row_bytes(width, groups)
    plans = []
    for rank in range(world):
        x, s, ids = _rank_inputs(rank, tokens, width, groups, experts, top_k, seed=world + experts, dtype=ids_dtype)
        got = parallel._plan_native(x, s, ids, experts, world, placement, row_bytes)
        want = parallel._plan_torch(x, s, ids, experts, world, placement, row_bytes)
        assert torch.equal(got[0], want[0]), "send counts"
        assert torch.equal(got[1], want[1]), "send positions"
        sent = int(want[0].sum())
        payload = slice(0, width + 4 * groups)  # the padding bytes of a packed row are not defined
        assert torch.equal(got[2][:sent, payload], want[2][:sent, payload]), "packed rows"
        assert sent == int((want[1] >= 0).sum())
        plans.append((got[0].view(world, e_local), got[2]))
    torch.cuda.synchronize()
    for dst in range(world):
        recv_counts = torch.stack([plans[src][0][dst] for src in range(world)])  # [source, local expert]
        pieces = []
        for src in range(world):
            counts, send = plans[src]
            start = int(counts[:dst].sum())
            pieces.append(send[start:start + int(counts[dst].sum())])
        recv = torch.cat(pieces)
        a, a_scale, counts, recv_rows = parallel._place_native(recv, recv_counts, capacity, width, groups, torch.float8_e4m3fn)
        wa, wa_scale, wcounts, wrecv_rows = parallel._place_torch(recv, recv_counts, capacity, width, groups, torch.float8_e4m3fn)
        assert torch.equal(counts, wcounts) and torch.equal(recv_rows, wrecv_rows)
        live = torch.zeros(e_local * capacity, dtype=torch.bool, device="cuda")
        for e in range(e_local):
            live[e * capacity:e * capacity + int(counts[e])] = True
        assert torch.equal(a.view(torch.uint8)[live], wa.view(torch.uint8)[live])
        assert torch.equal(a_scale[live], wa_scale[live])
        kept = recv_rows[recv_rows >= 0].long()
        assert kept.numel() == int(counts.sum()) and torch.unique(kept).numel() == kept.numel()
        assert bool(live[kept].all())


def test_gather_rows_kernel():
    from tensorbridge import parallel
    g = torch.Generator().manual_seed(3)
    src = torch.randn((50, 72), generator=g).bfloat16().cuda()  # 144-byte rows
    index = torch.randint(-1, 50, (200,), generator=g, dtype=torch.int32).cuda()
    out = parallel.gather_rows(src, index)
    want = torch.where((index >= 0).unsqueeze(1), src[index.clamp(min=0).long()], torch.zeros_like(src[:1]))
    assert torch.equal(out, want)
    assert parallel.gather_rows(src, index[:0]).shape == (0, 72)
    with pytest.raises(ValueError):
        parallel.gather_rows(src[:, :5].contiguous(), index)


@pytest.fixture(scope="module")
def one_rank_group():
    import os
    import torch.distributed as dist
    created = not dist.is_initialized()
    if created:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29700 + os.getpid() % 200))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    yield dist
    if created:
        dist.destroy_process_group()


def _moe_case(experts, n, k, tokens, top_k, probabilities, seed):
    import tb_oracle as orc
    from helpers import oracle_weight, seeded_activations, seeded_weight
    from tensorbridge.quant import fp8, nvfp4
    views = [oracle_weight(seeded_weight(n, k, seed=seed + e), "exact") for e in range(experts)]
    ex = nvfp4.prepare_experts(torch.stack([torch.from_numpy(v["packed"]) for v in views]).cuda(),
                               torch.stack([torch.from_numpy(v["scale"]) for v in views]).cuda().view(torch.float8_e4m3fn),
                               torch.cat([torch.from_numpy(v["global_scale"]) for v in views]).cuda(), bridge="exact")
    x = seeded_activations(tokens, k, seed=seed + 99)
    q, s = fp8.quantize(x.cuda())
    rng = np.random.default_rng(5)
    ids = torch.from_numpy(np.stack([rng.choice(experts, size=top_k, replace=False, p=probabilities) for _ in range(tokens)])).cuda()
    wq, ws = orc.quantize_fp8_per_token(x)
    return views, ex, q, s, ids, wq, ws


def _check_routes(back, ids, views, wq, ws, capacity, n, k, top_k):
    import tb_oracle as orc
    flat = ids.reshape(-1).cpu().numpy()
    seen = {e: 0 for e in range(len(views))}
    dropped = 0
    for r, e in enumerate(flat):
        seen[e] += 1
        row = back[r].float().cpu()
        if seen[e] > capacity:
            assert bool((row == 0).all())
            dropped += 1
            continue
        t = r // top_k
        want = orc.gemm_dense(wq[t:t + 1], ws[t:t + 1], views[e]["fp8"], float(views[e]["global_scale6"][0]), n, k)[0].float()
        assert float((row - want).abs().max()) <= float(want.abs().max()) * 2 ** -6
    return dropped


def test_dispatch_then_masked_gemm_then_combine_on_one_rank(one_rank_group):
    """The whole expert-parallel step with a world of one process (NCCL all-to-all with itself): every route comes back
    with the output row the masked grouped GEMM computed for it, routes over an expert's capacity come back as zeros."""
    import tensorbridge as tb
    from tensorbridge import parallel
    experts, n, k, tokens, top_k, capacity = 4, 128, 256, 24, 2, 8
    views, ex, q, s, ids, wq, ws = _moe_case(experts, n, k, tokens, top_k, [0.55, 0.25, 0.1, 0.1], seed=600)
    plan = parallel.dispatch_masked(q, s, ids, experts, capacity)
    y = tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, ex, tb.MaskedRouting(plan.counts), tokens * top_k)
    back = parallel.combine_masked(y, plan, tokens * top_k)
    tb.check_status()
    assert _check_routes(back, ids, views, wq, ws, capacity, n, k, top_k) > 0  # the skewed routing overfills the first expert


@pytest.mark.parametrize("placement", ["contiguous", "interleaved"])
def test_peer_memory_exchange_matches_the_collective_path(one_rank_group, placement):
    """The same step over peer memory (`PeerMaskedExchange`: plan, barrier carrying the counts, push, barrier, GEMM,
    barrier, pull): the masked buffers hold the same rows in the same places as the all-to-all path builds, and the
    combined output is the same, over two steps with different routing (the buffers and the barrier count are reused)."""
    import tensorbridge as tb
    from tensorbridge import parallel
    experts, n, k, tokens, top_k, capacity = 4, 128, 256, 24, 2, 8
    views, ex, q, s, ids, wq, ws = _moe_case(experts, n, k, tokens, top_k, [0.55, 0.25, 0.1, 0.1], seed=700)
    exchange = parallel.PeerMaskedExchange(experts, capacity, k, 1, n, placement=placement, wait_us=2_000_000,
                                           max_routes=tokens * top_k)
    try:
        for step in range(2):
            step_ids = ids if step == 0 else ids.flip(0).contiguous()
            want_plan = parallel.dispatch_masked(q, s, step_ids, experts, capacity, placement=placement)
            plan = exchange.dispatch(q, s, step_ids)
            assert torch.equal(plan.counts, want_plan.counts)
            for e in range(experts):
                lo, c = e * capacity, int(plan.counts[e])
                assert torch.equal(plan.a.view(torch.uint8)[lo:lo + c], want_plan.a.view(torch.uint8)[lo:lo + c])
                assert torch.equal(plan.a_scale[lo:lo + c], want_plan.a_scale[lo:lo + c])
            # experts sit in placed order in both paths
            order = list(range(experts))
            weights = ex
            tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, weights, tb.MaskedRouting(plan.counts), tokens * top_k, out=plan.out)
            back = exchange.combine(plan)
            want_y = tb.fp8_nvfp4_grouped_gemm(want_plan.a, want_plan.a_scale, weights, tb.MaskedRouting(want_plan.counts), tokens * top_k)
            want_back = parallel.combine_masked(want_y, want_plan, tokens * top_k)
            tb.check_status()
            assert torch.equal(back, want_back)
            # the combine fused into the GEMM's epilogue delivers the same rows
            fused = exchange.dispatch(q, s, step_ids, fused_combine=True)
            tb.fp8_nvfp4_grouped_gemm(fused.a, fused.a_scale, weights, tb.MaskedRouting(fused.counts), tokens * top_k,
                                      out=fused.out, scatter=fused.scatter)
            delivered = exchange.finish(fused)
            tb.check_status()
            assert torch.equal(delivered, want_back)
            del order
        if placement == "contiguous":
            assert _check_routes(back, ids.flip(0), views, wq, ws, capacity, n, k, top_k) > 0
    finally:
        exchange.close()
