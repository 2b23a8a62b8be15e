"""Opt-in measurement of candidate configs for one call shape; the winner is recorded with `override_config`.

Same entry points as the reference's `tensorbridge/jit/autotune.py` (`autotune`, `autotune_grouped`); the candidate
set is the B200 rule's pick plus its neighbours in token tile, K splits and ring depths.  Timing uses CUDA events
around a burst of launches that cycle through enough weight copies to defeat the L2, as the reference's protocol does
(`tensorbridge/jit/autotune.py:77-80`).
"""
from __future__ import annotations

import dataclasses

import torch

from tensorbridge.jit import runtime
from tensorbridge.jit.codegen import GemmConfig

L2_BYTES = 126 << 20


@dataclasses.dataclass
class Stats:
    """Counters of what autotune did in this process."""

    shapes: int = 0
    candidates: int = 0
    rejected: int = 0


stats = Stats()


def candidates(base: GemmConfig, m: int, layout: str, group_scales: bool) -> list[GemmConfig]:
    """`base` first, then its neighbours."""
    out = [base]
    tiles = [bm for bm in (16, 32, 64, 128, 256) if bm <= (64 if group_scales else 256)]
    for bm in tiles:
        if bm != base.block_m and (bm >= min(m, tiles[-1]) or layout != "dense" or m > tiles[-1]) and bm in (base.block_m // 2, base.block_m * 2):
            out.append(dataclasses.replace(base, block_m=bm, num_stages=min(base.num_stages, 8 if bm >= 128 else 12)))
    if layout == "dense" and not group_scales:
        if base.use_stream_k == 1:  # last round shared out in K blocks: the only alternative is whole tiles
            out.append(dataclasses.replace(base, use_stream_k=0))
        else:
            for splits in {0, max(base.use_stream_k - 1, 0), base.use_stream_k + 1, base.use_stream_k * 2}:
                if splits != base.use_stream_k and splits != 1:
                    out.append(dataclasses.replace(base, use_stream_k=splits))
    for bridged in (2, 8):  # 8 only fits where the accumulators leave 256 columns of tensor memory
        if bridged == 2 or not group_scales or base.block_m <= 32:
            out.append(dataclasses.replace(base, stream_k_aligned=bridged))
    if base.num_stages > 4:
        out.append(dataclasses.replace(base, num_stages=base.num_stages - 2))
    seen, unique = set(), []
    for config in out:
        if config not in seen:
            seen.add(config)
            unique.append(config)
    return unique


def time_call(call, copies: int, launches: int = 24, rounds: int = 3) -> float:
    """Median microseconds per launch of `call(i)` over `rounds` bursts; `i` cycles through `copies` weight copies."""
    for i in range(3):
        call(i % copies)
    torch.cuda.synchronize()
    times = []
    for _ in range(rounds):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(launches):
            call(i % copies)
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop) * 1000.0 / launches)
    return sorted(times)[len(times) // 2]


def _weight_copies(tensors: list[torch.Tensor]) -> int:
    nbytes = sum(t.numel() * t.element_size() for t in tensors)
    return max(1, min(-(-2 * L2_BYTES // max(nbytes, 1)) + 1, 16))


def autotune(a: torch.Tensor, a_scale: torch.Tensor, weight, *, group_scales: bool = False) -> GemmConfig:
    """Measure the dense GEMM of this `(M, N, K)` and serve it with the fastest config from now on."""
    from tensorbridge.gemm import fp8_nvfp4_gemm  # noqa: PLC0415

    n, k = weight.shape
    m = a.size(0)
    device = a.get_device()
    base = runtime.select_config(m, n, k, device=device, bridge=weight.bridge, group_scales=group_scales)
    copies = _weight_copies([weight.weight, weight.scale])
    clones = [weight] + [dataclasses.replace(weight, weight=weight.weight.clone(), scale=weight.scale.clone())
                         for _ in range(copies - 1)]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    best, best_us = base, float("inf")
    for config in candidates(base, m, "dense", group_scales):
        stats.candidates += 1
        try:
            us = time_call(lambda i, c=config: fp8_nvfp4_gemm(a, a_scale, clones[i], out=out, config=c,
                                                             group_scales=group_scales), copies)
        except ValueError:
            stats.rejected += 1
            continue
        if us < best_us:
            best, best_us = config, us
    stats.shapes += 1
    runtime.override_config(m, n, k, best, device, bridge=weight.bridge, group_scales=group_scales)
    return best


def autotune_grouped(a: torch.Tensor, a_scale: torch.Tensor, experts, routing, m: int, *,
                     group_scales: bool = False) -> GemmConfig:
    """Measure the grouped GEMM of this shape and routing and serve it with the fastest config from now on.  Indexed
    routing is tied to its `block_m`, so only ring depths vary there."""
    from tensorbridge.gemm import ContiguousRouting, IndexedRouting, fp8_nvfp4_grouped_gemm  # noqa: PLC0415

    num_experts, n, k = experts.shape
    layout = "indexed" if isinstance(routing, IndexedRouting) else "contiguous" if isinstance(routing, ContiguousRouting) else "masked"
    top_k = routing.top_k if layout == "indexed" else 1
    device = a.get_device()
    base = runtime.select_config(m, n, k, num_experts, layout, device=device, bridge=experts.bridge, top_k=top_k,
                                 group_scales=group_scales)
    if layout == "indexed":
        base = dataclasses.replace(base, block_m=routing.block_m)
    rows = a.size(0) * top_k if layout == "indexed" else a.size(0)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=a.device)
    best, best_us = base, float("inf")
    for config in candidates(base, m, layout, group_scales):
        if layout == "indexed" and config.block_m != routing.block_m:
            continue
        stats.candidates += 1
        try:
            us = time_call(lambda i, c=config: fp8_nvfp4_grouped_gemm(a, a_scale, experts, routing, m, out=out, config=c,
                                                                     group_scales=group_scales), 1)
        except ValueError:
            stats.rejected += 1
            continue
        if us < best_us:
            best, best_us = config, us
    stats.shapes += 1
    runtime.override_config(m, n, k, best, device, num_experts, layout, experts.bridge, top_k, group_scales)
    return best


# ---------------------------------------------------------------------------------------------------------------------
# Profile sweeper: measured configs for a weight shape over a list of M, written in the profile JSON format
# (`tensorbridge/jit/profiles.py`).  The reference's counterpart is `benchmarks/sweep_moe_profiles.py:197-390`.
# ---------------------------------------------------------------------------------------------------------------------
SWEEP_M = (1, 2, 4, 8, 16, 32, 64, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096, 6144, 8192)
LAST_SEGMENT = 2 ** 31 - 1


def _tile_defaults(bm: int, n: int, k: int, num_sms: int) -> GemmConfig:
    """The rule's ring depths for token tile `bm`: ask the rule at an M that makes it choose that tile."""
    probe = {192: 160, 256: 4096}.get(bm, bm)
    config = runtime.rule_config(probe, n, k, num_sms)
    if config.block_m != bm:  # the wave model preferred the other wide tile at this shape: keep its depths, they fit
        config = dataclasses.replace(config, block_m=bm, num_stages=min(config.num_stages, 6 if bm == 256 else 10))
    return config


def dense_candidates(m: int, n: int, k: int, num_sms: int) -> list[GemmConfig]:
    """Per-token dense candidates for one M: token tiles that cover M (or the two wide tiles), K splits that fill the
    SMs once, 8 warps in two teams or 16 in four, 4 or 8 bridged tiles.  The rule's own pick comes first."""
    n_tiles, k_blocks = -(-n // 128), -(-k // 128)
    out = [runtime.rule_config(m, n, k, num_sms)]
    if m <= 128:
        small = 16
        while small < m:
            small *= 2
        tiles_m = [small] + ([small * 2] if small < 128 else [192])
    else:
        tiles_m = [192, 256] + ([128] if m <= 512 else [])
        # narrow weights (column-parallel shards): wide tiles leave most SMs without a tile, so the narrower tiles and
        # their K splits compete as well
        if -(-m // 256) * n_tiles * 2 <= num_sms:
            tiles_m += [bm for bm in (128, 64) if bm not in tiles_m and -(-m // bm) * n_tiles <= 128]
    for bm in tiles_m:
        base = _tile_defaults(bm, n, k, num_sms)
        tiles = -(-m // bm) * n_tiles
        fill = num_sms // tiles if tiles else 0
        split_options = {0}
        if tiles <= 128:
            split_options |= {s for s in (fill, fill - 1, fill + 1, fill // 2, (fill + 2) // 3, 2)
                              if 2 <= s <= min(16, max(k_blocks // 2, 1)) and tiles * s <= 2 * num_sms}
        for splits in sorted(split_options):
            for warpgroups, teams in ((2, 2), (4, 4)):
                for bridged in (4, 8):
                    out.append(dataclasses.replace(base, use_stream_k=splits, math_warpgroups=warpgroups,
                                                   m_fast_tile_order=teams, stream_k_aligned=bridged))
    seen, unique = set(), []
    for config in out:
        if config not in seen:
            seen.add(config)
            unique.append(config)
    return unique


def time_graph(call, copies: int, launches: int = 24, rounds: int = 5) -> float:
    """Median microseconds per launch of `call(i)` replayed from one CUDA graph of `launches` launches (no launch gaps;
    `i` cycles through `copies` weight copies)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(2):
            call(i % copies)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(launches):
                call(i % copies)
        graph.replay()
        side.synchronize()
        times = []
        for _ in range(rounds):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(side)
            graph.replay()
            stop.record(side)
            stop.synchronize()
            times.append(start.elapsed_time(stop) * 1000.0 / launches)
    return sorted(times)[len(times) // 2]


def merge_segments(picks: list[tuple[int, GemmConfig]]) -> list[list]:
    """`[(m, best config)]` sorted by m -> profile segments `[[max_m, nine ints]]`: neighbours with one config merge,
    the last segment is open ended."""
    segments: list[list] = []
    for m, config in sorted(picks, key=lambda item: item[0]):
        values = config.to_list()
        if segments and segments[-1][1] == values:
            segments[-1][0] = m
        else:
            segments.append([m, values])
    if segments:
        segments[-1][0] = LAST_SEGMENT
    return segments


def sweep_dense_profile(n: int, k: int, ms=SWEEP_M, *, bridge: Bridge = "exact", device: int | None = None,
                        min_gain: float = 0.02, report=None) -> dict:
    """Measure `dense_candidates` for every M of `ms` on a seeded random `[n, k]` weight (launches chained by
    programmatic dependent launch with static weights, as the serving layers launch) and return the profile entry.
    A candidate replaces the rule's pick only when it is faster by more than `min_gain`."""
    from tensorbridge.gemm import PDL_STATIC_WEIGHTS, fp8_nvfp4_gemm  # noqa: PLC0415
    from tensorbridge.quant import fp8, nvfp4  # noqa: PLC0415

    device = torch.cuda.current_device() if device is None else device
    dev = torch.device("cuda", device)
    num_sms = runtime.get_num_sms(device)
    gen = torch.Generator().manual_seed(0)
    checkpoint = nvfp4.quantize((torch.randn((n, k), generator=gen) * 0.02).bfloat16().to(dev))
    first = nvfp4.prepare(*checkpoint, bridge=bridge)
    copies = _weight_copies([first.weight, first.scale])
    clones = [first] + [dataclasses.replace(first, weight=first.weight.clone(), scale=first.scale.clone())
                        for _ in range(copies - 1)]
    picks = []
    for m in ms:
        x = torch.randn((m, k), generator=gen).bfloat16().to(dev)
        a, a_scale = fp8.quantize(x)
        out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        best, best_us, rule_us = None, float("inf"), None
        for index, config in enumerate(dense_candidates(m, n, k, num_sms)):
            stats.candidates += 1
            try:
                us = time_graph(lambda i, c=config: fp8_nvfp4_gemm(a, a_scale, clones[i], out=out, config=c,
                                                                  enable_pdl=PDL_STATIC_WEIGHTS), copies)
            except ValueError:
                stats.rejected += 1
                continue
            if index == 0:
                best, best_us, rule_us = config, us, us
            elif us < best_us and us < rule_us * (1.0 - min_gain):
                best, best_us = config, us
        stats.shapes += 1
        picks.append((m, best))
        if report is not None:
            report(m, best, best_us, rule_us)
    return {"device": _name(device), "num_sms": num_sms, "n": codegen_pad(n), "k": codegen_pad(k), "num_experts": 0,
            "layout": "dense", "group_scales": False, "bridge": bridge, "segments": merge_segments(picks)}


def _name(device: int) -> str:
    return runtime._device_name(device)


def codegen_pad(size: int) -> int:
    from tensorbridge.jit.codegen import pad_to_unit  # noqa: PLC0415
    return pad_to_unit(size)


def write_profile(entries: list[dict], path: str) -> None:
    """Write (or replace, by key) `entries` in the profile JSON at `path`."""
    import json  # noqa: PLC0415
    import os  # noqa: PLC0415

    from tensorbridge.jit import profiles  # noqa: PLC0415

    existing = []
    if os.path.exists(path):
        with open(path) as handle:
            existing = json.load(handle)
    key = lambda e: (e["device"], e["num_sms"], e["n"], e["k"], e["num_experts"], e["layout"], e["group_scales"], e["bridge"])  # noqa: E731
    merged = {key(e): e for e in existing}
    merged.update({key(e): e for e in entries})
    with open(path, "w") as handle:
        json.dump(sorted(merged.values(), key=key), handle, indent=1)
        handle.write("\n")
    profiles.reload()


if __name__ == "__main__":
    import argparse
    import sys

    parser = argparse.ArgumentParser(description="Sweep dense per-token configs for weight shapes and write a profile JSON.")
    parser.add_argument("--shape", action="append", required=True, help="N,K (repeatable)")
    parser.add_argument("--bridge", action="append", default=None, choices=["exact", "fpma"])
    parser.add_argument("--out", required=True)
    cli = parser.parse_args()
    entries = []
    for shape in cli.shape:
        n_arg, k_arg = (int(v) for v in shape.split(","))
        for bridge_arg in cli.bridge or ["exact", "fpma"]:
            entries.append(sweep_dense_profile(
                n_arg, k_arg, bridge=bridge_arg,
                report=lambda m, c, us, rule_us: print(f"[{n_arg}x{k_arg} {bridge_arg}] M={m}: {us:.2f} us (rule {rule_us:.2f}) {c.to_list()}",
                                                       file=sys.stderr, flush=True)))
    write_profile(entries, cli.out)
    print(f"wrote {len(entries)} entries to {cli.out}; {stats.candidates} candidates timed, {stats.rejected} rejected")
