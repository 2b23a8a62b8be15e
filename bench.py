"""Benchmark of the FP8 x NVFP4 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload (benchmark config 2, "dense FFN sweep"): W = [N=6144, K=7168] NVFP4 from seeded BF16 N(0, 0.02^2) weights,
activations BF16 N(0,1) with 0.1 % outlier channels x20, quantised per token to FP8, M in {1..8192} (powers of two),
both bridges.  One step = one pass over the sweep: 14 M values x 2 bridges = 28 GEMM launches.  With N > 1 the weight
is split column-parallel over the ranks (N/G channels each, no data-path collective), so total work is fixed:
`"scaling": "strong"`.

Printed JSON line (rank 0):
* `value` = sweep FLOPs / device time of the GEMM launches with FP8 activations resident in HBM (quantisation untimed,
  as the reference's protocol times it).  The 27 launches of a step that are not the dominant kernel are captured in
  one CUDA graph and replayed (the reference times CUDA-graph bursts too); the dominant kernel (M = 8192, exact) is
  launched between two CUDA events every step, and their mean feeds `roofline`.  `value_eager` is the same step
  launched call by call from Python, `host_us_per_call` what one such call costs the host.
* `e2e` = the same FLOPs through the public API from pinned host BF16 activations: H2D copy, fp8.quantize,
  fp8_nvfp4_gemm (PDL), D2H copy of the BF16 output, all inside the timed region.  With N > 1 every rank copies and
  quantises only its M/N rows and the ranks all-gather the FP8 rows and scales over NVLink.
* `sweep` = per-M time / TFLOPS / GB/s from CUDA-graph bursts that cycle weight copies larger than the L2, launched
  plainly (`us_plain`) and chained with programmatic dependent launch and static weights (`us_pdl`); `us` is the
  smaller of the two.
* `sharded` = the two MoE configurations the benchmark shards: the expert-parallel masked MoE (config 3: E = 256 over
  the ranks, NCCL all-to-all dispatch, masked grouped GEMM, combine) and the contiguous [1,128] MoE (config 4: E = 128
  over the ranks), per token count, max over ranks.
* `parity_checked`: before anything is timed every (M, bridge) of the sweep is compared with an FP32 matmul of the same
  bridged operands on the GPU (2e-3 normwise); the `cpu_baseline` leg compares sampled rows with the CPU oracle too.

`--workload moe_masked | moe_contiguous | moe_indexed` runs the grouped GEMM alone at the benchmark's MoE configs
(`--tokens T` one size only, `--bridge-warps 8|16` pins the bridge width); `--case dense --m M` launches one dense
shape a few times for profilers.

`--impl reference` times the reference's CPU path for this workload (NVFP4 dequantisation through the bridge table +
FP32 torch matmul on the host cores, the code in oracle/) over the same M list, bridges, steps and warm-up.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, "atc26-tensorbridge_b200")]

N_FULL, K_FULL = 6144, 7168
SWEEP_M = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]
BRIDGES = ["exact", "fpma"]
L2_BYTES = 126 << 20
METRIC = "FP8xNVFP4 TFLOPS/GPU & weight GB/s vs roofline, M=1-8192, 1/2/4/8 B200"
WORKLOAD = "benchmark config 2: dense FFN sweep N=6144 K=7168, M=1..8192 x {exact,fpma}"
TOL = 2e-3
# DRAM traffic of the dominant launch (gemm_kernel<256, exact>, M = 8192, N = 6144, K = 7168) from one ncu capture:
# dram__bytes_read.sum + dram__bytes_write.sum (profiles/gemm_dense_m8192_n6144_k7168.md); scaled by the channel share
# of a rank when the weight is sharded (traffic is proportional to the channels a launch covers).
DOMINANT_TRAFFIC_BYTES = 85.3e6 + 78.3e6


def measured_peaks() -> tuple[float, float, str]:
    """(HBM GB/s, FP8 dense TFLOP/s, provenance).  The FP8 figure is twice the measured BF16 cuBLAS burst figure:
    the tensor pipe's FP8 rate is twice its BF16 rate and no FP8 number is measured on the pool."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            peaks = json.load(handle)
        return float(peaks["hbm_gbs"]), 2.0 * float(peaks["bf16_tflops"]), "measured (fp8 = 2 x measured bf16 burst; assumed, not measured)"
    return 6650.0, 2.0 * 1590.0, "fallback (fp8 = 2 x fallback bf16)"


def sustained_fp8_peak() -> float:
    """Twice the BF16 cuBLAS figure of a seconds-long loop under the power cap (measured on the pool, else the earlier
    measurement of 1.4 PFLOP/s): what a tensor-bound kernel can hold inside a long step."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return 2.0 * float(json.load(handle).get("bf16_tflops_sustained", 1400.0))
    return 2.0 * 1400.0


def dense_bytes(m: int, n: int, k: int) -> float:
    """Algorithmic bytes of one dense call: 0.5625 B per weight + FP8 activations and scales + BF16 output."""
    return 0.5625 * n * k + m * (k + 4) + 2.0 * m * n


def bench_config(world: int) -> dict:
    """The `config` object both arms print (the CPU arm runs the same workload, sharding included, on the host)."""
    weight_bytes = 0.5625 * (N_FULL // world) * K_FULL
    copies = int(-(-2 * L2_BYTES // weight_bytes)) + 1
    return {"workload": WORKLOAD, "sharding": f"column-parallel N/{world}" if world > 1 else "none",
            "timed": "28 GEMMs per step (14 M x 2 bridges) on FP8 activations already quantised; quantisation untimed",
            "l2": f"GPU arm: inputs larger than the L2, weights cycle through {copies} copies ({copies * weight_bytes / 2**20:.0f} MiB > 2 x L2); "
                  "CPU arm: the weight is dequantised anew every step"}


def sweep_flops() -> float:
    return sum(2.0 * m * N_FULL * K_FULL for m in SWEEP_M) * len(BRIDGES)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index: int) -> None:
        self.index, self.samples, self.stop_flag, self.thread = index, [], threading.Event(), None

    def _run(self) -> None:
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:  # noqa: BLE001
                pass
            self.stop_flag.wait(0.05)

    def start(self) -> None:
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=6)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_min_mhz": mhz[0], "sm_max_mhz": float(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


def build_inputs(rank: int, world: int):
    """Seeded on the CPU so every arm sees the same bits; the rank keeps its N/G channel slice."""
    from tensorbridge.synthetic import seeded_activations, seeded_weight

    n_local = N_FULL // world
    w = seeded_weight(N_FULL, K_FULL, seed=0)[rank * n_local:(rank + 1) * n_local]
    xs = {m: seeded_activations(m, K_FULL, seed=100 + m) for m in SWEEP_M}
    return w, xs, n_local


def init_distributed(local: int):
    """One process per GPU; a single process still gets a (one-rank) NCCL group, which the expert-parallel step uses."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and "MASTER_ADDR" not in os.environ:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(29600 + os.getpid() % 300)
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
    # a rank that fails must not leave the others waiting in a collective for the default ten minutes
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    return dist


def run_native(args) -> None:
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = init_distributed(local)
    import tensorbridge as tb
    from tensorbridge.quant import fp8, nvfp4

    w, xs, n_local = build_inputs(rank, world)
    dev = torch.device("cuda", local)
    hbm_peak, fp8_peak, peak_src = measured_peaks()
    warmup = max(args.warmup, 3)

    # Weights: quantise on the CPU path of the package (same bits on every rank), prepare on the GPU, and keep enough
    # copies that consecutive launches never find their weights in the 126 MB L2.
    packed, scale, gs = nvfp4.quantize(w)
    weight_bytes = 0.5625 * n_local * K_FULL
    copies = int(-(-2 * L2_BYTES // weight_bytes)) + 1
    weights = {b: [nvfp4.prepare(packed.to(dev), scale.to(dev), gs.to(dev), bridge=b) for _ in range(copies)] for b in BRIDGES}
    acts = {m: fp8.quantize(xs[m].to(dev)) for m in SWEEP_M}
    outs = {m: torch.empty((m, n_local), dtype=torch.bfloat16, device=dev) for m in SWEEP_M}
    counter = [0]

    def next_weight(bridge):
        counter[0] += 1
        return weights[bridge][counter[0] % copies]

    def barrier() -> None:
        dist.barrier()
        torch.cuda.synchronize()

    # ---- parity first: every (M, bridge) against an FP32 matmul of the same bridged operands, on this rank's channels
    parity_rows = {}
    worst = 0.0
    for bridge in BRIDGES:
        w_f32 = nvfp4.bridged_fp8(weights[bridge][0])[:n_local, :K_FULL].view(torch.float8_e4m3fn).float()
        for m in SWEEP_M:
            q, s = acts[m]
            got = tb.fp8_nvfp4_gemm(q, s, weights[bridge][0], out=outs[m], enable_pdl=tb.PDL_STATIC_WEIGHTS)
            rows = torch.arange(m, device=dev) if m <= 64 else torch.linspace(0, m - 1, 64, device=dev).long()
            ref = (q[rows].float() @ w_f32.T) * (s[rows] * weights[bridge][0].global_scale)
            err = float((got[rows].float() - ref).double().norm() / ref.double().norm())
            worst = max(worst, err)
            if err > TOL:
                raise SystemExit(f"parity check failed: M = {m}, bridge {bridge}: normwise relative error {err:.3e} > {TOL}")
            parity_rows[(bridge, m)] = (rows.cpu(), got[rows].cpu())
        del w_f32
    tb.check_status()

    # ---- the timed step
    m_big, dominant_bridge = SWEEP_M[-1], "exact"
    launches = [(b, m) for b in BRIDGES for m in SWEEP_M]
    rest = [(b, m) for b, m in launches if (b, m) != (dominant_bridge, m_big)]
    big_start, big_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dominant_ms = []

    def launch(bridge, m, mode):
        tb.fp8_nvfp4_gemm(acts[m][0], acts[m][1], next_weight(bridge), out=outs[m], enable_pdl=mode)

    def eager_step() -> None:
        for bridge, m in launches:
            launch(bridge, m, tb.PDL_STATIC_WEIGHTS)

    stream = torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(stream):
        for _ in range(2):  # lets this stream own its split-K scratch before the capture
            eager_step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for bridge, m in rest:
                launch(bridge, m, tb.PDL_STATIC_WEIGHTS)

    def graph_step(timed: bool) -> None:
        graph.replay()
        # the dominant launch stays plain so that its events bracket it alone
        big_start.record()
        launch(dominant_bridge, m_big, False)
        big_stop.record()
        if timed:
            big_stop.synchronize()
            dominant_ms.append(big_start.elapsed_time(big_stop))

    def timed_region(fn, steps: int) -> float:
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        stop.synchronize()
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local)
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            graph_step(False)
        tb.check_status()
        if rank == 0:
            sampler.start()
        total_ms = timed_region(lambda: graph_step(True), args.steps)
        for _ in range(warmup):
            eager_step()
        eager_ms = timed_region(eager_step, args.steps)
        # the same graph step for at least a second: long enough for the clock sampler and for the power cap to bite
        sustained_steps = max(args.steps, int(1000.0 / max(total_ms / args.steps, 1e-3)) + 1)
        sustained_ms = timed_region(lambda: graph_step(False), sustained_steps)
        # host cost of one call: a burst with no synchronisation inside
        torch.cuda.synchronize()
        q16, s16 = acts[16]
        begin = time.perf_counter()
        for i in range(400):
            tb.fp8_nvfp4_gemm(q16, s16, weights["exact"][i % copies], out=outs[16], enable_pdl=tb.PDL_STATIC_WEIGHTS)
        host_us = (time.perf_counter() - begin) / 400 * 1e6
        torch.cuda.synchronize()
    tb.check_status()

    # ---- end to end from pinned host memory
    e2e_ms, e2e_info = run_e2e(args, tb, fp8, dist, dev, rank, world, xs, weights, n_local, copies, timed_region)
    clocks = sampler.stop() if rank == 0 else {}
    tb.check_status()

    # ---- per-M detail: CUDA-graph bursts cycling the weight copies (kernel time without launch gaps), rank 0 only
    sweep = []
    if rank == 0:
        burst = 2 * copies

        def burst_us(m: int, bridge: str, pdl: bool) -> float:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            mode = tb.PDL_STATIC_WEIGHTS if pdl else False
            with torch.cuda.stream(side):
                for i in range(2):
                    tb.fp8_nvfp4_gemm(acts[m][0], acts[m][1], weights[bridge][i % copies], out=outs[m], enable_pdl=mode)
                side.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(burst):
                        tb.fp8_nvfp4_gemm(acts[m][0], acts[m][1], weights[bridge][i % copies], out=outs[m], enable_pdl=mode)
                g.replay()
                side.synchronize()
                times = []
                for _ in range(5):
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(side)
                    g.replay()
                    stop.record(side)
                    stop.synchronize()
                    times.append(start.elapsed_time(stop) * 1000.0 / burst)
            return sorted(times)[len(times) // 2]

        # M outermost: both bridges of a size are timed back to back, in the same power and clock state
        for m in SWEEP_M:
            for bridge in BRIDGES:
                us_plain = burst_us(m, bridge, False)
                us_pdl = burst_us(m, bridge, True)
                us = min(us_plain, us_pdl)
                flops = 2.0 * m * n_local * K_FULL
                nbytes = dense_bytes(m, n_local, K_FULL)
                tflops, gbs = flops / us / 1e6, nbytes / us / 1e3
                sweep.append({"bridge": bridge, "m": m, "us": round(us, 2), "us_plain": round(us_plain, 2),
                              "us_pdl": round(us_pdl, 2), "tflops": round(tflops, 1),
                              "gbs": round(gbs, 1), "frac_hbm": round(gbs / hbm_peak, 3),
                              "frac_tensor": round(tflops / fp8_peak, 3)})
        tb.check_status()

    # ---- the sharded MoE configurations (all ranks)
    sharded = None if args.no_sharded else run_sharded(args, tb, dist, dev, rank, world)

    if rank == 0:
        flops = sweep_flops()
        ms_per_step = total_ms / args.steps
        value = flops / (ms_per_step * 1e-3) / 1e12
        big_ms = sum(dominant_ms) / max(len(dominant_ms), 1)
        big_tflops = 2.0 * m_big * n_local * K_FULL / (big_ms * 1e-3) / 1e12
        small = [r for r in sweep if r["m"] <= 64]
        large = [r for r in sweep if r["m"] >= 2048]
        sm_mhz = clocks.get("sm_mhz")
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 x nvfp4 -> fp32 acc -> bf16", "data": "synthetic",
            "config": bench_config(world),
            "launch": "27 launches of a step replayed from one CUDA graph (PDL, static weights), the dominant one launched plainly "
                      "between two CUDA events",
            "value_eager": round(flops / (eager_ms / args.steps * 1e-3) / 1e12, 2),
            "host_us_per_call": round(host_us, 2),
            "sustained": {"value": round(flops / (sustained_ms / sustained_steps * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                          "steps": sustained_steps, "seconds": round(sustained_ms / 1e3, 3),
                          "ms_per_step_x_sm_mhz": None if not sm_mhz else round(sustained_ms / sustained_steps * sm_mhz, 1)},
            "e2e": dict({"value": round(flops / (e2e_ms / args.steps * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                         "ms_per_step": round(e2e_ms / args.steps, 3)}, **e2e_info),
            "gpu_launches": args.steps * len(launches) * world,
            "parity_checked": True, "parity_worst_err": round(worst, 6),
            "roofline": {"bound": "tensor", "achieved": round(big_tflops, 1), "peak": round(fp8_peak, 1), "unit": "TFLOP/s",
                         "frac": round(big_tflops / fp8_peak, 4), "frac_of_nominal_4500": round(big_tflops / 4500.0, 4),
                         "frac_of_sustained_peak": round(big_tflops / sustained_fp8_peak(), 4),
                         "traffic": round(DOMINANT_TRAFFIC_BYTES * n_local / N_FULL),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one M = 8192 launch at N = 6144, "
                                           "scaled by the rank's channel share",
                         "algorithmic_bytes": round(dense_bytes(m_big, n_local, K_FULL)),
                         "kernel": f"gemm_kernel<256, exact> M={m_big} N={n_local} K={K_FULL}", "us": round(big_ms * 1e3, 2),
                         "peak_source": peak_src},
            "roofline_small_m": {"bound": "hbm", "unit": "GB/s", "peak": hbm_peak,
                                 "worst_frac_m_le_64": min((r["frac_hbm"] for r in small), default=None),
                                 "best_frac_m_le_64": max((r["frac_hbm"] for r in small), default=None),
                                 "worst_frac_tensor_m_ge_2048": min((r["frac_tensor"] for r in large), default=None)},
            "clocks": clocks,
            "sweep": sweep,
        }
        if sharded is not None:
            line["sharded"] = sharded
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(parity_rows)
            line["parity_checked_vs_oracle"] = line["cpu_baseline"].pop("parity_ok")
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def run_e2e(args, tb, fp8, dist, dev, rank, world, xs, weights, n_local, copies, timed_region):
    """The sweep through the public API from pinned host memory.  Host-to-device copies, compute and device-to-host
    copies run on three streams ordered per buffer by events, so the PCIe directions overlap each other and the
    kernels; every byte of every step is inside the timed region (the stop event follows the last device-to-host copy).
    With several ranks each copies and quantises rows [rank * c, (rank + 1) * c), c = ceil(M / world), and the ranks
    all-gather the FP8 rows and the scales (NVLink) instead of each pulling the whole activation matrix over PCIe."""
    import torch

    chunk = {m: -(-m // world) for m in SWEEP_M}
    mine = {m: (min(rank * chunk[m], m), min((rank + 1) * chunk[m], m)) for m in SWEEP_M}
    host_x = {m: xs[m][mine[m][0]:mine[m][1]].contiguous().pin_memory() for m in SWEEP_M}
    host_out = {m: torch.empty((m, n_local), dtype=torch.bfloat16).pin_memory() for m in SWEEP_M}
    dev_x = {m: torch.empty((chunk[m], K_FULL), dtype=torch.bfloat16, device=dev) for m in SWEEP_M}
    q_local = {m: torch.zeros((chunk[m], K_FULL), dtype=torch.float8_e4m3fn, device=dev) for m in SWEEP_M}
    s_local = {m: torch.ones((chunk[m], 1), dtype=torch.float32, device=dev) for m in SWEEP_M}
    q_all = {m: torch.empty((world * chunk[m], K_FULL), dtype=torch.float8_e4m3fn, device=dev) for m in SWEEP_M}
    s_all = {m: torch.empty((world * chunk[m], 1), dtype=torch.float32, device=dev) for m in SWEEP_M}
    outs = {m: torch.empty((m, n_local), dtype=torch.bfloat16, device=dev) for m in SWEEP_M}
    main_stream = torch.cuda.current_stream(dev)
    h2d_stream, d2h_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = {m: torch.cuda.Event() for m in SWEEP_M}        # activations of m landed on the device
    ev_consumed = {m: torch.cuda.Event() for m in SWEEP_M}  # quantiser has read dev_x[m]
    ev_out = {m: torch.cuda.Event() for m in SWEEP_M}       # GEMM wrote outs[m]
    ev_saved = {m: torch.cuda.Event() for m in SWEEP_M}     # outs[m] copied to the host
    used = set()
    counter = [0]

    def e2e_step() -> None:
        for bridge in BRIDGES:
            for m in SWEEP_M:
                rows = mine[m][1] - mine[m][0]
                with torch.cuda.stream(h2d_stream):
                    if m in used:
                        h2d_stream.wait_event(ev_consumed[m])
                    if rows:
                        dev_x[m][:rows].copy_(host_x[m], non_blocking=True)
                    ev_in[m].record(h2d_stream)
                main_stream.wait_event(ev_in[m])
                if m in used:
                    main_stream.wait_event(ev_saved[m])
                if world == 1:
                    q, s = fp8.quantize(dev_x[m], out=(q_all[m], s_all[m]))
                else:
                    if rows:
                        fp8.quantize(dev_x[m][:rows], out=(q_local[m][:rows], s_local[m][:rows]))
                    dist.all_gather_into_tensor(q_all[m].view(torch.uint8), q_local[m].view(torch.uint8))
                    dist.all_gather_into_tensor(s_all[m], s_local[m])
                    q, s = q_all[m][:m], s_all[m][:m]
                ev_consumed[m].record(main_stream)
                counter[0] += 1
                tb.fp8_nvfp4_gemm(q, s, weights[bridge][counter[0] % copies], out=outs[m],
                                  enable_pdl=tb.PDL_STATIC_WEIGHTS if world == 1 else False)
                ev_out[m].record(main_stream)
                with torch.cuda.stream(d2h_stream):
                    d2h_stream.wait_event(ev_out[m])
                    host_out[m].copy_(outs[m], non_blocking=True)
                    ev_saved[m].record(d2h_stream)
                used.add(m)
        main_stream.wait_stream(d2h_stream)
        main_stream.wait_stream(h2d_stream)

    for _ in range(2):
        e2e_step()
    e2e_ms = timed_region(e2e_step, args.steps)
    info = {"h2d_bytes_per_step": sum(m * K_FULL * 2 for m in SWEEP_M) * len(BRIDGES),
            "d2h_bytes_per_step": sum(m * N_FULL * 2 for m in SWEEP_M) * len(BRIDGES),
            "bytes_counted": "whole job: every activation row crosses PCIe once (on one rank), every rank returns its columns",
            "path": ("pinned host BF16 -> H2D -> fp8.quantize -> fp8_nvfp4_gemm(enable_pdl) -> D2H BF16; copies and compute on "
                     "three streams") if world == 1 else
                    (f"pinned host BF16 rows M/{world} per rank -> H2D -> fp8.quantize -> NCCL all-gather of FP8 rows + scales -> "
                     "fp8_nvfp4_gemm on the rank's channels -> D2H BF16 columns; copies and compute on three streams")}
    return e2e_ms, info


# ---------------------------------------------------------------------------------------------------------------------
# The sharded MoE configurations inside the default run: config 3 expert-parallel end to end, config 4 experts sharded.
# ---------------------------------------------------------------------------------------------------------------------
def gpu_experts(torch, nvfp4, count: int, n: int, k: int, seed: int, dev, group: bool):
    import dataclasses

    gen = torch.Generator(device=dev)
    packed, scales, gss = [], [], []
    for e in range(count):
        gen.manual_seed(seed + e)
        w = (torch.randn((n, k), generator=gen, device=dev) * 0.02).bfloat16()
        pk, sc, gs = nvfp4.quantize(w)
        packed.append(pk); scales.append(sc); gss.append(gs)
    ex = nvfp4.prepare_experts(torch.stack(packed), torch.stack(scales), torch.cat(gss), bridge="exact")
    if group:
        sc = ex.scale.view(torch.uint8).view(count, k // 128, 8, n).permute(0, 1, 3, 2).contiguous()
        ex = dataclasses.replace(ex, scale=sc.view(torch.float8_e4m3fn))
    return ex


def run_sharded(args, tb, dist, dev, rank: int, world: int) -> dict:
    import torch
    from tensorbridge import parallel, synthetic
    from tensorbridge.quant import fp8, nvfp4

    hbm_peak, fp8_peak, _ = measured_peaks()
    out = {"note": "times are the maximum over ranks; every rank holds E / n_gpus experts"}

    def max_over_ranks(value: float) -> float:
        t = torch.tensor([value], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(value: float) -> float:
        t = torch.tensor([value], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- config 3: E = 256, N = 4096, K = 7168, top_k = 8, Zipf(1.1) routing, capacity 2 * T * 8 / 256
    experts, n, k, top_k = 256, 4096, 7168, 8
    if experts % world == 0:
        e_local = experts // world
        mine = parallel.local_experts(experts, rank, world, "interleaved")
        ex = gpu_experts(torch, nvfp4, e_local, n, k, 1_000_000 + rank * e_local, dev, False)
        del mine
        rows_out = []
        for tokens in (64, 512, 4096):
            local_tokens = max(tokens // world, 1)
            ids_all = synthetic.zipf_topk(local_tokens * world, experts, top_k, seed=1000 + tokens)
            ids = ids_all[rank * local_tokens:(rank + 1) * local_tokens].to(dev)
            capacity = max(2 * local_tokens * world * top_k // experts, 1)
            x = synthetic.seeded_activations(local_tokens, k, seed=2000 + tokens + rank).to(dev)
            gemm_start, gemm_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            gemm_ms = []
            routes = local_tokens * top_k

            def collective_step(timed: bool = False):
                q, s = fp8.quantize(x)
                plan = parallel.dispatch_masked(q, s, ids, experts, capacity, placement="interleaved")
                gemm_start.record()
                y = tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, ex, tb.MaskedRouting(plan.counts), routes)
                gemm_stop.record()
                result = parallel.combine_masked(y, plan, routes)
                if timed:
                    gemm_stop.synchronize()
                    gemm_ms.append(gemm_start.elapsed_time(gemm_stop))
                return result, plan

            exchange, why_not = None, None
            try:
                exchange = parallel.PeerMaskedExchange(experts, capacity, k, 1, n, placement="interleaved", max_routes=routes)
            except Exception as exc:  # noqa: BLE001  peer mapping unavailable on this box: the collective path is timed alone
                why_not = f"{type(exc).__name__}: {exc}"
            usable = torch.tensor([exchange is not None], device=dev, dtype=torch.int32)
            dist.all_reduce(usable, op=dist.ReduceOp.MIN)
            if not bool(usable.item()) and exchange is not None:
                exchange.close()
                exchange = None

            def peer_step(timed: bool = False, events: bool = True):
                q, s = fp8.quantize(x)
                plan = exchange.dispatch(q, s, ids)
                if events:
                    gemm_start.record()
                tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, ex, tb.MaskedRouting(plan.counts), routes, out=plan.out)
                if events:
                    gemm_stop.record()
                result = exchange.combine(plan)
                if timed:
                    gemm_stop.synchronize()
                    gemm_ms.append(gemm_start.elapsed_time(gemm_stop))
                return result, plan

            def fused_step(timed: bool = False, events: bool = True):
                # the combine fused into the GEMM's epilogue: every output row is stored into its origin rank's buffer
                q, s = fp8.quantize(x)
                plan = exchange.dispatch(q, s, ids, fused_combine=True)
                if events:
                    gemm_start.record()
                tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, ex, tb.MaskedRouting(plan.counts), routes, out=plan.out,
                                          scatter=plan.scatter)
                if events:
                    gemm_stop.record()
                result = exchange.finish(plan)
                if timed:
                    gemm_stop.synchronize()
                    gemm_ms.append(gemm_start.elapsed_time(gemm_stop))
                return result, plan

            result, plan = collective_step()
            kept = int((plan.recv_rows >= 0).sum())
            # Checks of the first step.  Dispatch and combine with the identity as expert: the first 64 FP8 bytes of every
            # row, sent to its expert's rank and back, must return to the route they left from (or as zeros, when the
            # route fell past its expert's capacity); over all ranks as many routes return as were kept.
            q0, _ = fp8.quantize(x)
            echo = parallel.combine_masked(plan.a.view(torch.uint8)[:, :64].to(torch.bfloat16).contiguous(), plan, routes)
            want = q0.view(torch.uint8)[:, :64].to(torch.bfloat16).repeat_interleave(top_k, 0)
            same, zero = (echo == want).all(1), (echo == 0).all(1)
            returned = sum_over_ranks(int((same & ~zero).sum()))
            if not bool((same | zero).all()) or returned > sum_over_ranks(kept) or returned < 0.98 * sum_over_ranks(kept):
                raise SystemExit(f"expert-parallel round trip failed at T = {local_tokens * world} on rank {rank}")
            # and the grouped GEMM on what was received: every expert's rows against an FP32 product of the same operands
            y0 = tb.fp8_nvfp4_grouped_gemm(plan.a, plan.a_scale, ex, tb.MaskedRouting(plan.counts), routes)
            bridged = nvfp4.bridged_fp8(ex)
            for e in range(0, e_local, max(e_local // 8, 1)):
                c = int(plan.counts[e])
                if c:
                    lo = e * capacity
                    ref = (plan.a[lo:lo + c].float() @ bridged[e].view(torch.float8_e4m3fn).float().T) * (plan.a_scale[lo:lo + c] * ex.global_scale[e])
                    err = float((y0[lo:lo + c].float() - ref).double().norm() / ref.double().norm())
                    if err > TOL:
                        raise SystemExit(f"expert-parallel GEMM parity failed: T = {local_tokens * world}, rank {rank}, expert {e}: {err:.3e}")
            del bridged, y0, echo, want
            # the exchange over peer memory must return what the collective path returns, bit for bit
            if exchange is not None:
                peer_result, _ = peer_step()
                if not torch.equal(peer_result, result):
                    raise SystemExit(f"peer-memory exchange disagrees with the collective path at T = {local_tokens * world} on rank {rank}")
                fused_result, _ = fused_step()
                torch.cuda.synchronize()
                if not torch.equal(fused_result, result):
                    raise SystemExit(f"fused combine disagrees with the collective path at T = {local_tokens * world} on rank {rank}")
                tb.check_status()

            def time_steps(step):
                gemm_ms.clear()
                for _ in range(3):
                    step()
                dist.barrier(); torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 10
                start.record()
                for _ in range(reps):
                    step(True)
                stop.record(); stop.synchronize()
                return max_over_ranks(start.elapsed_time(stop) / reps), max_over_ranks(sum(gemm_ms) / len(gemm_ms))

            nccl_ms, nccl_gemm_ms = time_steps(collective_step)
            pull_ms, pull_gemm_ms = time_steps(peer_step) if exchange is not None else (nccl_ms, nccl_gemm_ms)
            step_ms, g_ms = time_steps(fused_step) if exchange is not None else (nccl_ms, nccl_gemm_ms)
            graph_ms = None
            if exchange is not None:
                # the whole step reads nothing back to the host, so it replays from one CUDA graph per rank
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    fused_step(events=False)
                    side.synchronize()
                    step_graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(step_graph, stream=side):
                        graph_result, _ = fused_step(events=False)
                    for _ in range(3):
                        step_graph.replay()
                    side.synchronize()
                    if not torch.equal(graph_result, result):
                        raise SystemExit(f"replayed expert-parallel step disagrees at T = {local_tokens * world} on rank {rank}")
                    dist.barrier(); torch.cuda.synchronize()
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(side)
                    for _ in range(20):
                        step_graph.replay()
                    stop.record(side); stop.synchronize()
                graph_ms = max_over_ranks(start.elapsed_time(stop) / 20)
                torch.cuda.current_stream(dev).wait_stream(side)
                tb.check_status()
                del step_graph, graph_result
            best_ms = min(step_ms, graph_ms) if graph_ms is not None else step_ms
            routed = sum_over_ranks(kept)
            rows_out.append({"tokens": local_tokens * world, "capacity": capacity,
                             "exchange": "peer memory (NVLink stores by the library's kernels; combine fused into the GEMM's epilogue)" if exchange is not None
                                         else f"NCCL all-to-all (peer mapping unavailable: {why_not})",
                             "step_ms": round(step_ms, 4), "gemm_ms": round(g_ms, 4),
                             "dispatch_combine_ms": round(step_ms - g_ms, 4),
                             "step_ms_graph": None if graph_ms is None else round(graph_ms, 4),
                             "tokens_per_s": round(local_tokens * world / best_ms * 1e3, 1),
                             "step_ms_separate_combine": round(pull_ms, 4), "step_ms_nccl": round(nccl_ms, 4), "routes_kept": int(routed), "routes": local_tokens * world * top_k,
                             "gemm_tflops": round(2.0 * routed * n * k / g_ms / 1e9, 1)})
            if exchange is not None:
                exchange.close()
            del result, plan
        tb.check_status()
        out["moe_masked_expert_parallel"] = {
            "config": "benchmark config 3: E=256 (E/n_gpus per GPU, interleaved placement), N=4096, K=7168, top_k=8, Zipf(1.1) routing; "
                      "step = fp8.quantize -> dispatch -> masked grouped GEMM -> combine; over peer memory (plan, barrier carrying the "
                      "counts, push, barrier, GEMM whose epilogue stores every row into its origin rank's buffer, barrier: no host "
                      "read; step_ms_separate_combine: GEMM into a local buffer, barrier, pull kernel) and, as step_ms_nccl, over NCCL (counts all-to-all, host "
                      "read of the split sizes, packed-row all-to-all, place, GEMM, gather, all-to-all, gather); strong scaling in tokens, "
                      "weights sharded",
            "experts_per_gpu": e_local, "results": rows_out}
        del ex
        torch.cuda.empty_cache()

    # ---- config 4: E = 128, N = 7168, K = 2048, contiguous routing, [1,128] scales, Dirichlet(0.3) rows per expert
    experts, n, k = 128, 7168, 2048
    if experts % world == 0:
        e_local = experts // world
        ex = gpu_experts(torch, nvfp4, e_local, n, k, 4_000_000 + rank * e_local, dev, True)
        rows_out = []
        for total_rows in (256, 2048, 16384):
            counts = synthetic.dirichlet_rows(total_rows, experts, seed=40 + total_rows)[rank * e_local:(rank + 1) * e_local]
            offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)])
            rows = int(offsets[-1])
            x = synthetic.seeded_activations(max(rows, 1), k, seed=4100 + total_rows + rank)[:rows].to(dev)
            us = 0.0
            if rows:
                q, s = fp8.quantize_group_128(x)
                s = s.contiguous()
                route = tb.ContiguousRouting(offsets.to(dev))
                result = torch.empty((rows, n), dtype=torch.bfloat16, device=dev)
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    for _ in range(2):
                        tb.fp8_nvfp4_grouped_gemm(q, s, ex, route, rows, out=result, group_scales=True)
                    side.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        for _ in range(8):
                            tb.fp8_nvfp4_grouped_gemm(q, s, ex, route, rows, out=result, group_scales=True)
                    g.replay(); side.synchronize()
                    times = []
                    for _ in range(5):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record(side); g.replay(); b.record(side); b.synchronize()
                        times.append(a.elapsed_time(b) * 1000.0 / 8)
                us = sorted(times)[len(times) // 2]
            us_max = max_over_ranks(us)
            rows_max = max_over_ranks(rows)
            rows_sum = sum_over_ranks(rows)
            rows_out.append({"rows": int(rows_sum), "rows_per_gpu_max": int(rows_max), "rows_per_gpu_mean": round(rows_sum / world, 1),
                             "imbalance_max_over_mean": round(rows_max / max(rows_sum / world, 1e-9), 3), "us_max": round(us_max, 2),
                             "tflops_total": round(2.0 * rows_sum * n * k / max(us_max, 1e-9) / 1e6, 1)})
        tb.check_status()
        out["moe_contiguous_sharded"] = {
            "config": "benchmark config 4: E=128 sharded E/n_gpus per GPU, N=7168, K=2048, [1,128] activation scales, rows per expert "
                      "multinomial over Dirichlet(0.3); no collective; CUDA-graph bursts of 8 launches",
            "experts_per_gpu": e_local, "results": rows_out}
        del ex
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------------------------------------------------------
# CPU legs: the reference's path (dequantise through the bridge table, FP32 matmul) on the host cores, from oracle/.
# ---------------------------------------------------------------------------------------------------------------------
def cpu_reference_step(orc, views: dict, acts: dict, channels: int, keep: dict | None = None) -> float:
    """One pass of the reference's CPU path over the whole sweep for both bridges, on the first `channels` channels of
    the weight: dequantise (bridge table -> FP8 bytes -> float32) once per bridge, then one FP32 matmul per M on all
    host cores.  Returns the FLOPs done.  `keep` collects the BF16 outputs per (bridge, M)."""
    import numpy as np
    import torch

    flops = 0.0
    for bridge in BRIDGES:
        view = views[bridge]
        w = orc.dequant_weight_f32(view["codes"][:channels], view["raw"][:channels], bridge)[:, :K_FULL]
        gs6 = float(view["global_scale6"][0])
        for m in SWEEP_M:
            q, s = acts[m]
            a = torch.from_numpy(q).view(torch.float8_e4m3fn).to(torch.float32)  # the FP8 activations as torch decodes them
            out = ((a @ w.T) * torch.from_numpy(s * np.float32(gs6))).to(torch.bfloat16)
            if keep is not None:
                keep[(bridge, m)] = out
            flops += 2.0 * m * channels * K_FULL
        del w, out
    return flops


def cpu_inputs():
    import torch

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import tb_oracle as orc
    from tensorbridge.synthetic import seeded_activations, seeded_weight

    torch.set_num_threads(len(os.sched_getaffinity(0)))
    w = seeded_weight(N_FULL, K_FULL, seed=0)
    packed, scale, gs = orc.quantize_nvfp4(w)
    views = {b: orc.prepare_reference_view(packed, scale, gs, bridge=b) for b in BRIDGES}
    acts = {m: orc.quantize_fp8_per_token(seeded_activations(m, K_FULL, seed=100 + m)) for m in SWEEP_M}
    return orc, views, acts


def cpu_baseline(parity_rows: dict) -> dict:
    """One pass of the full sweep on the host cores, timed; its outputs are also the oracle the GPU's sampled rows are
    checked against (2e-3 normwise against each other: both are BF16 roundings of the same FP32 value up to summation
    order)."""
    import torch

    orc, views, acts = cpu_inputs()
    keep: dict = {}
    start = time.perf_counter()
    flops = cpu_reference_step(orc, views, acts, N_FULL, keep)
    seconds = time.perf_counter() - start
    ok, worst = True, 0.0
    for (bridge, m), (rows, got) in parity_rows.items():
        want = keep[(bridge, m)][rows].float()
        err = float((got.float() - want).double().norm() / want.double().norm())
        worst = max(worst, err)
        ok = ok and err <= TOL
    return {"value": round(flops / seconds / 1e12, 5), "unit": "TFLOP/s", "cores": len(os.sched_getaffinity(0)),
            "kind": "port", "seconds": round(seconds, 2), "parity_ok": ok, "parity_worst_err_vs_gpu": round(worst, 6),
            "sample": "one full pass: all 14 M x {exact,fpma} at N=6144, K=7168; weight dequantised once per bridge per pass"}


def run_reference(args) -> None:
    """The reference's CPU path (oracle port: the reference's GEMM kernels are Hopper-only and its prepare/quantise
    kernels need Triton on a GPU) on the host cores; rank 0 only.  Same M list, bridges, steps and warm-up as the GPU
    arm; when the whole run would not end within a few minutes every step covers a bounded share of the weight's
    channels instead of all 6144 (the M list stays whole, the throughput is per FLOP either way)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    orc, views, acts = cpu_inputs()
    warmup = max(args.warmup, 3)
    budget_s = float(os.environ.get("TB_REFERENCE_BUDGET_S", "240"))
    cpu_reference_step(orc, views, acts, 128)  # warms the thread pool
    begin = time.perf_counter()
    cpu_reference_step(orc, views, acts, 1536)  # sizes the channel share
    probe_s = (time.perf_counter() - begin) * (N_FULL / 1536)
    channels = N_FULL
    if probe_s * (warmup + args.steps) > budget_s:
        channels = max(128, int(N_FULL * budget_s / (probe_s * (warmup + args.steps))) // 128 * 128)
    for _ in range(warmup):
        cpu_reference_step(orc, views, acts, channels)
    start = time.perf_counter()
    flops = sum(cpu_reference_step(orc, views, acts, channels) for _ in range(args.steps))
    seconds = time.perf_counter() - start
    value = flops / seconds / 1e12
    cores = len(os.sched_getaffinity(0))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sample = (f"all 14 M x {{exact,fpma}} per step on {channels} of the 6144 channels, K=7168; weight dequantised once per bridge per "
              f"step; {args.steps} steps after {warmup} warm-up steps")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(seconds / args.steps * 1e3, 1), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 matmul of dequantised fp8 operands", "data": "synthetic",
        "config": bench_config(world),
        "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_case(args) -> None:
    """A handful of launches of one dense shape of the sweep, for a profiler: `--case dense --m M [--bridge B]
    [--launches L]`.  Weight copies cycle so every launch streams its weights from HBM."""
    import torch
    import tensorbridge as tb
    from tensorbridge.quant import fp8, nvfp4
    from tensorbridge.synthetic import seeded_activations, seeded_weight

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    packed, scale, gs = nvfp4.quantize(seeded_weight(N_FULL, K_FULL, seed=0))
    copies = int(-(-2 * L2_BYTES // (0.5625 * N_FULL * K_FULL))) + 1
    weights = [nvfp4.prepare(packed.to(dev), scale.to(dev), gs.to(dev), bridge=args.bridge) for _ in range(copies)]
    q, s = fp8.quantize(seeded_activations(args.m, K_FULL, seed=100 + args.m).to(dev))
    out = torch.empty((args.m, N_FULL), dtype=torch.bfloat16, device=dev)
    for i in range(args.launches):
        tb.fp8_nvfp4_gemm(q, s, weights[i % copies], out=out)
    torch.cuda.synchronize()
    tb.check_status()
    print(json.dumps({"case": "dense", "m": args.m, "bridge": args.bridge, "launches": args.launches,
                      "config": tb.select_config(args.m, N_FULL, K_FULL, bridge=args.bridge).to_list()}))


# ---------------------------------------------------------------------------------------------------------------------
# Grouped (MoE) workloads alone: benchmark configs 3, 4 and 5.  `--workload moe_masked | moe_contiguous | moe_indexed`.
# One rank holds E / world experts (config 3: 32, one rank of eight, at every N); no collective in the timed region.
# ---------------------------------------------------------------------------------------------------------------------
MOE_SHAPES = {
    "moe_masked": dict(experts=256, shard=8, n=4096, k=7168, tokens=[64, 512, 4096], top_k=8, group=False),
    "moe_contiguous": dict(experts=128, shard=1, n=7168, k=2048, tokens=[256, 2048, 16384], top_k=1, group=True),
    "moe_indexed": dict(experts=128, shard=1, n=1536, k=2048, tokens=[1, 8, 64, 512, 4096], top_k=8, group=False),
}


def grouped_bytes(active_experts: int, rows_read: int, rows_out: int, n: int, k: int, group: bool) -> float:
    scale_bytes = 4 * (k // 128) if group else 4
    return 0.5625 * n * k * active_experts + rows_read * (k + scale_bytes) + 2.0 * rows_out * n


def run_moe(args) -> None:
    import dataclasses

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = init_distributed(local)

    import tensorbridge as tb
    from tensorbridge import routing, synthetic
    from tensorbridge.quant import fp8, nvfp4

    shape = MOE_SHAPES[args.workload]
    n, k, top_k, group = shape["n"], shape["k"], shape["top_k"], shape["group"]
    experts_global = shape["experts"]
    experts_local = experts_global // max(shape["shard"], world) if shape["shard"] > 1 else experts_global // world
    hbm_peak, fp8_peak, peak_src = measured_peaks()
    ex = gpu_experts(torch, nvfp4, experts_local, n, k, 1_000_000 + rank * experts_local, dev, group)

    cpu_gen = torch.Generator().manual_seed(7 + rank)
    results = []
    for tokens in (shape["tokens"] if not args.tokens else [args.tokens]):
        print(f"[{args.workload}] rank {rank}: {tokens} tokens", file=sys.stderr, flush=True)
        if args.workload == "moe_masked":
            top = synthetic.zipf_topk(tokens, experts_global, top_k, seed=11 + tokens)
            capacity = max(2 * tokens * top_k // experts_global, 1)
            first = (rank * experts_local) % experts_global
            counts = torch.bincount(top.reshape(-1), minlength=experts_global)[first:first + experts_local].clamp(max=capacity)
            rows = experts_local * capacity
            x = torch.randn((rows, k), generator=cpu_gen).bfloat16().to(dev)
            route = tb.MaskedRouting(counts.to(torch.int32).to(dev))
            valid_rows = int(counts.sum())
            active = int((counts > 0).sum())
            rows_read = valid_rows
            hint = valid_rows
        elif args.workload == "moe_contiguous":
            counts = synthetic.dirichlet_rows(tokens, experts_global, seed=40 + tokens)[rank * experts_local:(rank + 1) * experts_local]
            offsets = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)])
            rows = int(offsets[-1])
            x = torch.randn((max(rows, 1), k), generator=cpu_gen).bfloat16().to(dev)[:rows]
            route = tb.ContiguousRouting(offsets.to(dev))
            valid_rows, active, rows_read, hint = rows, int((counts > 0).sum()), rows, rows
        else:
            ids = torch.stack([torch.randperm(experts_global, generator=cpu_gen)[:top_k] for _ in range(tokens)])
            first = rank * experts_local
            local_ids = torch.where((ids >= first) & (ids < first + experts_local), ids - first, torch.full_like(ids, -1))
            x = torch.randn((tokens, k), generator=cpu_gen).bfloat16().to(dev)
            rows = tokens
            hint = int((local_ids >= 0).sum())
            config = tb.select_config(max(hint, 1), n, k, experts_local, "indexed", device=local, top_k=top_k)
            route = routing.align_routes(local_ids.to(dev), experts_local, config.block_m)
            valid_rows, active, rows_read = hint, int(torch.unique(local_ids[local_ids >= 0]).numel()), tokens
        if rows == 0:
            continue
        quant = fp8.quantize_group_128 if group else fp8.quantize
        q, s = quant(x)
        if group:
            s = s.contiguous()
        out_rows = rows * top_k if args.workload == "moe_indexed" else rows
        out = torch.zeros((out_rows, n), dtype=torch.bfloat16, device=dev)

        pinned = None
        if args.bridge_warps:  # tuning knob: the rule's config with another bridge width (8 warps / 2 teams, 16 / 4)
            layout = {"moe_masked": "masked", "moe_contiguous": "contiguous", "moe_indexed": "indexed"}[args.workload]
            base = tb.select_config(max(hint, 1), n, k, experts_local, layout, device=local, top_k=top_k, group_scales=group)
            pinned = dataclasses.replace(base, math_warpgroups=args.bridge_warps // 4, m_fast_tile_order=args.bridge_warps // 4)

        def call(pdl: bool = False) -> None:
            tb.fp8_nvfp4_grouped_gemm(q, s, ex, route, max(hint, 1), out=out, enable_pdl=pdl, group_scales=group, config=pinned)

        call(); call()
        torch.cuda.synchronize()
        tb.check_status()
        first_out = out.clone()
        call()
        torch.cuda.synchronize()
        identical = bool(torch.equal(first_out, out))
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        burst = 8
        with torch.cuda.stream(side):
            call()  # scratch buffers are per stream: let this stream allocate its own before the capture
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(burst):
                    call()
            graph.replay()
            side.synchronize()
            times = []
            for _ in range(5):
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record(side)
                graph.replay()
                stop.record(side)
                stop.synchronize()
                times.append(start.elapsed_time(stop) * 1000.0 / burst)
        us = sorted(times)[len(times) // 2]
        tb.check_status()
        flops = 2.0 * valid_rows * n * k
        nbytes = grouped_bytes(active, rows_read, valid_rows, n, k, group)
        row = {"tokens": tokens, "rows": valid_rows, "active_experts": active, "us": round(us, 2),
               "tflops": round(flops / us / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1),
               "frac_hbm": round(nbytes / us / 1e3 / hbm_peak, 3), "frac_tensor": round(flops / us / 1e6 / fp8_peak, 3),
               "bit_identical": identical}
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, row)
            if rank == 0:
                worst = max(g["us"] for g in gathered)
                row = {"tokens": tokens, "per_rank": gathered, "us_max": worst,
                       "tflops_total": round(sum(2.0 * g["rows"] * n * k for g in gathered) / worst / 1e6, 1)}
        results.append(row)
    if rank == 0:
        print(json.dumps({"workload": args.workload, "n_gpus": world, "experts_per_gpu": experts_local, "n": n, "k": k,
                          "top_k": top_k, "group_scales": group, "bridge": "exact", "scaling": "weak",
                          "timing": "CUDA-graph bursts of 8 launches, weights (>= 226 MB per rank) stream from HBM",
                          "peaks": {"hbm_gbs": hbm_peak, "fp8_tflops": fp8_peak, "source": peak_src}, "results": results}))
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-sharded", action="store_true", help="skip the sharded MoE block of the default run")
    parser.add_argument("--case", default=None, choices=["dense"], help="profile mode: a few launches of one shape")
    parser.add_argument("--m", type=int, default=16)
    parser.add_argument("--bridge", default="exact", choices=BRIDGES)
    parser.add_argument("--launches", type=int, default=6)
    parser.add_argument("--workload", default="dense", choices=["dense"] + list(MOE_SHAPES))
    parser.add_argument("--tokens", type=int, default=0, help="MoE workloads: run this token count only")
    parser.add_argument("--bridge-warps", type=int, default=0, choices=[0, 8, 16], help="MoE workloads: pin the bridge warps")
    args = parser.parse_args()
    if args.workload != "dense":
        run_moe(args)
    elif args.case is not None:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
