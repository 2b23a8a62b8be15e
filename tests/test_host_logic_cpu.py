"""Host-side logic that needs no GPU: the profile registry, the serving-side shape helpers, the JIT's source generator
and NVRTC compile step (NVRTC cross-compiles sm_100a without a device) and its disk cache."""
import dataclasses
import json

import pytest
import torch


def test_profile_registry_round_trip(tmp_path):
    from tensorbridge import GemmConfig
    from tensorbridge.jit import profiles
    a, b = GemmConfig(block_m=16, use_stream_k=3), GemmConfig(block_m=256, num_stages=4)
    profiles.clear_profiles()
    try:
        assert profiles.lookup("NVIDIA B200", 148, 6144, 7168, 0, "dense", False, "exact", 8) is None
        profiles.register_profile("NVIDIA B200", 148, 6100, 7168, 0, "dense", False, "exact",
                                  [profiles.ProfileSegment(0, b), profiles.ProfileSegment(64, a)])
        # keys are padded to the 128-wide weight block; segments are ordered with the open tail last
        assert profiles.lookup("NVIDIA B200", 148, 6144, 7168, 0, "dense", False, "exact", 64) == a
        assert profiles.lookup("NVIDIA B200", 148, 6144, 7168, 0, "dense", False, "exact", 65) == b
        assert profiles.lookup("NVIDIA B200", 132, 6144, 7168, 0, "dense", False, "exact", 8) is None
        with pytest.raises(ValueError):
            profiles.register_profile("x", 1, 128, 128, 0, "dense", False, "exact",
                                      [profiles.ProfileSegment(0, a), profiles.ProfileSegment(0, b)])
        key = ("NVIDIA B200", 148, 6144, 7168, 0, "dense", False, "exact")
        path = tmp_path / "saved.json"
        profiles.save_profile_file(path, [(key, [profiles.ProfileSegment(0, b), profiles.ProfileSegment(64, a)])], {"note": "t"})
        written = json.loads(path.read_text())
        assert written["schema_version"] == 1 and written["entries"][0]["segments"][0] == {"max_m": 64, "config": a.to_list()}
        profiles.clear_profiles()
        assert profiles.load_profile_file(path) == 1
        assert profiles.lookup(*key, 1000) == b
        # the compact form of the profile sweeper loads too; two segments with one max_m do not need orderable configs
        compact = tmp_path / "compact.json"
        compact.write_text(json.dumps([{"device": "d", "num_sms": 4, "n": 128, "k": 128, "num_experts": 0, "layout": "dense",
                                        "group_scales": False, "bridge": "fpma",
                                        "segments": [[32, a.to_list()], [32, b.to_list()], [2 ** 31 - 1, b.to_list()]]}]))
        assert profiles.load_profile_file(compact) == 1
        assert profiles.lookup("d", 4, 128, 128, 0, "dense", False, "fpma", 5) in (a, b)
    finally:
        profiles.clear_profiles(reload_defaults=True)
    # the shipped profile is read again on demand
    assert profiles.lookup("NVIDIA B200", 148, 6144, 7168, 0, "dense", False, "exact", 16) is not None


def test_compress_segments():
    from tensorbridge import GemmConfig
    from tensorbridge.jit.profiles import ProfileSegment, compress_segments
    a, b = GemmConfig(block_m=16), GemmConfig(block_m=64)
    assert compress_segments([]) == []
    got = compress_segments([(64, b), (1, a), (16, a), (256, b)])
    assert got == [ProfileSegment(32, a), ProfileSegment(256, b)]  # boundary at sqrt(16 * 64)
    assert compress_segments([(1, a), (2, b)], unbounded_tail=True) == [ProfileSegment(1, a), ProfileSegment(0, b)]


def _fake_moe(layout="indexed", experts=4, hidden=256, inter=128, top_k=2, global_experts=16, **kwargs):
    from tensorbridge import NVFP4Experts
    from tensorbridge.serving import NVFP4MoE

    def make(n, k):
        return NVFP4Experts(torch.zeros((experts, n, k // 8), dtype=torch.int32), torch.zeros((experts, k // 16, n), dtype=torch.uint8),
                            torch.ones(experts), torch.zeros(1024, dtype=torch.int32), "exact")
    return NVFP4MoE(make(2 * inter, hidden), make(hidden, inter), top_k, global_experts, 1, layout, None, **kwargs)


def test_moe_shape_helpers():
    from tensorbridge import serving
    moe = _fake_moe()
    gate_up, down = serving.moe_grouped_shapes(moe)
    assert (gate_up.n, gate_up.k, gate_up.input_top_k, gate_up.top_k) == (256, 256, 2, 2)
    assert (down.n, down.k, down.input_top_k, down.layout) == (256, 128, 1, "indexed")
    assert serving.moe_grouped_shapes(_fake_moe("masked"))[0].input_top_k == 1
    assert serving.moe_rows(moe, 64) == 16
    # post-dispatch rows: between one and top_k routes per received token, all of them without expert parallelism
    assert serving.moe_post_dispatch_rows(moe, 0) == 0
    rows = serving.moe_post_dispatch_rows(moe, 100)
    share = 4 / 16
    assert rows == round(100 * 2 * share / (1 - (1 - share) ** 2)) and 100 <= rows <= 200
    assert serving.moe_post_dispatch_rows(_fake_moe(global_experts=4), 10) == 20
    assert serving.moe_post_dispatch_rows(_fake_moe(top_k=1), 10) == 10
    assert serving.normalize_dense_shape((0, 128, 256, "fpma")) == serving.DenseShape(0, 128, 256, "fpma", "per_token")
    assert serving.dense_tuned_key(0, 148, 1, 2, 3, "exact", "per_token") == (0, 148, 1, 2, 3, "exact")
    assert serving.dense_tuned_key(0, 148, 1, 2, 3, "exact", "group_128")[-1] == "group_128"
    locks = torch.zeros(1024, dtype=torch.int32)
    assert serving.locks_for_current_stream(locks) is locks


@pytest.mark.parametrize("layout,rows,input_rows", [("indexed", 20, 10), ("contiguous", 20, 20), ("masked", 40, 40)])
def test_moe_buffer_specs(layout, rows, input_rows):
    from tensorbridge import serving
    moe = _fake_moe(layout, gate_up_quant="group_128")
    specs = serving.moe_buffer_specs(moe, 10, unfused_activation=True)
    assert specs["input"] == ((input_rows, 256), torch.float8_e4m3fn)
    assert specs["input_scale"] == ((input_rows, 2), torch.float32)
    assert specs["gate_up"] == ((rows, 256), torch.bfloat16)
    assert specs["intermediate"] == ((rows, 128), torch.float8_e4m3fn)
    assert specs["intermediate_scale"] == ((rows, 1), torch.float32)
    assert specs["output"] == ((rows, 256), torch.bfloat16)
    assert specs["activated"] == ((rows, 128), torch.bfloat16)
    assert "activated" not in serving.moe_buffer_specs(moe, 10)


def test_codegen_points_and_validation():
    from tensorbridge import GemmConfig
    from tensorbridge.jit import codegen
    aot = codegen.kernel_point(GemmConfig(block_m=256, m_fast_tile_order=4, math_warpgroups=4), "exact")
    assert codegen.is_ahead_of_time(aot) and aot.threads == (8 + 16 + 3) * 32
    assert not codegen.is_ahead_of_time(codegen.kernel_point(GemmConfig(block_m=224, m_fast_tile_order=2, math_warpgroups=4)))
    assert not codegen.is_ahead_of_time(codegen.kernel_point(GemmConfig(block_m=128, m_fast_tile_order=2, math_warpgroups=4)))
    assert not codegen.is_ahead_of_time(codegen.kernel_point(GemmConfig(block_m=192), group_scales=True))
    src = codegen.generate(6144, 7168, GemmConfig(block_m=96, m_fast_tile_order=2, math_warpgroups=2), bridge="fpma")
    assert src.name == "tb_jit_m96_fpma_t_w8_t2" and "tb::gemm_body<96, false, false, 8, 2>" in src.source
    assert codegen.generate_pgroup(128, 128, GemmConfig(block_m=48, m_fast_tile_order=1)).point.group_scales
    for bad in (GemmConfig(block_m=24), GemmConfig(block_m=80), GemmConfig(block_m=272), GemmConfig(block_m=64, math_warpgroups=3),
                GemmConfig(block_m=224, m_fast_tile_order=4, math_warpgroups=4),  # two accumulator sets leave two bridged tiles
                GemmConfig(block_m=64, m_fast_tile_order=4, math_warpgroups=2)):  # teams of two warps
        with pytest.raises(ValueError):
            codegen.generate(128, 128, bad)
    with pytest.raises(ValueError):
        codegen.generate_pgroup(128, 128, GemmConfig(block_m=160))


def test_nvrtc_build_and_disk_cache(tmp_path, monkeypatch):
    """NVRTC compiles a template point the library has no instance of to an sm_100a cubin without a GPU; the second
    build of the same source is served from the disk cache, a different source gets its own entry."""
    pytest.importorskip("cuda.bindings.nvrtc")
    from tensorbridge import GemmConfig
    from tensorbridge.jit import codegen, compiler
    monkeypatch.setenv("TENSORBRIDGE_CACHE_DIR", str(tmp_path))
    source = codegen.generate(512, 512, GemmConfig(block_m=48, m_fast_tile_order=2, math_warpgroups=2))
    first = compiler.build(source)
    assert not first.cached and first.entry == "tb_jit_m48_exact_t_w8_t2" and first.stats.registers > 0
    with open(first.cubin_path, "rb") as handle:
        assert handle.read(4) == b"\x7fELF"
    again = compiler.build(source)
    assert again.cached and again.cubin_path == first.cubin_path
    other = compiler.build(dataclasses.replace(source, source=source.source + "\n// another program\n"))
    assert not other.cached and other.cubin_path != first.cubin_path
    broken = dataclasses.replace(source, source=source.source.replace("gemm_body", "no_such_body"))
    with pytest.raises(RuntimeError, match="NVRTC failed"):
        compiler.build(broken)


def test_local_route_plan_and_moe_support_check():
    """Host side of the MoE adapter: routes sorted by expert (torch path of `parallel.plan_local`) against a brute-force
    stable sort, the scatter table built from it, and the support check's reasons on a duck-typed layer."""
    import types
    import torch
    from tensorbridge import parallel, vllm_moe
    g = torch.Generator().manual_seed(4)
    experts = 6
    ids = torch.randint(-1, experts + 1, (11, 3), generator=g)  # -1 and `experts` are routes of experts held elsewhere
    counts, positions = parallel.plan_local(ids, experts)
    flat = ids.reshape(-1).tolist()
    order = sorted((i for i, e in enumerate(flat) if 0 <= e < experts), key=lambda i: (flat[i], i))
    want = [-1] * len(flat)
    for rank, route in enumerate(order):
        want[route] = rank
    assert positions.tolist() == want
    assert counts.tolist() == [sum(1 for e in flat if e == x) for x in range(experts)]
    offsets, scatter = vllm_moe.prepare_scatter(ids, experts)
    assert scatter.shape == ids.shape and offsets.tolist() == [0] + torch.cumsum(counts, 0).tolist()

    assert vllm_moe.uses_fused_silu("silu") and vllm_moe.uses_fused_silu("SiLU")
    assert not vllm_moe.uses_fused_silu("gelu") and not vllm_moe.uses_fused_silu("silu", swiglu_limit=7.0)
    layer = types.SimpleNamespace(moe_config=types.SimpleNamespace(in_dtype=torch.bfloat16, hidden_dim=2048,
                                                                   intermediate_size_per_partition=1536))
    reason = vllm_moe.unsupported_moe_reason(layer)
    if not torch.cuda.is_available():
        assert reason is not None and "Blackwell" in reason
    with pytest.raises(ValueError):
        vllm_moe.TensorBridgeMoEMethod(8, 128, checkpoint="gguf")
    with pytest.raises(ValueError):
        vllm_moe.make_experts(None, activation="gelu")  # a separate activation needs its function
