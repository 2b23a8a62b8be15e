"""GPU parity, part 7: kernels compiled at run time.  Template points the library has no ahead-of-time instance of are
generated, compiled with NVRTC, loaded through the driver API, registered with the library and launched by the same
entry points; their results are held to the same bar as the built-in instances."""
import numpy as np
import pytest
import torch

import tb_oracle as orc
from helpers import assert_close_to_oracle, oracle_weight, seeded_activations, seeded_weight, to_cuda_checkpoint

pytestmark = pytest.mark.gpu


def _dense_case(m, n, k, bridge, seed):
    from tensorbridge.quant import fp8, nvfp4
    view = oracle_weight(seeded_weight(n, k, seed=seed), bridge)
    weight = nvfp4.prepare(*to_cuda_checkpoint(view), bridge=bridge)
    x = seeded_activations(m, k, seed=seed + 1)
    q, s = fp8.quantize(x.cuda())
    wq, ws = orc.quantize_fp8_per_token(x)
    gs6 = float(view["global_scale6"][0])
    want = orc.gemm_dense(wq, ws, view["fp8"], gs6, n, k)
    fp32 = orc.gemm_fp32(wq, view["fp8"], n, k).astype(np.float64) * (ws.astype(np.float64) * gs6)
    return weight, q, s, want, fp32


@pytest.mark.parametrize("bridge", ["exact", "fpma"])
@pytest.mark.parametrize("config", [dict(block_m=224, num_stages=4, stream_k_aligned=2, math_warpgroups=4, m_fast_tile_order=2),
                                    dict(block_m=96, num_stages=8, stream_k_aligned=4, math_warpgroups=2, m_fast_tile_order=2),
                                    dict(block_m=48, num_stages=8, stream_k_aligned=4, math_warpgroups=4, m_fast_tile_order=4),
                                    dict(block_m=128, num_stages=8, stream_k_aligned=4, math_warpgroups=4, m_fast_tile_order=2),
                                    dict(block_m=160, num_stages=6, use_stream_k=2, stream_k_aligned=4, math_warpgroups=2, m_fast_tile_order=2)])
def test_run_time_compiled_tiles_match_the_oracle(config, bridge):
    import tensorbridge as tb
    from tensorbridge import _native
    from tensorbridge.jit import codegen, runtime
    cfg = tb.GemmConfig(**config)
    m, n, k = 500, 384, 1280
    weight, q, s, want, fp32 = _dense_case(m, n, k, bridge, seed=900 + cfg.block_m)
    point = codegen.kernel_point(cfg, bridge)
    assert not codegen.is_ahead_of_time(point)
    if (0, point) not in runtime.loaded_kernels:
        with pytest.raises(ValueError, match="compile one"):  # nothing serves this point before the JIT has
            tb.fp8_nvfp4_gemm(q, s, weight, config=cfg)
    before = _native.load().tb_registered_kernels()
    loaded = runtime.get_kernel(n, k, cfg, bridge=bridge)
    assert loaded is not None and loaded.compiled.entry == point.entry
    assert runtime.get_kernel(n, k, cfg, bridge=bridge) is loaded  # compiled and registered once
    assert _native.load().tb_registered_kernels() >= before
    outs = [tb.fp8_nvfp4_gemm(q, s, weight, config=cfg, enable_pdl=mode) for mode in (False, tb.PDL_STATIC_WEIGHTS, False)]
    tb.check_status()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert_close_to_oracle(outs[0], want, fp32)
    # a built-in point needs no compile
    assert runtime.get_kernel(n, k, tb.GemmConfig(block_m=256, m_fast_tile_order=4, math_warpgroups=4)) is None


def test_run_time_compiled_tile_in_a_grouped_launch():
    import tensorbridge as tb
    from tensorbridge.jit import runtime
    from tensorbridge.quant import fp8, nvfp4
    e, n, k = 3, 256, 512
    views = [oracle_weight(seeded_weight(n, k, seed=950 + i), "exact") for i in range(e)]
    ex = nvfp4.prepare_experts(torch.stack([torch.from_numpy(v["packed"]) for v in views]).cuda(),
                               torch.stack([torch.from_numpy(v["scale"]) for v in views]).cuda().view(torch.float8_e4m3fn),
                               torch.cat([torch.from_numpy(v["global_scale"]) for v in views]).cuda(), bridge="exact")
    counts = [100, 0, 37]
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    x = seeded_activations(sum(counts), k, seed=960)
    q, s = fp8.quantize(x.cuda())
    cfg = tb.GemmConfig(block_m=96, num_stages=8, stream_k_aligned=4, math_warpgroups=2, m_fast_tile_order=2)
    runtime.get_grouped_kernel(n, k, e, "contiguous", cfg)
    out = tb.fp8_nvfp4_grouped_gemm(q, s, ex, tb.ContiguousRouting(torch.from_numpy(offsets).cuda()), sum(counts), config=cfg)
    tb.check_status()
    wq, ws = orc.quantize_fp8_per_token(x)
    want = orc.gemm_contiguous(wq, ws, [v["fp8"] for v in views], [v["global_scale6"][0] for v in views], offsets, n, k)
    err = float((out.float().cpu() - want.float()).norm() / want.float().norm())
    assert err <= 2e-3, err


def test_precompile_prepared_loads_what_selection_can_pick():
    """Every config the selection rule or the shipped profile picks for a prepared shape is launchable afterwards; with
    the built-in tiles nothing has to be compiled."""
    import tensorbridge as tb
    from tensorbridge import serving
    from tensorbridge.quant import nvfp4
    view = oracle_weight(seeded_weight(256, 512, seed=970), "exact")
    packed, scale, gs = to_cuda_checkpoint(view)
    serving.prepare_linear(packed, scale, 1.0 / gs, bridge="exact")
    assert serving.precompile_prepared(0) == 0
    assert serving.precompile_prepared(300) >= 0
    assert any(shape.n == 256 and shape.k == 512 for shape, _, tokens in serving.precompiled_dense if tokens == 300)
    assert serving.precompile_prepared(300) == 0  # nothing left to do
    tb.check_status()
