"""GPU parity, part 2: the dense FP8 x NVFP4 GEMM through the public API (and so through the C ABI)."""
import dataclasses

import numpy as np
import pytest
import torch

import tb_oracle as orc
from helpers import assert_close_to_oracle, oracle_weight, seeded_activations, seeded_weight, to_cuda_checkpoint

pytestmark = pytest.mark.gpu


def _case(m, n, k, bridge, seed=0, group=False):
    import tensorbridge  # noqa: F401
    from tensorbridge import experimental
    from tensorbridge.quant import fp8, nvfp4
    view = oracle_weight(seeded_weight(n, k, seed=seed + 1), bridge)
    packed, scale, gs = to_cuda_checkpoint(view)
    weight = (experimental.prepare if group else nvfp4.prepare)(packed, scale, gs, bridge=bridge)
    x = seeded_activations(m, k, seed=seed + 2)
    if group:
        q, s = fp8.quantize_group_128(x.cuda())
        wq, ws = orc.quantize_fp8_group128(x)
    else:
        q, s = fp8.quantize(x.cuda())
        wq, ws = orc.quantize_fp8_per_token(x)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), wq)
    return view, weight, q, s, wq, ws


def _check(out, view, wq, ws, n, k, group=False):
    gs6 = float(view["global_scale6"][0])
    if group:
        want = orc.gemm_dense_group_scales(wq, ws, view["fp8"], gs6, n, k)
        a = orc.e4m3_decode(wq[:, :k]).astype(np.float64)
        w = orc.e4m3_decode(view["fp8"][:n, :k]).astype(np.float64)
        fp32 = np.zeros((wq.shape[0], n))
        for kb in range(-(-k // 128)):
            fp32 += (a[:, kb * 128:(kb + 1) * 128] @ w[:, kb * 128:(kb + 1) * 128].T) * ws[:, kb:kb + 1]
        fp32 *= gs6
    else:
        want = orc.gemm_dense(wq, ws, view["fp8"], gs6, n, k)
        fp32 = orc.gemm_fp32(wq, view["fp8"], n, k).astype(np.float64) * (ws.astype(np.float64) * gs6)
    assert_close_to_oracle(out, want, fp32)


@pytest.mark.parametrize("bridge", ["exact", "fpma"])
@pytest.mark.parametrize("m,n,k", [(16, 128, 128), (1, 256, 512), (17, 384, 1024), (64, 128, 2048), (100, 512, 256),
                                   (128, 256, 384), (300, 256, 512), (520, 128, 256)])
def test_dense_matches_oracle(bridge, m, n, k):
    import tensorbridge as tb
    view, weight, q, s, wq, ws = _case(m, n, k, bridge, seed=m + n + k)
    out = tb.fp8_nvfp4_gemm(q, s, weight)
    tb.check_status()
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    _check(out, view, wq, ws, n, k)
    assert int(weight.locks.abs().sum()) == 0


@pytest.mark.parametrize("n,k", [(72, 208), (8, 16), (200, 144)])
def test_dense_ragged_n_and_k(n, k):
    import tensorbridge as tb
    view, weight, q, s, wq, ws = _case(5, n, k, "exact", seed=n)
    out = torch.full((5, n), 7.0, dtype=torch.bfloat16, device="cuda")
    res = tb.fp8_nvfp4_gemm(q, s, weight, out=out)
    tb.check_status()
    assert res is out
    _check(out, view, wq, ws, n, k)


@pytest.mark.parametrize("m,n,k,offset", [(5, 128, 256, 1), (300, 256, 384, 3), (300, 72, 208, 4),
                                          (5, 128, 256, 8), (300, 264, 384, 8)])
def test_dense_output_without_16_byte_words(m, n, k, offset):
    """The drain writes 16-byte words only when eight channels of an output row make an aligned word (channel counts
    are multiples of eight): an output that starts off a 16-byte boundary takes the 2-byte stores -- same results, and
    nothing written outside the output (the last two cases take the 16-byte words, for the same guard)."""
    import tensorbridge as tb
    view, weight, q, s, wq, ws = _case(m, n, k, "exact", seed=m + n)
    buffer = torch.full((m * n + 16,), 7.0, dtype=torch.bfloat16, device="cuda")
    out = buffer[offset:offset + m * n].view(m, n)
    res = tb.fp8_nvfp4_gemm(q, s, weight, out=out)
    tb.check_status()
    assert res is out
    _check(out, view, wq, ws, n, k)
    assert bool((buffer[:offset] == 7.0).all()) and bool((buffer[offset + m * n:] == 7.0).all())


@pytest.mark.parametrize("splits", [0, 2, 3, 7])
@pytest.mark.parametrize("block_m", [16, 64])
def test_dense_split_k_is_deterministic_and_correct(splits, block_m):
    import tensorbridge as tb
    m, n, k = 13, 256, 1792
    view, weight, q, s, wq, ws = _case(m, n, k, "exact", seed=5)
    config = tb.GemmConfig(block_m=block_m, num_stages=6, use_stream_k=splits, stream_k_aligned=3)
    outs = [tb.fp8_nvfp4_gemm(q, s, weight, config=config) for _ in range(3)]
    tb.check_status()
    _check(outs[0], view, wq, ws, n, k)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert int(weight.locks.abs().sum()) == 0


@pytest.mark.parametrize("m,n,k,num_sms", [(1024, 6144, 1024, 0), (777, 6400, 1280, 0), (512, 640, 1024, 7),
                                            (700, 384, 2048, 4), (700, 384, 2048, 7), (2048, 1152, 1024, 17)])
def test_dense_shared_last_round(m, n, k, num_sms):
    """`use_stream_k = 1` on the 256-token tile: the tiles of the last, partial round are shared out, two to four CTAs
    per tile here, each with a range of K blocks; the parts exchange FP32 partial sums and each finishes some of the
    tile's columns.  Right against the oracle, bit-identical from launch to launch (the parts are always added in the
    same order), within an FP32 rounding of the whole-tile launch -- and the launch did take the shared path (flags of
    the CTAs that published carry its tag)."""
    import ctypes
    import tensorbridge as tb
    from tensorbridge import _native as native
    lib = native.load()
    view, weight, q, s, wq, ws = _case(m, n, k, "exact", seed=m + k)
    shared = native.Config(256, 4, 1, 4, 128, 128, 1, 4, 4)
    whole = native.Config(256, 4, 0, 4, 128, 128, 1, 4, 4)
    need = lib.tb_workspace_bytes(m, n, ctypes.byref(shared))
    assert need > 0
    workspace = torch.zeros(need // 4, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    tb.check_status()

    def run(config):
        out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
        a = native.GemmArgs(q.data_ptr(), s.data_ptr(), 1, 0, weight.weight.data_ptr(), weight.scale.data_ptr(),
                            weight.global_scale.data_ptr(), weight.locks.data_ptr(), workspace.data_ptr(), need,
                            out.data_ptr(), m, n, k, native.BRIDGE_IDS["exact"], 0, 0, num_sms,
                            native.status_words(0).data_ptr())
        native.check(lib.tb_gemm_dense(stream, ctypes.byref(a), ctypes.byref(config)))
        tb.check_status()
        return out

    outs = [run(shared) for _ in range(3)]
    _check(outs[0], view, wq, ws, n, k)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    head = workspace.view(torch.int32)[:1024].cpu()
    assert int(head[0]) == 3, "three launches numbered themselves"
    assert int((head[16:] == 3).sum()) > 0, "no CTA published a partial tile: the launch ran whole tiles"
    reference = run(whole)
    difference = (outs[0].float() - reference.float()).abs()
    assert float(difference.max()) <= float(reference.float().abs().max()) * 2 ** -7
    assert float((difference > 0).float().mean()) < 0.2  # only the cut tiles can differ, by a rounding


@pytest.mark.parametrize("num_sms", [0, 1])
def test_split_k_wait_runs_out_reports_and_recovers(num_sms):
    """A bounded wait that runs out ends the launch with a status code instead of a hang.  Made to happen from the host:
    only the last of a tile's two K splits is launched (`only_split`), with a 2 ms budget, so the partial sums it waits
    for never arrive.  The kernel must return, report the split-K wait site, leave the output alone, and the next
    ordinary launch on the same workspace must be right -- with all CTAs resident (the splits share the columns) and
    on one SM (the last split reduces)."""
    import ctypes
    import tensorbridge as tb
    from tensorbridge import _native as native
    lib = native.load()
    m, n, k = 13, 256, 1792
    view, weight, q, s, wq, ws = _case(m, n, k, "exact", seed=5)
    config = native.Config(16, 4, 2, 2, 128, 128, 1, 4, 2)
    need = lib.tb_workspace_bytes(m, n, ctypes.byref(config))
    workspace = torch.zeros(need // 4, dtype=torch.float32, device="cuda")
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device="cuda")
    tb.check_status()

    def args(only_split, wait_us):
        return native.GemmArgs(q.data_ptr(), s.data_ptr(), 1, 0, weight.weight.data_ptr(), weight.scale.data_ptr(),
                               weight.global_scale.data_ptr(), weight.locks.data_ptr(), workspace.data_ptr(), need,
                               out.data_ptr(), m, n, k, native.BRIDGE_IDS["exact"], 0, 0, num_sms,
                               native.status_words(0).data_ptr(), wait_us, only_split)

    stream = torch.cuda.current_stream().cuda_stream
    a = args(only_split=2, wait_us=2000)
    native.check(lib.tb_gemm_dense(stream, ctypes.byref(a), ctypes.byref(config)))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match=f"site {9}"):
        tb.check_status()
    assert bool((out == 7.0).all())  # the waiting split wrote nothing, the other never ran
    tb.check_status()  # the status words were cleared by the failing check
    for _ in range(2):  # the same workspace, not zeroed: this launch numbers itself past the one that gave up
        a = args(only_split=0, wait_us=0)
        native.check(lib.tb_gemm_dense(stream, ctypes.byref(a), ctypes.byref(config)))
        torch.cuda.synchronize()
        tb.check_status()
        _check(out, view, wq, ws, n, k)
        out.fill_(7.0)


@pytest.mark.parametrize("bridge_warps", [(2, 2), (4, 4)])
@pytest.mark.parametrize("m,block_m,splits", [(200, 64, 3), (200, 128, 3), (131, 192, 2), (200, 192, 3), (250, 256, 5), (7, 64, 4)])
def test_dense_split_k_shared_reduction(m, block_m, splits, bridge_warps):
    """From 64-token tiles up, with a CTA per unit, the splits of a tile share the reduction of its columns: uneven
    column shares, ragged last token tiles, and the same bits on every run and as the unsplit launch's order allows."""
    import tensorbridge as tb
    n, k = 256, 1792
    view, weight, q, s, wq, ws = _case(m, n, k, "exact", seed=15)
    config = tb.GemmConfig(block_m=block_m, num_stages=6, use_stream_k=splits, stream_k_aligned=4,
                           math_warpgroups=bridge_warps[0], m_fast_tile_order=bridge_warps[1])
    outs = [tb.fp8_nvfp4_gemm(q, s, weight, config=config, enable_pdl=tb.PDL_STATIC_WEIGHTS) for _ in range(3)]
    tb.check_status()
    _check(outs[0], view, wq, ws, n, k)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("config", [dict(block_m=32, num_stages=2, stream_k_aligned=2), dict(block_m=128, num_stages=3, stream_k_aligned=4),
                                    dict(block_m=256, num_stages=4, stream_k_aligned=2), dict(block_m=16, num_stages=12, stream_k_aligned=3),
                                    dict(block_m=64, num_stages=5, stream_k_aligned=3, math_warpgroups=2, m_fast_tile_order=2),
                                    dict(block_m=64, num_stages=6, stream_k_aligned=4, math_warpgroups=4, m_fast_tile_order=4),
                                    dict(block_m=32, num_stages=7, stream_k_aligned=4, math_warpgroups=4, m_fast_tile_order=4),
                                    dict(block_m=256, num_stages=4, stream_k_aligned=3, math_warpgroups=2, m_fast_tile_order=2),
                                    dict(block_m=256, num_stages=5, stream_k_aligned=8, m_fast_tile_order=2),
                                    dict(block_m=192, num_stages=10, stream_k_aligned=4, math_warpgroups=4, m_fast_tile_order=4),
                                    dict(block_m=192, num_stages=4, stream_k_aligned=2, m_fast_tile_order=1),
                                    dict(block_m=128, num_stages=8, stream_k_aligned=8, m_fast_tile_order=1)])
def test_dense_pinned_configs(config):
    import tensorbridge as tb
    m, n, k = 40, 384, 1280
    view, weight, q, s, wq, ws = _case(m, n, k, "fpma", seed=11)
    out = tb.fp8_nvfp4_gemm(q, s, weight, config=tb.GemmConfig(**config))
    tb.check_status()
    _check(out, view, wq, ws, n, k)


def test_dense_c1_shape_exact_bridge():
    """benchmark config 1: N = K = 8192, M = 16, seed 0, exact bridge."""
    import tensorbridge as tb
    m, n, k = 16, 8192, 8192
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    x = torch.randn(m, k, generator=g).bfloat16()
    from tensorbridge.quant import fp8, nvfp4
    checkpoint = nvfp4.quantize(w.cuda())
    weight = nvfp4.prepare(*checkpoint, bridge="exact")
    q, s = fp8.quantize(x.cuda())
    out = tb.fp8_nvfp4_gemm(q, s, weight)
    tb.check_status()
    # size-independent check: FP32 matmul of the same bridged operands, on the GPU in FP32
    w_fp8 = nvfp4.bridged_fp8(weight).view(torch.float8_e4m3fn)[:n, :k].float()
    ref = (q.float() @ w_fp8.T) * (s * weight.global_scale)
    err = float((out.float() - ref).norm() / ref.norm())
    assert err <= 2e-3, err
    # the package's quantiser run on the CPU is the oracle's, bit for bit, on a slice of channels (on the GPU torch
    # divides by the constant 6 through a reciprocal, so its codes can differ from the CPU's at rounding ties)
    view = oracle_weight(w[:256], "exact")
    packed, scale, gs = nvfp4.quantize(w[:256])
    assert np.array_equal(packed.numpy(), view["packed"])
    assert np.array_equal(scale.view(torch.uint8).numpy(), view["scale"])
    # bridged bytes of the GPU-quantised checkpoint against the oracle's bridge of the same checkpoint
    gp, gsc, ggs = checkpoint
    ref_view = orc.prepare_reference_view(gp[:256].cpu().numpy(), gsc[:256].view(torch.uint8).cpu().numpy(), ggs.cpu().numpy())
    assert np.array_equal(nvfp4.bridged_fp8(weight)[:256].cpu().numpy(), ref_view["fp8"])


@pytest.mark.parametrize("m,n,k", [(16, 128, 256), (50, 256, 640), (64, 384, 1024), (9, 72, 208)])
@pytest.mark.parametrize("bridge", ["exact", "fpma"])
def test_dense_group_scales(m, n, k, bridge):
    from tensorbridge import experimental
    import tensorbridge as tb
    view, weight, q, s, wq, ws = _case(m, n, k, bridge, seed=3 * m, group=True)
    assert weight.scale.shape == (orc.pad_unit(k) // 128, orc.pad_unit(n), 8)
    out = experimental.fp8_nvfp4_group_quant_gemm(q, s, weight)
    tb.check_status()
    _check(out, view, wq, ws, n, k, group=True)
    out2 = experimental.fp8_nvfp4_group_quant_gemm(q, s.contiguous(), weight)  # K-major scales
    assert torch.equal(out, out2)


def test_dense_argument_errors():
    import tensorbridge as tb
    view, weight, q, s, wq, ws = _case(4, 128, 128, "exact")
    with pytest.raises(ValueError):
        tb.fp8_nvfp4_gemm(q[:, :64].contiguous(), s, weight)
    with pytest.raises(ValueError):
        tb.fp8_nvfp4_gemm(q, s[:2], weight)
    with pytest.raises(ValueError):
        tb.fp8_nvfp4_gemm(q, s, weight, out=torch.empty((4, 64), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        tb.fp8_nvfp4_gemm(q, s, weight, config=tb.GemmConfig(block_m=24))
    empty = tb.fp8_nvfp4_gemm(q[:0], s[:0], weight)
    assert empty.shape == (0, 128)


def test_linear_module_with_pdl():
    import tensorbridge as tb
    w = seeded_weight(256, 512, seed=21)
    layer = tb.NVFP4Linear.from_float(w.cuda(), bridge="exact")
    x = seeded_activations(24, 512, seed=22)
    out = layer(x.cuda())
    tb.check_status()
    # from_float quantises on the GPU, where torch divides by the constant 6 through a reciprocal and so can pick a
    # different code than the CPU at rounding ties: take the operands the layer really holds.
    from tensorbridge.quant import nvfp4
    view = {"fp8": nvfp4.bridged_fp8(layer.prepared()).cpu().numpy(), "global_scale6": layer.global_scale.cpu().numpy()}
    wq, ws = orc.quantize_fp8_per_token(x)
    _check(out, view, wq, ws, 256, 512)
    assert set(layer.state_dict()) == {"weight", "scale", "global_scale", "locks"}


def test_profile_sweep_writes_a_profile_that_select_config_serves(tmp_path, monkeypatch):
    import json
    import tensorbridge as tb
    from tensorbridge.jit import autotune, profiles, runtime
    n, k = 256, 512
    seen = []
    entry = autotune.sweep_dense_profile(n, k, ms=(4, 40), bridge="fpma", report=lambda m, c, us, rule_us: seen.append((m, us, rule_us)))
    assert [m for m, _, _ in seen] == [4, 40] and all(us <= rule_us for _, us, rule_us in seen)
    assert entry["segments"][-1][0] == autotune.LAST_SEGMENT and entry["n"] == 256 and entry["k"] == 512
    path = tmp_path / "swept.json"
    autotune.write_profile([entry], str(path))
    assert json.loads(path.read_text())[0]["bridge"] == "fpma"
    monkeypatch.setenv("TENSORBRIDGE_PROFILE_PATH", str(path))
    profiles.reload()
    runtime.selected_configs.clear()
    try:
        served = tb.select_config(4, n, k, bridge="fpma")
        assert served.to_list() == entry["segments"][0][1]
    finally:
        monkeypatch.delenv("TENSORBRIDGE_PROFILE_PATH")
        profiles.reload()
        runtime.selected_configs.clear()
    tb.check_status()
