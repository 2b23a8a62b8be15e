"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every declared symbol, and the host-only
entry points (selection rule, workspace size, argument validation) behave."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__
    __graft_entry__.build()
    from tensorbridge import _native
    return _native.load()


def test_every_declared_symbol_is_exported(lib):
    from tensorbridge import _native
    header = open(os.path.join(ROOT, "include", "tensorbridge_b200.h")).read()
    declared = set(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_native.SYMBOLS), declared ^ set(_native.SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert b"sm_100a" in lib.tb_version()


def test_struct_sizes_match_header(lib):
    from tensorbridge import _native
    assert ctypes.sizeof(_native.Config) == 36
    assert ctypes.sizeof(_native.Problem) == 48
    assert ctypes.sizeof(_native.GemmArgs) == 21 * 8  # + wait_us / only_split, row_target, peer_out, peer_count / reserved
    assert ctypes.sizeof(_native.Routing) == 8 + 5 * 8 + 8 + 8 + 16


def test_rule_small_m_splits_k_and_large_m_does_not(lib):
    from tensorbridge.jit import runtime
    small = runtime.rule_config(16, 6144, 7168, 148)
    assert small.block_m == 16 and small.use_stream_k == 3  # 48 tiles x 3 splits = 144 CTAs
    assert runtime.rule_config(64, 6144, 7168, 148).block_m == 64
    large = runtime.rule_config(8192, 6144, 7168, 148)
    assert large.block_m == 256 and large.block_n == 128 and large.use_stream_k == 0
    assert runtime.rule_config(16, 6144, 7168, 148, split_k_override=0).use_stream_k == 0
    grouped = runtime.rule_config(4096, 4096, 7168, 148, 32, "masked")
    assert grouped.use_stream_k == 0 and grouped.block_m == 256  # twice the mean of 128 rows per expert
    assert runtime.rule_config(16384, 7168, 2048, 148, 128, "contiguous", True).block_m == 128  # [1,128] scales: up to 128 tokens
    for m in (1, 300, 5000):
        cfg = runtime.rule_config(m, 6144, 7168, 148)
        assert 2 <= cfg.num_stages <= 16 and cfg.block_n == 128 and cfg.block_k == 128
    with pytest.raises(ValueError):
        runtime.rule_config(16, 0, 128, 148)


def test_workspace_bytes(lib):
    from tensorbridge import _native
    cfg = _native.Config(16, 8, 3, 0, 128, 128, 1, 3, 2)
    assert lib.tb_workspace_bytes(16, 6144, ctypes.byref(cfg)) == 4096 + 48 * 3 * 16 * 128 * 8
    cfg.use_stream_k = 0
    assert lib.tb_workspace_bytes(16, 6144, ctypes.byref(cfg)) == 0
    # a token tile the library does not have is answered with 0, not a division by zero
    for bad in (0, 24, -16):
        cfg = _native.Config(bad, 8, 3, 0, 128, 128, 1, 3, 2)
        assert lib.tb_workspace_bytes(16, 6144, ctypes.byref(cfg)) == 0


def test_static_scratch_entry_validates_before_sizing(lib):
    """The allocation-free entry point refuses an unknown token tile with an error code, and sizes its scratch by the
    splits the launch really makes: more splits than K blocks, or [1,128] scales, need little or none and are not
    refused for size (they fail later, on the null tensors, with the ordinary message)."""
    from tensorbridge import _native
    args = _native.GemmArgs()
    args.rows, args.n, args.k = 256, 2048, 256
    cfg = _native.Config(0, 4, 8, 2, 128, 128, 1, 3, 2)
    assert lib.tb_gemm_dense_static_scratch(None, ctypes.byref(args), ctypes.byref(cfg)) == _native.ERR_INVALID
    assert b"block_m" in lib.tb_last_error()
    # 16 tiles x 16 splits x 256 x 128 x 8 B = 64 MiB by the config, but K = 256 allows only two splits: 8 MiB + header
    cfg = _native.Config(256, 4, 16, 2, 128, 128, 1, 3, 2)
    args.rows, args.n = 256, 1024  # 8 tiles x 2 splits x 256 x 128 x 8 B = 4 MiB
    assert lib.tb_workspace_bytes(256, 1024, ctypes.byref(cfg)) > 8 << 20
    # past the size check the call goes on to the device (no GPU here: a CUDA error) or to the null tensors
    assert lib.tb_gemm_dense_static_scratch(None, ctypes.byref(args), ctypes.byref(cfg)) != _native.OK
    assert b"split-K scratch" not in lib.tb_last_error()
    args.group_scales = 1
    args.rows, args.n = 256, 2048
    assert lib.tb_gemm_dense_static_scratch(None, ctypes.byref(args), ctypes.byref(cfg)) != _native.OK
    assert b"split-K scratch" not in lib.tb_last_error()
    args.group_scales = 0  # and the same shape with per-token scales is refused for its size
    cfg.use_stream_k = 2
    args.k = 1024
    args.rows, args.n = 512, 2048  # 32 tiles x 2 splits x 256 x 128 x 8 B = 16 MiB
    assert lib.tb_gemm_dense_static_scratch(None, ctypes.byref(args), ctypes.byref(cfg)) == _native.ERR_INVALID
    assert b"split-K scratch" in lib.tb_last_error()


def test_validation_needs_no_gpu(lib):
    from tensorbridge import _native
    args = _native.GemmArgs()
    cfg = _native.Config(24, 8, 0, 0, 128, 128, 1, 3, 2)
    args.rows, args.n, args.k = 4, 128, 100
    assert lib.tb_gemm_dense(None, ctypes.byref(args), ctypes.byref(cfg)) == _native.ERR_INVALID
    assert lib.tb_last_error() != b""
    assert lib.tb_gemm_grouped(None, ctypes.byref(args), None, ctypes.byref(cfg)) == _native.ERR_INVALID
    assert lib.tb_quantize_fp8(None, None, 0, 0, -1, 8, 0, None, None, 0, 0) == _native.ERR_INVALID
    args.rows = 0
    assert lib.tb_gemm_dense(None, ctypes.byref(args), ctypes.byref(cfg)) == _native.OK  # empty input: no launch


def test_gemm_config_wire_format():
    from tensorbridge import GemmConfig
    cfg = GemmConfig.from_list([64, 10, 3, 0, 128, 128, 1, 3, 2])
    assert cfg.block_m == 64 and cfg.use_stream_k == 3 and cfg.to_list() == [64, 10, 3, 0, 128, 128, 1, 3, 2]
    with pytest.raises(ValueError):
        GemmConfig.from_list([1, 2, 3])


def test_profile_lookup(tmp_path, monkeypatch):
    import json
    from tensorbridge.jit import profiles
    path = tmp_path / "p.json"
    path.write_text(json.dumps([{"device": "NVIDIA B200", "num_sms": 148, "n": 6272, "k": 7296, "num_experts": 0,
                                 "layout": "dense", "group_scales": False, "bridge": "exact",
                                 "segments": [[16, [16, 12, 3, 0, 128, 128, 1, 3, 2]], [256, [64, 8, 2, 0, 128, 128, 1, 3, 2]]]}]))
    monkeypatch.setenv("TENSORBRIDGE_PROFILE_PATH", str(path))
    profiles.reload()
    assert profiles.lookup("NVIDIA B200", 148, 6272, 7296, 0, "dense", False, "exact", 9).block_m == 16
    assert profiles.lookup("NVIDIA B200", 148, 6272, 7296, 0, "dense", False, "exact", 100).block_m == 64
    assert profiles.lookup("NVIDIA B200", 148, 6272, 7296, 0, "dense", False, "exact", 1000) is None
    assert profiles.lookup("NVIDIA B200", 148, 6272, 7296, 0, "dense", False, "fpma", 9) is None
    monkeypatch.delenv("TENSORBRIDGE_PROFILE_PATH")
    profiles.reload()


def test_align_routes_matches_oracle_on_cpu():
    import numpy as np
    import torch
    import tb_oracle as orc
    from tensorbridge.routing import align_routes, padded_capacity
    rng = np.random.default_rng(0)
    for tokens, top_k, experts, block_m in [(1, 2, 4, 16), (9, 4, 6, 16), (70, 3, 8, 64), (33, 8, 128, 32)]:
        topk = np.stack([rng.choice(experts, size=top_k, replace=False) for _ in range(tokens)])
        want_ids, want_experts, want_padded = orc.align_routes(topk, experts, block_m)
        got = align_routes(torch.from_numpy(topk), experts, block_m)
        n = int(got.num_tokens_padded)
        assert n == int(want_padded[0]) and got.sorted_ids.numel() == padded_capacity(tokens * top_k, experts, block_m)
        assert np.array_equal(got.sorted_ids[:n].numpy(), want_ids)
        assert np.array_equal(got.expert_ids[: n // block_m].numpy(), want_experts)
        assert (got.sorted_ids[n:] == tokens * top_k).all()
    # routes of experts outside [0, E) are dropped
    got = align_routes(torch.tensor([[0, 5], [7, 1]]), 2, 16)
    assert int(got.num_tokens_padded) == 32 and sorted(got.sorted_ids[:32][got.sorted_ids[:32] < 4].tolist()) == [0, 3]


def test_profile_sweeper_candidates_and_segments():
    """Host logic of the profile sweeper: the rule's pick first, every candidate a legal config, segments merged."""
    from tensorbridge.jit import autotune
    from tensorbridge.jit.codegen import GemmConfig
    from tensorbridge.jit.runtime import rule_config
    for m in (1, 16, 100, 160, 300, 2048):
        cands = autotune.dense_candidates(m, 6144, 7168, 148)
        assert cands[0] == rule_config(m, 6144, 7168, 148)
        assert len(set(cands)) == len(cands) > 4
        for c in cands:
            assert c.block_m in (16, 32, 64, 128, 192, 256) and (c.block_m >= m or m > 128)
            assert (c.math_warpgroups, c.m_fast_tile_order) in ((2, 2), (4, 4)) and c.stream_k_aligned in (4, 8)
            assert c.use_stream_k == 0 or 2 <= c.use_stream_k <= 16
    a, b = GemmConfig(block_m=16), GemmConfig(block_m=32)
    segments = autotune.merge_segments([(8, b), (1, a), (2, a), (4, b), (16, a)])
    assert segments == [[2, a.to_list()], [8, b.to_list()], [autotune.LAST_SEGMENT, a.to_list()]]
