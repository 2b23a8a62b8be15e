"""Kernel configuration types shared by the Python API and the native library, and the source generator of the JIT.

Mirrors the names of the reference's `tensorbridge/jit/codegen.py:15-138` (`Bridge`, `GroupedLayout`, `LAYOUT_IDS`,
`pad_to_unit`, `GemmConfig`, `KernelSource`, `generate`, `generate_pgroup`).  The reference generates one translation
unit per weight shape because its kernels take `(N, K)` as template arguments.  Here shapes, layouts and ring depths
are run-time parameters, the common template points are compiled ahead of time into libtensorbridge_b200.so, and
`generate` emits a translation unit only for the template point a config names -- (token tile, bridge, scale
granularity, bridge warps, teams) -- which `tensorbridge.jit.compiler` compiles with NVRTC when the library has no
instance of it (token tiles of 48, 96, 160, 224 tokens, sixteen bridge warps in two teams, ...).
"""
from __future__ import annotations

import dataclasses
from typing import Literal

Bridge = Literal["fpma", "exact"]
GroupedLayout = Literal["dense", "indexed", "contiguous", "masked"]
LAYOUT_IDS: dict[str, int] = {"dense": 0, "indexed": 1, "contiguous": 2, "masked": 3}
WEIGHT_UNIT = 128  # weights are zero padded to whole 128 x 128 blocks


def pad_to_unit(size: int) -> int:
    """`size` rounded up to a multiple of the 128-wide weight block."""
    return (size + WEIGHT_UNIT - 1) // WEIGHT_UNIT * WEIGHT_UNIT


@dataclasses.dataclass(frozen=True)
class GemmConfig:
    """The nine configuration fields, in the reference's wire order (profiles store them positionally).

    On B200 they are read as: `block_m` token tile (16/32/64/128/256); `num_stages` depth of the weight ring (the token ring takes the
    rest of shared memory);
    `use_stream_k` dense GEMM: 0 whole tiles, 1 the tiles of the last partial round shared out in K blocks (256-token
    tiles, more tiles than SMs; never picked by the rule), 2..16 that many deterministic K splits of every tile; `m_fast_tile_order`
    number of bridge teams that alternate K blocks (0/1, 2 or 4); `block_k` 128; `block_n` 128; `ctas_per_sm` 1; `stream_k_aligned` bridged FP8 weight
    tiles kept in tensor memory (2..8, 0 = default 4); `math_warpgroups` bridge warps / 4 (2 or 4).
    """

    block_m: int = 128
    num_stages: int = 4
    use_stream_k: int = 0
    m_fast_tile_order: int = 0
    block_k: int = 128
    block_n: int = 128
    ctas_per_sm: int = 1
    stream_k_aligned: int = 0
    math_warpgroups: int = 2

    @classmethod
    def from_list(cls, values: list[int]) -> "GemmConfig":
        names = [f.name for f in dataclasses.fields(cls)]
        if len(values) != len(names):
            raise ValueError(f"GemmConfig takes {len(names)} values, got {len(values)}")
        return cls(**{name: int(value) for name, value in zip(names, values)})

    def to_list(self) -> list[int]:
        return [int(getattr(self, f.name)) for f in dataclasses.fields(self)]


@dataclasses.dataclass(frozen=True)
class KernelPoint:
    """One point of the kernel template `tb::gemm_body<block_m, exact, group_scales, bridge_warps, teams>`."""

    block_m: int
    exact: bool
    group_scales: bool
    bridge_warps: int
    teams: int

    @property
    def entry(self) -> str:
        return f"tb_jit_m{self.block_m}_{'exact' if self.exact else 'fpma'}_{'g' if self.group_scales else 't'}_w{self.bridge_warps}_t{self.teams}"

    @property
    def threads(self) -> int:
        return ((8 if self.block_m >= 64 else 4) + self.bridge_warps + 3) * 32


@dataclasses.dataclass(frozen=True)
class KernelSource:
    source: str
    name: str  # entry point of the translation unit (a plain C name: no lowered-name lookup is needed)
    point: KernelPoint


# Token tiles the ahead-of-time library holds for every bridge arrangement in AOT_BRIDGES.
AOT_BLOCK_M = (16, 32, 64, 128, 192, 256)
AOT_BRIDGES = ((8, 1), (8, 2), (16, 4))  # (bridge warps, teams)


def kernel_point(config: GemmConfig, bridge: Bridge = "exact", group_scales: bool = False) -> KernelPoint:
    """The template point `config` launches."""
    teams = 1 if config.m_fast_tile_order <= 1 else int(config.m_fast_tile_order)
    return KernelPoint(int(config.block_m), bridge == "exact", bool(group_scales), int(config.math_warpgroups) * 4, teams)


def is_ahead_of_time(point: KernelPoint) -> bool:
    tiles = AOT_BLOCK_M[:4] if point.group_scales else AOT_BLOCK_M
    return point.block_m in tiles and (point.bridge_warps, point.teams) in AOT_BRIDGES


def validate_point(point: KernelPoint) -> None:
    bm = point.block_m
    if bm < 16 or bm > 256 or bm % 16 or (bm >= 64 and bm % 32):
        raise ValueError(f"block_m must be a multiple of 16 up to 256 (of 32 from 64 up), got {bm}")
    if point.bridge_warps not in (8, 16) or point.teams < 1 or point.bridge_warps % point.teams or (point.bridge_warps // point.teams) % 4:
        raise ValueError(f"{point.bridge_warps} bridge warps in {point.teams} teams: teams of 4, 8 or 16 warps of 8 or 16")
    if point.group_scales and bm > 128:
        raise ValueError("[1,128] activation scales take token tiles up to 128")
    accumulators = (min(384 // bm, 8) if point.group_scales else (2 if 2 * bm + 64 <= 512 else 1)) * bm
    if accumulators + 32 * max(2, point.teams) > 512:
        raise ValueError(f"{bm} tokens leave no tensor memory for a bridged tile per team ({point.teams} teams)")


def generate(n: int, k: int, config: GemmConfig, num_experts: int = 0, layout: GroupedLayout = "dense",
             bridge: Bridge = "exact", *, group_scales: bool = False) -> KernelSource:
    """The translation unit for `config`: one entry point that wraps the template point it names.  `n`, `k`,
    `num_experts` and `layout` are accepted for the reference's signature; they are run-time parameters of the kernel
    here and do not change the source."""
    if layout not in LAYOUT_IDS:
        raise ValueError(f"unknown layout {layout!r}")
    point = kernel_point(config, bridge, group_scales)
    validate_point(point)
    cpp = lambda flag: "true" if flag else "false"  # noqa: E731
    source = f"""\
#include "tb_gemm.cuh"

extern "C" __global__ void __launch_bounds__({point.threads}, 1) {point.entry}(const __grid_constant__ tb::GemmParams p) {{
    tb::gemm_body<{point.block_m}, {cpp(point.exact)}, {cpp(point.group_scales)}, {point.bridge_warps}, {point.teams}>(p);
}}
"""
    return KernelSource(source, point.entry, point)


def generate_pgroup(n: int, k: int, config: GemmConfig, scale_m_major: bool = True, bridge: Bridge = "exact",
                    num_experts: int = 0, layout: GroupedLayout = "dense") -> KernelSource:
    """`generate` for `[1,128]` activation scales (the kernel reads the scale strides at run time, so
    `scale_m_major` does not change the source)."""
    del scale_m_major
    return generate(n, k, config, num_experts, layout, bridge, group_scales=True)
