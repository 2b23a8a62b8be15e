"""Config selection front end: autotune override -> profile -> the native B200 rule, cached per shape.

Keeps the call signature of the reference's `select_config` (`tensorbridge/jit/runtime.py:73-108`).  There is no
NVRTC step: `get_kernel` / `get_grouped_kernel` of the reference resolve to template instances that already live in
libtensorbridge_b200.so, so selection is the whole "JIT" front end here.
"""
from __future__ import annotations

import ctypes
import functools
import os

import torch

from tensorbridge import _native
from tensorbridge.jit import codegen, profiles
from tensorbridge.jit.codegen import Bridge, GemmConfig

SelectionKey = tuple
selected_configs: dict[SelectionKey, GemmConfig] = {}


_num_sms: dict[tuple[int, str | None], int] = {}


def get_num_sms(device: int | None = None) -> int:
    """SMs available to a launch on `device`, after the `TENSORBRIDGE_NUM_SMS` cap (looked up once per device and
    value of that variable)."""
    device = torch.cuda.current_device() if device is None else device
    key = (device, os.environ.get("TENSORBRIDGE_NUM_SMS"))
    hit = _num_sms.get(key)
    if hit is None:
        out = ctypes.c_int(0)
        _native.check(_native.load().tb_num_sms(int(device), ctypes.byref(out)))
        hit = _num_sms[key] = out.value
    return hit


@functools.cache
def _device_name(device: int) -> str:
    return str(torch.cuda.get_device_name(device))


def rule_config(m: int, n: int, k: int, num_sms: int, num_experts: int = 0, layout: str = "dense",
                group_scales: bool = False, split_k_override: int = -1) -> GemmConfig:
    """The native selection rule alone (needs no GPU)."""
    problem = _native.Problem(max(int(m), 1), int(n), int(k), int(num_sms), int(num_experts),
                              codegen.LAYOUT_IDS[layout], int(group_scales), int(split_k_override))
    config = _native.Config()
    _native.check(_native.load().tb_select_config(ctypes.byref(problem), ctypes.byref(config)))
    return GemmConfig.from_list([getattr(config, name) for name, _ in _native.Config._fields_])


def select_config(
    m: int, n: int, k: int, num_experts: int = 0, layout: codegen.GroupedLayout = "dense", device: int | None = None,
    *, bridge: Bridge = "exact", top_k: int = 1, use_stream_k: bool | None = None, group_scales: bool = False,
) -> GemmConfig:
    """The config serving this shape on `device`: an autotune override, else a profile entry, else the rule.
    `n`, `k` are the weight's unpadded sizes, `m` the (routed) row count.  `use_stream_k` forces the dense K split
    off or on and bypasses overrides and profiles; grouped layouts never split K."""
    device = torch.cuda.current_device() if device is None else device
    num_sms = get_num_sms(device)
    key = (device, num_sms, m, n, k, num_experts, layout, bridge, top_k, use_stream_k, group_scales)
    hit = selected_configs.get(key)
    if hit is not None:
        return hit
    if layout not in codegen.LAYOUT_IDS:
        raise ValueError(f"unknown layout {layout!r}")
    config = None
    if use_stream_k is None:
        config = profiles.lookup(_device_name(device), num_sms, codegen.pad_to_unit(n), codegen.pad_to_unit(k),
                                 num_experts, layout, group_scales, bridge, max(m, 1))
    if config is None:
        override = 0 if layout != "dense" else -1 if use_stream_k is None else (0 if not use_stream_k else -2)
        if override == -2:  # forced on: let the rule size it, but at least two splits
            config = rule_config(m, n, k, num_sms, num_experts, layout, group_scales, -1)
            if config.use_stream_k <= 1:
                config = rule_config(m, n, k, num_sms, num_experts, layout, group_scales, 2)
        else:
            config = rule_config(m, n, k, num_sms, num_experts, layout, group_scales, override)
    selected_configs[key] = config
    return config


def override_config(m: int, n: int, k: int, config: GemmConfig, device: int, num_experts: int = 0,
                    layout: codegen.GroupedLayout = "dense", bridge: Bridge = "exact", top_k: int = 1,
                    group_scales: bool = False) -> None:
    """Serve this shape with `config` from now on (what autotune records)."""
    key = (device, get_num_sms(device), m, n, k, num_experts, layout, bridge, top_k, None, group_scales)
    selected_configs[key] = config
