"""Config selection front end (autotune override -> profile -> the native B200 rule, cached per shape) and the kernel
registry of the JIT.

Keeps the call signatures of the reference's `select_config` (`tensorbridge/jit/runtime.py:73-108`) and of its
`get_kernel` / `get_grouped_kernel` (`:162-244`).  A config that names a template point the library was built with
resolves to that ahead-of-time instance; any other point is generated (`codegen.generate`), compiled with NVRTC
(`compiler.build`, cached on disk), loaded with the driver API and registered with the library
(`tb_register_kernel`), after which launches with that config run it.
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


# ---- kernels compiled at run time --------------------------------------------------------------------------------
loaded_kernels: dict[tuple, "LoadedKernel"] = {}


class LoadedKernel:
    """A module loaded on one device and the function registered with the library (the module must stay loaded)."""

    def __init__(self, device: int, point: codegen.KernelPoint, compiled, module, function) -> None:
        self.device, self.point, self.compiled, self.module, self.function = device, point, compiled, module, function


def _driver_check(result, what: str) -> None:
    from cuda.bindings import driver  # noqa: PLC0415

    if result != driver.CUresult.CUDA_SUCCESS:
        raise RuntimeError(f"{what} failed: {result}")


def get_kernel(n: int, k: int, config: GemmConfig, device: int | None = None, *, bridge: Bridge = "exact",
               group_scales: bool = False, num_experts: int = 0, layout: codegen.GroupedLayout = "dense") -> "LoadedKernel | None":
    """Make sure the library can launch `config` on `device`: returns None when the ahead-of-time library holds the
    template point, else the kernel compiled (or fetched from the disk cache), loaded and registered for it.  Call it
    outside CUDA-graph capture; launches with `config` need nothing further."""
    from cuda.bindings import driver  # noqa: PLC0415

    from tensorbridge.jit import compiler  # noqa: PLC0415

    device = torch.cuda.current_device() if device is None else device
    point = codegen.kernel_point(config, bridge, group_scales)
    codegen.validate_point(point)
    if codegen.is_ahead_of_time(point):
        return None
    key = (device, point)
    hit = loaded_kernels.get(key)
    if hit is not None:
        return hit
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("get_kernel compiles and loads a module: call it before CUDA graph capture, not during it")
    compiled = compiler.build(codegen.generate(n, k, config, num_experts, layout, bridge, group_scales=group_scales))
    with torch.cuda.device(device):
        torch.cuda.current_stream()  # makes sure the device's primary context is current
        with open(compiled.cubin_path, "rb") as handle:
            image = handle.read()
        result, module = driver.cuModuleLoadData(image)
        _driver_check(result, "cuModuleLoadData")
        result, function = driver.cuModuleGetFunction(module, compiled.entry.encode())
        _driver_check(result, "cuModuleGetFunction")
        _driver_check(driver.cuFuncSetAttribute(function, driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                                227 * 1024)[0], "cuFuncSetAttribute")
        if point.group_scales and point.block_m == 128 and point.bridge_warps == 8:
            # this instance moves registers from its bridge warpgroups to its epilogue warpgroups (64 and 128 a thread):
            # with fewer than 96 of its own the epilogue's request could never be met
            result, registers = driver.cuFuncGetAttribute(driver.CUfunction_attribute.CU_FUNC_ATTRIBUTE_NUM_REGS, function)
            _driver_check(result, "cuFuncGetAttribute")
            if registers < 96:
                raise RuntimeError(f"{compiled.entry} was compiled with {registers} registers a thread; its register hand-over needs 96")
        native_key = _native.KernelKey(device, point.block_m, int(point.exact), int(point.group_scales), point.bridge_warps, point.teams)
        _native.check(_native.load().tb_register_kernel(ctypes.byref(native_key), ctypes.c_void_p(int(function))))
    loaded = loaded_kernels[key] = LoadedKernel(device, point, compiled, module, function)
    return loaded


def get_grouped_kernel(n: int, k: int, num_experts: int, layout: codegen.GroupedLayout, config: GemmConfig,
                       device: int | None = None, *, bridge: Bridge = "exact", group_scales: bool = False) -> "LoadedKernel | None":
    """`get_kernel` for a grouped call (the kernel is the same template; the layout is a run-time parameter)."""
    return get_kernel(n, k, config, device, bridge=bridge, group_scales=group_scales, num_experts=num_experts, layout=layout)
