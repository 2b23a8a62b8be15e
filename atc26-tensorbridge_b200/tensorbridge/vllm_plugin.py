"""vLLM plugin hooks with the names the reference registers (`tensorbridge/vllm_plugin.py:124-231,312-391,474-480` and
the entry point `tensorbridge.vllm_plugin:register` of its `pyproject.toml:53-54`).

What is here works on any `torch.nn.Module` that carries vLLM's linear-layer attributes and is tested without vLLM:
the option parser, the `tensorbridge_linear` operator body and its fake, `unsupported_linear_reason`,
`prepare_linear_layer` / `apply_linear_layer` (checkpoint tensors -> kernel layout on the layer; BF16 activations ->
output, bias added), and `TensorBridgeLinearMethod`, a linear method with vLLM's `create_weights` /
`process_weights_after_loading` / `apply` protocol for ModelOpt-style NVFP4 checkpoints (`weight`, `weight_scale`,
`weight_scale_2`).  `register()` registers the custom op when vLLM is importable.  The quantisation-config subclasses
that route a model's layers to the method (`TensorBridgeCompressedTensorsConfig`, `TensorBridgeModelOptConfig`) and the
MoE adapter are tied to internals of the vLLM version the reference pins (0.32), which is not available here, and are
not provided.
"""
from __future__ import annotations

import dataclasses
import warnings

import torch

from tensorbridge import serving
from tensorbridge.quant import nvfp4


@dataclasses.dataclass(frozen=True)
class Options:
    """`additional_config["tensorbridge"]` of a vLLM launch."""

    bridge: str = "exact"
    input_quant: str = "per_token"
    autotune: bool = False


def read_options(additional_config: dict | None) -> Options:
    raw = dict((additional_config or {}).get("tensorbridge", {}))
    unknown = set(raw) - {f.name for f in dataclasses.fields(Options)}
    if unknown:
        raise ValueError(f"unknown tensorbridge options: {sorted(unknown)}")
    options = Options(**raw)
    if options.bridge not in ("exact", "fpma") or options.input_quant not in ("per_token", "group_128"):
        raise ValueError(f"bad tensorbridge options: {options}")
    return options


def tensorbridge_linear(x: torch.Tensor, packed_weight: torch.Tensor, weight_scale: torch.Tensor,
                        global_scale: torch.Tensor, locks: torch.Tensor, output: torch.Tensor, exact_bridge: bool,
                        group_128: bool) -> None:
    """Operator body: `output = x @ dequant(weight).T`, mutating `locks` and `output` as the reference's op declares."""
    n = output.size(-1)
    k = x.size(-1)
    weight = nvfp4.NVFP4Weight(packed_weight, weight_scale, global_scale, locks, (n, k), "exact" if exact_bridge else "fpma")
    serving.linear(x.reshape(-1, k), weight, output.view(-1, n), input_quant="group_128" if group_128 else "per_token")


def register() -> None:
    """vLLM general-plugin entry point: registers `vllm.tensorbridge_linear` when vLLM is present."""
    try:
        from vllm.utils.torch_utils import direct_register_custom_op  # noqa: PLC0415
    except Exception:  # noqa: BLE001  vLLM absent or a version with another layout: nothing to register
        return
    try:
        direct_register_custom_op(op_name="tensorbridge_linear", op_func=tensorbridge_linear,
                                  mutates_args=["locks", "output"], fake_impl=tensorbridge_linear_fake)
    except Exception:  # noqa: BLE001  already registered
        return


def tensorbridge_linear_fake(x: torch.Tensor, packed_weight: torch.Tensor, weight_scale: torch.Tensor,
                             global_scale: torch.Tensor, locks: torch.Tensor, output: torch.Tensor, exact_bridge: bool,
                             group_128: bool = False) -> None:
    """Shape-only stand-in of `tensorbridge_linear` for tracing: the op writes into `output` and returns nothing."""
    return None


warned_linear_fallbacks: set[str] = set()


def unsupported_linear_reason(layer: torch.nn.Module, model_dtype=None) -> str | None:
    """Why `layer` cannot run on this library's NVFP4 dense kernels, or None when it can: they need a B200-class GPU
    (compute capability 10.0), BF16 parameters and activations, and a local weight of N % 8 == 0, K % 16 == 0."""
    if not torch.cuda.is_available() or torch.cuda.get_device_capability() != (10, 0):
        return "these kernels require a Blackwell B200-class GPU (sm_100)"
    dtype = getattr(layer, "params_dtype", torch.bfloat16)
    if dtype != torch.bfloat16:
        return f"params_dtype={dtype} (requires torch.bfloat16)"
    if hasattr(layer, "output_partition_sizes") and hasattr(layer, "input_size"):
        k = layer.input_size // getattr(layer, "tp_size", 1) if type(layer).__name__ == "RowParallelLinear" else layer.input_size
        k = getattr(layer, "input_size_per_partition", k)
        n = sum(layer.output_partition_sizes)
        if n <= 0 or k <= 0 or n % 8 or k % nvfp4.GROUP_SIZE:
            return f"local linear shape (N={n}, K={k}) requires N % 8 == 0 and K % 16 == 0"
    if model_dtype is not None and model_dtype not in (torch.bfloat16, "bfloat16", "auto"):
        return f"model dtype={model_dtype} (requires bfloat16)"
    return None


def warn_linear_fallback(prefix: str | None, reason: str) -> None:
    """One warning per distinct reason that a layer is left to the framework's own method."""
    if reason not in warned_linear_fallbacks:
        warned_linear_fallbacks.add(reason)
        warnings.warn(f"tensorbridge: linear layer {prefix or '<linear>'} skipped ({reason}); the framework's own method serves it",
                      stacklevel=3)


def prepare_linear_layer(layer: torch.nn.Module, packed: torch.Tensor, scale: torch.Tensor, global_scale: torch.Tensor,
                         scale_convention: str, bridge: str, input_quant: str = "per_token",
                         capture_sizes: list[int] | None = None) -> None:
    """Put the kernel layout of a loaded NVFP4 linear layer on `layer` as the buffers `tensorbridge_weight`,
    `tensorbridge_scale`, `tensorbridge_global_scale`, `tensorbridge_locks` (the caller drops the checkpoint tensors).
    `layer.logical_widths` gives the fused shards, `capture_sizes` the token counts a CUDA graph will capture: with
    `TENSORBRIDGE_AUTOTUNE=1` they are measured now."""
    prepared = serving.prepare_linear(packed, scale, global_scale, bridge, scale_convention,
                                      getattr(layer, "logical_widths", None), input_quant=input_quant)
    for name in ("weight", "scale", "global_scale", "locks"):
        layer.register_buffer(f"tensorbridge_{name}", getattr(prepared, name))
    layer.tensorbridge_shape = prepared.shape
    if capture_sizes:
        serving.autotune_prepared(capture_sizes)


def apply_linear_layer(layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None, bridge: str,
                       input_quant: str = "per_token") -> torch.Tensor:
    """`x[..., K]` (BF16) through the prepared layer: `[..., N]`, bias added when given.  Goes through
    `torch.ops.vllm.tensorbridge_linear` when `register()` has registered it, else calls the operator body."""
    if x.dtype != torch.bfloat16:
        raise ValueError(f"tensorbridge linear expects bfloat16 activations, got {x.dtype}")
    n = getattr(layer, "output_size_per_partition", None) or layer.tensorbridge_shape[0]
    output = torch.empty((x.numel() // x.shape[-1], n), dtype=torch.bfloat16, device=x.device)
    op = tensorbridge_linear
    vllm_ops = getattr(torch.ops, "vllm", None)
    if vllm_ops is not None and hasattr(vllm_ops, "tensorbridge_linear"):
        op = vllm_ops.tensorbridge_linear
    op(x.reshape(-1, x.shape[-1]), layer.tensorbridge_weight, layer.tensorbridge_scale, layer.tensorbridge_global_scale,
       layer.tensorbridge_locks, output, bridge == "exact", input_quant == "group_128")
    output = output.reshape(*x.shape[:-1], n)
    return output if bias is None else output + bias


class TensorBridgeLinearMethod:
    """Linear method for ModelOpt-style NVFP4 checkpoints with vLLM's protocol (`create_weights`,
    `process_weights_after_loading`, `apply`): registers `weight` uint8 `[N, K/2]`, `weight_scale` E4M3 `[N, K/16]` and
    `weight_scale_2` FP32 `[shards]` (the per-shard global multiplier) for the loader, then swaps them for the kernel
    layout.  It does not subclass vLLM's `LinearMethodBase`: an adapter for a given vLLM version derives from both."""

    def __init__(self, bridge: str = "exact", input_quant: str = "per_token") -> None:
        self.bridge, self.input_quant = bridge, input_quant

    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int, output_partition_sizes: list[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra) -> None:
        n = sum(output_partition_sizes)
        if n % 8 or input_size_per_partition % nvfp4.GROUP_SIZE:
            raise ValueError(f"local linear shape (N={n}, K={input_size_per_partition}) requires N % 8 == 0 and K % 16 == 0")
        layer.logical_widths = list(output_partition_sizes)
        layer.input_size_per_partition, layer.output_size_per_partition = input_size_per_partition, n
        parameter = lambda t: torch.nn.Parameter(t, requires_grad=False)  # noqa: E731
        layer.register_parameter("weight", parameter(torch.empty((n, input_size_per_partition // 2), dtype=torch.uint8)))
        layer.register_parameter("weight_scale", parameter(torch.empty((n, input_size_per_partition // nvfp4.GROUP_SIZE),
                                                                       dtype=torch.float8_e4m3fn)))
        layer.register_parameter("weight_scale_2", parameter(torch.empty(len(output_partition_sizes), dtype=torch.float32)))

    def process_weights_after_loading(self, layer: torch.nn.Module, capture_sizes: list[int] | None = None) -> None:
        packed, scale, multiplier = layer.weight.data, layer.weight_scale.data, layer.weight_scale_2.data
        prepare_linear_layer(layer, packed, scale, multiplier, "multiplier", self.bridge, self.input_quant, capture_sizes)
        del layer.weight, layer.weight_scale, layer.weight_scale_2

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return apply_linear_layer(layer, x, bias, self.bridge, self.input_quant)
