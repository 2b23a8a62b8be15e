"""Checkpoint-facing helpers that do not depend on an inference framework.

    share_global_scale   one global scale for the shards of a fused weight
    prepare_linear       once per linear layer, when its weights are loaded
    prepare_moe          once per MoE layer, after checkpoint sharding
    linear               in a layer's forward: quantise BF16 activations, then the GEMM with PDL

    moe_forward_*        two grouped GEMMs around activation and quantisation, into caller buffers

Names, arguments and conventions follow the reference's `tensorbridge/serving.py:33-170,173-353,356-703`.
`precompile_prepared` loads (compiling with NVRTC where the library has no ahead-of-time instance) every kernel the
selection can pick for the prepared shapes; `autotune_prepared` measures the prepared dense shapes.
"""
from __future__ import annotations

import dataclasses
import os
import warnings
from collections.abc import Callable, Sequence
from typing import Literal, TypedDict

import torch

from tensorbridge import experimental
from tensorbridge.gemm import (PDL_STATIC_WEIGHTS, ContiguousRouting, IndexedRouting, MaskedRouting, fp8_nvfp4_gemm,
                               fp8_nvfp4_grouped_gemm)
from tensorbridge.jit import autotune as _autotune
from tensorbridge.jit import codegen, runtime
from tensorbridge.jit.codegen import Bridge, GemmConfig
from tensorbridge.quant import fp8, nvfp4

@dataclasses.dataclass(frozen=True, order=True)
class DenseShape:
    """A dense weight shape prepared on `device` (`tensorbridge/serving.py:33-42`)."""

    device: int
    n: int
    k: int
    bridge: Bridge
    input_quant: fp8.InputQuant = "per_token"


@dataclasses.dataclass(frozen=True, order=True)
class GroupedShape:
    """One prepared projection of a MoE layer (`tensorbridge/serving.py:44-59`): `top_k` is the layer's routes per
    token (turns a captured token count into routed rows), `input_top_k` the indexed gather factor of this projection
    (the down projection reads one row per route)."""

    device: int
    n: int
    k: int
    num_experts: int
    top_k: int
    input_top_k: int
    layout: Literal["indexed", "contiguous", "masked"]
    bridge: Bridge
    dispatch_ranks: int
    num_global_experts: int
    input_quant: fp8.InputQuant = "per_token"


DenseTunedKey = tuple

# Bookkeeping per process, under the reference's names: dense shapes and layers prepared, shapes autotune serves, calls
# captured without a measured config, grouped projections prepared and tuned.
prepared_shapes: set[DenseShape | tuple] = set()
prepared_layers = 0
tuned: set[DenseTunedKey] = set()
captured_untuned = 0
warned_untuned: set = set()
prepared_grouped: set[GroupedShape] = set()
tuned_grouped: set[tuple[GroupedShape, int, int]] = set()
precompiled_dense: set[tuple[DenseShape, int, int]] = set()
precompiled_grouped: set[tuple[GroupedShape, int, int]] = set()
stream_locks: dict[tuple[int, int], torch.Tensor] = {}


def autotune_enabled() -> bool:
    return os.environ.get("TENSORBRIDGE_AUTOTUNE") == "1"


def locks_for_current_stream(fallback: torch.Tensor) -> torch.Tensor:
    """The lock array a launch on the current stream should carry.  The reference hands every stream its own Stream-K
    counters here (`tensorbridge/serving.py:84-97`); the sm_100a kernels keep no counters in `locks` (the split-K
    reduction works on tagged partial sums in per-stream scratch, see `tensorbridge.gemm`), so the weight's own array
    is returned and nothing is allocated."""
    return fallback


def normalize_dense_shape(entry: DenseShape | tuple) -> DenseShape:
    """`prepared_shapes` entries are `DenseShape`s; older 4-tuples `(device, n, k, bridge)` are accepted."""
    if isinstance(entry, DenseShape):
        return entry
    if len(entry) == 5:
        return DenseShape(*entry)
    device, n, k, bridge = entry
    return DenseShape(device, n, k, bridge, "per_token")


def dense_tuned_key(device: int, num_sms: int, n: int, k: int, m: int, bridge: Bridge, input_quant: fp8.InputQuant) -> tuple:
    base = (device, num_sms, n, k, m, bridge)
    return base if input_quant == "per_token" else base + (input_quant,)


def share_global_scale(weight_scale: torch.Tensor, global_scales: torch.Tensor, shard_sizes: Sequence[int]
                       ) -> tuple[torch.Tensor, torch.Tensor]:
    """The kernel applies one global scale per weight (per expert).  `weight_scale` is E4M3 `[..., N, K/16]` with the
    shards of a fused weight concatenated along N and `global_scales` their multipliers `[..., S]`.  The shared scale
    is the largest; every other shard's group scales are multiplied by own/largest and rounded to the nearest E4M3.
    Shards that already agree are returned unchanged."""
    if sum(shard_sizes) != weight_scale.shape[-2] or len(shard_sizes) != global_scales.shape[-1]:
        raise ValueError(f"shards {list(shard_sizes)} do not match the {weight_scale.shape[-2]} channels and "
                         f"{global_scales.shape[-1]} global scales")
    largest = global_scales.amax(-1, keepdim=True)
    if torch.equal(global_scales, largest.expand_as(global_scales)):
        return weight_scale, largest.squeeze(-1)
    per_channel = (global_scales / largest).repeat_interleave(
        torch.tensor(list(shard_sizes), device=global_scales.device), dim=-1)
    rescaled = (weight_scale.float() * per_channel.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return rescaled, largest.squeeze(-1)


def prepare_linear(weight_packed: torch.Tensor, weight_scale: torch.Tensor, weight_global_scale: torch.Tensor,
                   bridge: Bridge = "exact", scale_convention: Literal["inverse", "multiplier"] = "inverse",
                   shard_sizes: Sequence[int] | None = None, *, input_quant: fp8.InputQuant = "per_token"
                   ) -> nvfp4.NVFP4Weight:
    """Kernel layout of an NVFP4 linear layer.  `weight_packed` uint8 `[N, K/2]`, `weight_scale` E4M3 `[N, K/16]`
    (fused shards concatenated along N), `weight_global_scale` one FP32 value per shard: compressed-tensors stores
    the `inverse` of the global scale, ModelOpt the `multiplier`.  Shards with different global scales need
    `shard_sizes` and are brought to a shared one.  `input_quant="group_128"` prepares the `[K/128, N, 8]` scales."""
    global prepared_layers
    if scale_convention not in ("inverse", "multiplier"):
        raise ValueError(f"unknown scale convention {scale_convention!r}")
    stored = weight_global_scale.float().reshape(-1)
    multipliers = 1.0 / stored if scale_convention == "inverse" else stored
    if shard_sizes is not None:
        weight_scale, shared = share_global_scale(weight_scale, multipliers, shard_sizes)
    elif torch.equal(multipliers, multipliers[:1].expand_as(multipliers)):
        shared = multipliers[0]
    else:
        raise ValueError("fused shards with different global scales need their shard_sizes")
    prepare = experimental.prepare if input_quant == "group_128" else nvfp4.prepare
    weight = prepare(weight_packed, weight_scale, shared.reshape(1), bridge=bridge)
    prepared_shapes.add(DenseShape(weight.weight.get_device(), *weight.shape, bridge, input_quant))
    prepared_layers += 1
    return weight


def linear(x: torch.Tensor, weight: nvfp4.NVFP4Weight, output: torch.Tensor, *,
           input_quant: fp8.InputQuant = "per_token") -> None:
    """`output[M, N] = x[M, K] @ dequant(weight).T` for BF16 `x`: quantise to FP8 (`per_token` or `group_128`), then
    the GEMM launched with programmatic dependent launch behind the quantiser."""
    if input_quant == "group_128":
        q, s = fp8.quantize_group_128(x)
        experimental.fp8_nvfp4_group_quant_gemm(q, s, weight, out=output, enable_pdl=PDL_STATIC_WEIGHTS)
    else:
        q, s = fp8.quantize(x)
        fp8_nvfp4_gemm(q, s, weight, out=output, enable_pdl=PDL_STATIC_WEIGHTS)


@dataclasses.dataclass(frozen=True)
class NVFP4MoE:
    """Both prepared projections of a MoE layer with their routing layout and input quantisation."""

    w13: nvfp4.NVFP4Experts  # [E, 2I, H] gated, [E, I, H] otherwise
    w2: nvfp4.NVFP4Experts  # [E, H, I]
    top_k: int
    num_global_experts: int
    dispatch_ranks: int
    layout: Literal["indexed", "contiguous", "masked"]
    configs: tuple[GemmConfig, GemmConfig] | None
    gate_up_quant: fp8.InputQuant = "per_token"
    down_quant: fp8.InputQuant = "per_token"
    is_gated: bool = True


def _group_scale_layout(experts: nvfp4.NVFP4Experts) -> nvfp4.NVFP4Experts:
    """`[E, K/16, N]` scales -> `[E, K/128, N, 8]` for group-128 input."""
    e, n, k = experts.shape
    regrouped = experts.scale.view(torch.uint8).view(e, k // 128, 8, n).permute(0, 1, 3, 2).contiguous()
    return dataclasses.replace(experts, scale=regrouped.view(torch.float8_e4m3fn))


def prepare_moe(w13_packed: torch.Tensor, w13_scale: torch.Tensor, w13_global_scale: torch.Tensor,
                w2_packed: torch.Tensor, w2_scale: torch.Tensor, w2_global_scale: torch.Tensor, top_k: int,
                num_global_experts: int | None = None, dispatch_ranks: int = 1, bridge: Bridge = "exact", *,
                configs: tuple[GemmConfig, GemmConfig] | None = None,
                layout: Literal["indexed", "contiguous", "masked"] = "indexed",
                scale_convention: Literal["inverse", "multiplier"] = "inverse",
                gate_up_quant: fp8.InputQuant = "per_token", down_quant: fp8.InputQuant = "per_token",
                is_gated: bool = True, layer_name: str = "MoE") -> NVFP4MoE:
    """Prepare the experts of one MoE layer after sharding.  w13 global scales are `[E, 2]` (gated) or `[E]`/`[E, 1]`,
    w2's `[E]`; a gated expert's gate and up halves are brought to a shared global scale.  `num_global_experts`
    defaults to the local count (no expert parallelism)."""
    num_experts, w13_channels, half_hidden = w13_packed.shape
    halves = 2 if is_gated else 1
    half_inter = w13_channels // (2 * halves)
    if w13_channels % (2 * halves) != 0 or tuple(w2_packed.shape) != (num_experts, half_hidden * 2, half_inter):
        raise ValueError(f"{layer_name}: gate/up and down projection shapes do not match")
    if configs is not None and any(int(c.use_stream_k) > 1 for c in configs):
        raise ValueError("grouped GEMM does not split K")
    if layout not in ("indexed", "contiguous", "masked"):
        raise ValueError(f"unknown layout {layout!r}")
    invert = scale_convention == "inverse"
    g13 = 1.0 / w13_global_scale.float() if invert else w13_global_scale.float()
    g2 = 1.0 / w2_global_scale.float() if invert else w2_global_scale.float()
    if is_gated:
        w13_scale, g13 = share_global_scale(w13_scale, g13.reshape(num_experts, 2), [w13_channels // 2] * 2)
    else:
        g13 = g13.reshape(num_experts)
    w13 = nvfp4.prepare_experts(w13_packed, w13_scale, g13, bridge=bridge)
    w2 = nvfp4.prepare_experts(w2_packed, w2_scale, g2.reshape(num_experts), bridge=bridge)
    if gate_up_quant == "group_128":
        w13 = _group_scale_layout(w13)
    if down_quant == "group_128":
        w2 = _group_scale_layout(w2)
    moe = NVFP4MoE(w13, w2, top_k, num_experts if num_global_experts is None else num_global_experts, dispatch_ranks,
                   layout, configs, gate_up_quant, down_quant, is_gated)
    if configs is None:
        prepared_grouped.update(moe_grouped_shapes(moe))
    return moe


class MoEBuffers(TypedDict):
    """Caller-owned contiguous buffers, with the shapes and dtypes of `moe_buffer_specs`."""

    input: torch.Tensor
    input_scale: torch.Tensor
    gate_up: torch.Tensor
    intermediate: torch.Tensor
    intermediate_scale: torch.Tensor
    output: torch.Tensor


# Custom activation `(output_bf16 [..., I], gate_up_bf16 [..., w13 channels]) -> None` for non-gated or unusual layers.
ActivationFn = Callable[[torch.Tensor, torch.Tensor], None]


def moe_grouped_shapes(moe: NVFP4MoE) -> tuple[GroupedShape, GroupedShape]:
    """The gate/up and down projections as `GroupedShape`s.  Both see the same routed rows; only an indexed gate/up
    projection gathers them from token rows (`input_top_k = top_k`)."""
    device = moe.w13.weight.get_device()
    shared = dict(device=device, num_experts=moe.w13.shape[0], top_k=moe.top_k, layout=moe.layout,
                  dispatch_ranks=moe.dispatch_ranks, num_global_experts=moe.num_global_experts)
    gather = moe.top_k if moe.layout == "indexed" else 1
    return (GroupedShape(n=moe.w13.shape[1], k=moe.w13.shape[2], input_top_k=gather, bridge=moe.w13.bridge,
                         input_quant=moe.gate_up_quant, **shared),
            GroupedShape(n=moe.w2.shape[1], k=moe.w2.shape[2], input_top_k=1, bridge=moe.w2.bridge,
                         input_quant=moe.down_quant, **shared))


def record_grouped_capture(moe: NVFP4MoE, rows: int) -> None:
    """While a CUDA graph is being captured with autotune on, count (and warn once per shape about) projections whose
    `rows` were never measured: they keep the rule's config for the life of the graph.  Pinned configs opt out."""
    global captured_untuned
    if moe.configs is not None or not autotune_enabled() or not torch.cuda.is_current_stream_capturing():
        return
    num_sms = runtime.get_num_sms(moe.w13.weight.get_device())
    for shape in moe_grouped_shapes(moe):
        key = (shape, num_sms, rows)
        if key in tuned_grouped:
            continue
        captured_untuned += 1
        if key not in warned_untuned:
            warned_untuned.add(key)
            warnings.warn(f"tensorbridge: grouped GEMM with {rows} routed rows of (N, K, E) = ({shape.n}, {shape.k}, "
                          f"{shape.num_experts}) captured without autotune; it keeps the selection rule's config", stacklevel=3)


def moe_rows(moe: NVFP4MoE, num_routes: int) -> int:
    """Expected routed rows on this rank from the global pre-dispatch `num_routes` (a scheduling hint only)."""
    return (num_routes * moe.w13.shape[0] + moe.num_global_experts - 1) // moe.num_global_experts


def moe_post_dispatch_rows(moe: NVFP4MoE, received_tokens: int) -> int:
    """Expected routed rows on this rank when the dispatch sends each token at most once per rank: a received token
    has at least one local route, and under uniform routing `top_k * p / (1 - (1 - p)^top_k)` of them in expectation,
    `p` the local share of the experts.  Bounded by one and `top_k` routes per received token."""
    if received_tokens <= 0:
        return 0
    local = moe.w13.shape[0]
    if moe.top_k <= 1 or local >= moe.num_global_experts:
        return received_tokens * moe.top_k
    share = local / moe.num_global_experts
    per_token = moe.top_k * share / (1.0 - (1.0 - share) ** moe.top_k)
    return max(received_tokens, min(received_tokens * moe.top_k, round(received_tokens * per_token)))


def moe_block_sizes(moe: NVFP4MoE, rows: int) -> tuple[int, int]:
    """Token tiles of the gate/up and down projections for `rows` routed rows: what indexed routes must be aligned to.
    Ask after autotune and before aligning."""
    if moe.configs is not None:
        return moe.configs[0].block_m, moe.configs[1].block_m
    tiles = [runtime.select_config(rows, shape.n, shape.k, shape.num_experts, shape.layout, shape.device, bridge=shape.bridge,
                                   top_k=shape.input_top_k, group_scales=shape.input_quant == "group_128").block_m
             for shape in moe_grouped_shapes(moe)]
    return tiles[0], tiles[1]


def precompile_prepared(max_tokens: int) -> int:
    """Make sure every kernel `select_config` can pick for 1 .. `max_tokens` tokens on the prepared dense and grouped
    shapes of the current device is loaded, so that no launch meets a compile.  Template points the library was built
    with cost nothing; the others are compiled with NVRTC (or fetched from the disk cache) and registered.  Returns the
    number of kernels compiled or loaded by this call (`tensorbridge/serving.py:173-257`)."""
    if max_tokens < 1:
        return 0
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("precompile builds kernels: call it before CUDA graph capture, not during it")
    device = torch.cuda.current_device()
    num_sms = runtime.get_num_sms(device)
    # every M up to 256, then every eighth, then the maximum: the sizes decode steps and prefill chunks produce
    ms = list(range(1, min(max_tokens, 256) + 1)) + list(range(264, max_tokens + 1, 8))
    if ms[-1] != max_tokens:
        ms.append(max_tokens)
    before = len(runtime.loaded_kernels)
    for entry in sorted({normalize_dense_shape(e) for e in prepared_shapes}):
        if entry.device != device or (entry, num_sms, max_tokens) in precompiled_dense:
            continue
        group = entry.input_quant == "group_128"
        for config in dict.fromkeys(runtime.select_config(m, entry.n, entry.k, device=device, bridge=entry.bridge, group_scales=group)
                                    for m in ms):
            runtime.get_kernel(entry.n, entry.k, config, device, bridge=entry.bridge, group_scales=group)
        precompiled_dense.add((entry, num_sms, max_tokens))
    for shape in sorted(prepared_grouped):
        if shape.device != device or (shape, num_sms, max_tokens) in precompiled_grouped:
            continue
        group = shape.input_quant == "group_128"
        rows = sorted({(shape.dispatch_ranks * m * shape.top_k * shape.num_experts + shape.num_global_experts - 1) // shape.num_global_experts
                       for m in ms})
        for config in dict.fromkeys(runtime.select_config(r, shape.n, shape.k, shape.num_experts, shape.layout, device,
                                                          bridge=shape.bridge, top_k=shape.input_top_k, group_scales=group) for r in rows):
            runtime.get_grouped_kernel(shape.n, shape.k, shape.num_experts, shape.layout, config, device, bridge=shape.bridge,
                                       group_scales=group)
        precompiled_grouped.add((shape, num_sms, max_tokens))
    return len(runtime.loaded_kernels) - before


def autotune_prepared(ms: Sequence[int]) -> None:
    """With `TENSORBRIDGE_AUTOTUNE=1`: measure every dense shape prepared on the current device at the token counts
    `ms` (the sizes a CUDA graph will capture) on seeded random weights and activations of that shape, and serve the
    winners from then on.  Call it before capture; sizes already measured are skipped
    (`tensorbridge/serving.py:269-353`; grouped projections are measured by `autotune_grouped` with real routing)."""
    if not autotune_enabled() or not ms:
        return
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("autotune times kernels: call it before CUDA graph capture, not during it")
    device = torch.cuda.current_device()
    num_sms = runtime.get_num_sms(device)
    dev = torch.device("cuda", device)
    gen = torch.Generator(device=dev).manual_seed(0)
    for entry in sorted({normalize_dense_shape(e) for e in prepared_shapes}):
        if entry.device != device:
            continue
        todo = [m for m in ms if m > 0 and dense_tuned_key(device, num_sms, entry.n, entry.k, m, entry.bridge, entry.input_quant) not in tuned]
        if not todo:
            continue
        group = entry.input_quant == "group_128"
        checkpoint = nvfp4.quantize((torch.randn((entry.n, entry.k), generator=gen, device=dev) * 0.02).bfloat16())
        weight = (experimental.prepare if group else nvfp4.prepare)(*checkpoint, bridge=entry.bridge)
        for m in todo:
            x = torch.randn((m, entry.k), generator=gen, device=dev).bfloat16()
            a, a_scale = (fp8.quantize_group_128 if group else fp8.quantize)(x)
            _autotune.autotune(a, a_scale.contiguous() if group else a_scale, weight, group_scales=group)
            tuned.add(dense_tuned_key(device, num_sms, entry.n, entry.k, m, entry.bridge, entry.input_quant))


def moe_buffer_specs(moe: NVFP4MoE, num_tokens: int, *, unfused_activation: bool = False
                     ) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
    """Shapes and dtypes of the buffers `moe_forward_*` needs for `num_tokens` tokens seen by this rank, sized for the
    worst routing.  Rows follow from the layout: a masked layer gives every local expert a block of `num_tokens` rows,
    the other two hold one row per route (`num_tokens * top_k`); only an indexed layer keeps its input per token, since
    its gate/up projection gathers rows by route.  Scale columns are one per row, or one per 128 input columns of the
    projection that reads them."""
    experts, gate_up_channels, hidden = moe.w13.shape
    intermediate = moe.w2.shape[2]
    routed = num_tokens * (experts if moe.layout == "masked" else moe.top_k)
    tokens_in = num_tokens if moe.layout == "indexed" else routed

    def scale_columns(width: int, quant: str) -> int:
        return width // 128 if quant == "group_128" else 1

    specs = {
        "input": ((tokens_in, hidden), torch.float8_e4m3fn),
        "input_scale": ((tokens_in, scale_columns(hidden, moe.gate_up_quant)), torch.float32),
        "gate_up": ((routed, gate_up_channels), torch.bfloat16),
        "intermediate": ((routed, intermediate), torch.float8_e4m3fn),
        "intermediate_scale": ((routed, scale_columns(intermediate, moe.down_quant)), torch.float32),
        "output": ((routed, moe.w2.shape[1]), torch.bfloat16),
    }
    if unfused_activation:
        specs["activated"] = ((routed, intermediate), torch.bfloat16)
    return specs


def _configs(moe: NVFP4MoE) -> tuple[GemmConfig | None, GemmConfig | None]:
    return (None, None) if moe.configs is None else moe.configs


def _activate_and_quantize(moe: NVFP4MoE, buffers: MoEBuffers, activation_fn: ActivationFn | None,
                           activated_buffer: torch.Tensor | None, *, expert_counts: torch.Tensor | None = None,
                           num_valid_rows: torch.Tensor | None = None) -> None:
    """gate/up output -> FP8 intermediate + scales: the fused SiLU-mul quantiser, or `activation_fn` then a quantiser."""
    out = (buffers["intermediate"], buffers["intermediate_scale"])
    intermediate = moe.w2.shape[2]
    if activation_fn is not None:
        activated = activated_buffer
        if activated is None:
            activated = torch.empty((buffers["gate_up"].size(0), intermediate), dtype=torch.bfloat16,
                                    device=buffers["gate_up"].device)
        if expert_counts is not None:
            experts = moe.w13.shape[0]
            activation_fn(activated.view(experts, -1, intermediate), buffers["gate_up"].view(experts, -1, buffers["gate_up"].size(1)))
        else:
            activation_fn(activated, buffers["gate_up"])
        if moe.down_quant == "group_128" or expert_counts is not None or num_valid_rows is not None:
            fp8.quantize_moe(activated, moe.down_quant, expert_counts=expert_counts, num_valid_rows=num_valid_rows, out=out)
        else:
            fp8.quantize(activated, out=out)
    elif moe.down_quant == "group_128" or expert_counts is not None:
        fp8.quantize_moe(buffers["gate_up"], moe.down_quant, activation=True, expert_counts=expert_counts,
                         num_valid_rows=num_valid_rows, out=out)
    else:
        fp8.silu_mul_quantize(buffers["gate_up"], num_valid_rows=num_valid_rows, out=out)


def moe_forward_indexed(moe: NVFP4MoE, hidden_states: torch.Tensor, routing13: IndexedRouting, routing2: IndexedRouting,
                        buffers: MoEBuffers, input_scale: torch.Tensor | None = None, *,
                        local_rows_hint: int | None = None, activation_fn: ActivationFn | None = None,
                        activated_buffer: torch.Tensor | None = None) -> torch.Tensor:
    """quantise -> gate/up grouped GEMM (routes gather their token rows) -> activation + quantise -> down grouped GEMM
    (`top_k = 1`, one input row per route).  Returns `[T * top_k, H]` in route order; the caller weights and sums the
    top-k outputs.  Each projection may be aligned to its own block_m."""
    if moe.layout != "indexed" or routing13.top_k != moe.top_k or routing2.top_k != 1:
        raise ValueError("indexed MoE needs gate/up top_k routes and down top_k=1 routes")
    if not moe.is_gated and activation_fn is None:
        raise ValueError("non-gated MoE requires an explicit activation_fn")
    rows = moe_rows(moe, hidden_states.size(0) * moe.top_k) if local_rows_hint is None else local_rows_hint
    cfg13, cfg2 = _configs(moe)
    if input_scale is not None:
        inputs, scales = hidden_states, input_scale
    elif moe.gate_up_quant == "group_128":
        inputs, scales = fp8.quantize_moe(hidden_states, "group_128", out=(buffers["input"], buffers["input_scale"]))
    else:
        inputs, scales = fp8.quantize(hidden_states, out=(buffers["input"], buffers["input_scale"]))
    fp8_nvfp4_grouped_gemm(inputs, scales, moe.w13, routing13, rows, out=buffers["gate_up"], config=cfg13,
                           enable_pdl=input_scale is None, group_scales=moe.gate_up_quant == "group_128")
    _activate_and_quantize(moe, buffers, activation_fn, activated_buffer)
    return fp8_nvfp4_grouped_gemm(buffers["intermediate"], buffers["intermediate_scale"], moe.w2, routing2, rows,
                                  out=buffers["output"], config=cfg2, enable_pdl=True,
                                  group_scales=moe.down_quant == "group_128")


def moe_forward_contiguous(moe: NVFP4MoE, hidden_states: torch.Tensor, scatter_idx: torch.Tensor,
                           routing: ContiguousRouting, buffers: MoEBuffers, input_scale: torch.Tensor | None = None,
                           num_routes: int | None = None, *, local_rows_hint: int | None = None,
                           activation_fn: ActivationFn | None = None, activated_buffer: torch.Tensor | None = None
                           ) -> torch.Tensor:
    """scatter-quantise (or scatter already quantised FP8) into expert order -> gate/up GEMM -> activation + quantise
    -> down GEMM.  Only rows below the device-side `expert_offsets[-1]` are valid in the expert-ordered output; no
    row count is read on the host."""
    if moe.layout != "contiguous":
        raise ValueError("contiguous MoE needs a layer prepared for contiguous dispatch")
    if not moe.is_gated and activation_fn is None:
        raise ValueError("non-gated MoE requires an explicit activation_fn")
    capacity = buffers["input"].size(0)
    rows = local_rows_hint if local_rows_hint is not None else moe_rows(
        moe, hidden_states.size(0) * moe.top_k if num_routes is None else num_routes)
    cfg13, cfg2 = _configs(moe)
    pdl_first = True
    if input_scale is not None:
        if hidden_states.data_ptr() == buffers["input"].data_ptr():
            inputs, scales, pdl_first = hidden_states, input_scale, False
        else:
            inputs, scales = fp8.scatter_fp8(hidden_states, input_scale, scatter_idx,
                                             out=(buffers["input"], buffers["input_scale"]))
    elif moe.gate_up_quant == "group_128":
        inputs, scales = fp8.quantize_moe(hidden_states, "group_128", scatter_idx=scatter_idx,
                                          out=(buffers["input"], buffers["input_scale"]))
    else:
        inputs, scales = fp8.scatter_quantize(hidden_states, scatter_idx, capacity,
                                              out=(buffers["input"], buffers["input_scale"]))
    fp8_nvfp4_grouped_gemm(inputs, scales, moe.w13, routing, rows, out=buffers["gate_up"], config=cfg13,
                           enable_pdl=pdl_first, group_scales=moe.gate_up_quant == "group_128")
    valid = routing.expert_offsets[-1:]
    _activate_and_quantize(moe, buffers, activation_fn, activated_buffer, num_valid_rows=valid)
    return fp8_nvfp4_grouped_gemm(buffers["intermediate"], buffers["intermediate_scale"], moe.w2, routing, rows,
                                  out=buffers["output"], config=cfg2, enable_pdl=True,
                                  group_scales=moe.down_quant == "group_128")


def moe_forward_masked(moe: NVFP4MoE, hidden_states: torch.Tensor, routing: MaskedRouting, buffers: MoEBuffers,
                       input_scale: torch.Tensor | None = None, num_routes: int | None = None, *,
                       activation_fn: ActivationFn | None = None, activated_buffer: torch.Tensor | None = None
                       ) -> torch.Tensor:
    """Consume the flattened `[E * capacity, H]` expert buffers of a masked dispatch; returns `[E * capacity, H]`."""
    if moe.layout != "masked":
        raise ValueError("masked MoE needs a layer prepared for masked dispatch")
    if not moe.is_gated and activation_fn is None:
        raise ValueError("non-gated MoE requires an explicit activation_fn")
    rows = hidden_states.size(0) if num_routes is None else moe_rows(moe, num_routes)
    cfg13, cfg2 = _configs(moe)
    if input_scale is None:
        inputs, scales = fp8.quantize_moe(hidden_states, moe.gate_up_quant, expert_counts=routing.expert_counts,
                                          out=(buffers["input"], buffers["input_scale"]))
    else:
        inputs, scales = hidden_states, input_scale
    fp8_nvfp4_grouped_gemm(inputs, scales, moe.w13, routing, rows, out=buffers["gate_up"], config=cfg13,
                           enable_pdl=input_scale is None, group_scales=moe.gate_up_quant == "group_128")
    _activate_and_quantize(moe, buffers, activation_fn, activated_buffer, expert_counts=routing.expert_counts)
    return fp8_nvfp4_grouped_gemm(buffers["intermediate"], buffers["intermediate_scale"], moe.w2, routing, rows,
                                  out=buffers["output"], config=cfg2, enable_pdl=True,
                                  group_scales=moe.down_quant == "group_128")
