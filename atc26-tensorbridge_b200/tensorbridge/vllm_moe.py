"""MoE experts in the shape of the reference's vLLM adapter, runnable without vLLM.

The reference's `tensorbridge/vllm_moe.py` plugs three things into vLLM 0.32's modular MoE kernel: a support check
(`unsupported_moe_reason`, `:58-89`), a quantisation method that prepares a layer's checkpoint tensors after loading
(`TensorBridgeMoEMethod.process_weights_after_loading`, `:168-214`) and an experts object whose `apply` turns routed
hidden states into the layer's output (`make_experts`, `:238-409`).  vLLM owns routing and communication there, and
three of its helper kernels sit on that path: `moe_align_block_size`, `moe_fused_mul_sum` and the
`moe_prepare_scatter` / `moe_unpermute` pair.

This module keeps those three pieces and their argument meaning, with duck-typed layers instead of vLLM classes, and
brings its own helpers: `tensorbridge.routing.align_routes` builds the indexed tables, the library's dispatch plan
kernel (`tb_ep_plan`) sorts routes by expert for the contiguous layout, and `tb_moe_combine` weights and sums the
top-k outputs of either.  A vLLM quantisation method wraps `TensorBridgeMoEMethod` by forwarding its
`process_weights_after_loading` and `apply`.
"""
from __future__ import annotations

import math
import warnings
from typing import Literal

import torch

from tensorbridge import serving
from tensorbridge.gemm import ContiguousRouting, IndexedRouting, MaskedRouting
from tensorbridge.routing import align_routes

warned_moe_fallbacks: set[str] = set()

SUPPORTED_ACTIVATIONS = ("silu", "gelu", "relu2_no_mul", "silu_no_mul", "gelu_no_mul")


def uses_fused_silu(activation: str, swiglu_limit: float | None = None, swiglu_alpha: float | None = None,
                    swiglu_beta: float | None = None) -> bool:
    """Whether a layer runs the fused `silu(gate) * up -> FP8` kernel rather than a separate activation
    (`tensorbridge/vllm_moe.py:48-55`): plain SiLU gating without clamp or slope parameters."""
    return str(activation).lower() == "silu" and swiglu_limit is None and swiglu_alpha is None and swiglu_beta is None


def unsupported_moe_reason(layer, group_size: int | None = None) -> str | None:
    """Why `layer` cannot run on the grouped kernels, or None if it can (`tensorbridge/vllm_moe.py:58-89`).

    `layer.moe_config` carries `in_dtype`, `hidden_dim`, `intermediate_size_per_partition` and, optionally, `has_bias`,
    `is_lora_enabled`, `activation`; `layer.apply_router_weight_on_input` is optional.  `group_size` is the weight
    group size of a ModelOpt checkpoint (16 is the only one the kernels take)."""
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
        return "TensorBridge MoE on this build requires Blackwell (sm_100)"
    moe = layer.moe_config
    if getattr(moe, "in_dtype", torch.bfloat16) != torch.bfloat16:
        return f"in_dtype={moe.in_dtype} (requires torch.bfloat16)"
    if getattr(moe, "has_bias", False) or getattr(moe, "is_lora_enabled", False):
        return "bias and LoRA are not supported"
    if getattr(layer, "apply_router_weight_on_input", False):
        return "apply_router_weight_on_input is not supported"
    if group_size is not None and group_size != 16:
        return f"group_size={group_size} (requires 16)"
    activation = str(getattr(moe, "activation", "silu")).lower()
    if activation not in SUPPORTED_ACTIVATIONS:
        return f"activation {activation!r} is not supported"
    hidden, intermediate = moe.hidden_dim, moe.intermediate_size_per_partition
    if hidden <= 0 or intermediate <= 0 or hidden % 128 != 0 or intermediate % 128 != 0:
        return f"local MoE shape (H={hidden}, I_local={intermediate}) must be positive multiples of 128"
    return None


def warn_moe_fallback(prefix: str, reason: str) -> None:
    """One warning per distinct reason (`tensorbridge/vllm_moe.py:92-98`)."""
    if reason not in warned_moe_fallbacks:
        warned_moe_fallbacks.add(reason)
        warnings.warn(f"TensorBridge MoE skipped {prefix} ({reason}); falling back to the native MoE method", stacklevel=3)


def combine_routes(routed: torch.Tensor, topk_weights: torch.Tensor, index: torch.Tensor | None = None,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """`out[t] = sum_j topk_weights[t, j] * routed[index[t, j]]` (`index` None: row `t * top_k + j`), FP32 sums in slot
    order; a negative index adds nothing.  One kernel for vLLM's `moe_fused_mul_sum` and `moe_unpermute`."""
    from tensorbridge import _native  # noqa: PLC0415
    tokens, top_k = topk_weights.shape
    width = routed.size(-1)
    if routed.dtype != torch.bfloat16 or not routed.is_contiguous() or width % 8:
        raise ValueError("routed rows must be contiguous BF16 with a multiple of 8 channels")
    if out is None:
        out = torch.empty((tokens, width), dtype=torch.bfloat16, device=routed.device)
    weights = topk_weights.to(torch.float32).contiguous()
    rows = index.to(torch.int32).contiguous() if index is not None else None
    with torch.cuda.device(routed.device):
        _native.check(_native.load().tb_moe_combine(_native.stream_ptr(routed.device.index), routed.data_ptr(),
                                                    None if rows is None else rows.data_ptr(), weights.data_ptr(), tokens,
                                                    top_k, width, out.data_ptr()))
    return out


def prepare_scatter(topk_ids: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Routes sorted by (local) expert: int64 `offsets[E + 1]` and, per route, its row in expert order as int32
    `[T, top_k]` (-1 for a route whose id is outside `[0, num_experts)`).  Routes of one expert keep their order.
    No value is read back to the host."""
    from tensorbridge import parallel  # noqa: PLC0415
    counts, positions = parallel.plan_local(topk_ids, num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=topk_ids.device)
    offsets[1:] = torch.cumsum(counts.to(torch.int64), 0)
    return offsets, positions.view(topk_ids.shape)


class TensorBridgeExperts:
    """The experts of one prepared layer (`tensorbridge/vllm_moe.py:238-409`): `apply` writes the layer's output for the
    hidden states this rank holds.

    `indexed`: `hidden_states [T, H]`, `topk_ids [T, top_k]` (global expert ids, mapped through `expert_map` when the
    rank holds a subset), output `[T, H]` = weighted sum of each token's routed outputs.  `contiguous`: the same call;
    rows are first scattered into expert order.  `masked`: `hidden_states [E_local, capacity, H]` as a masked dispatch
    delivers them, `expert_num_tokens [E_local]`, output `[E_local, capacity, H]` per received row (the dispatcher
    weights and sums after its combine)."""

    def __init__(self, prepared: serving.NVFP4MoE, activation: str = "silu", activation_fn: serving.ActivationFn | None = None):
        self.prepared = prepared
        self.activation = activation
        if activation_fn is None and not uses_fused_silu(activation):
            raise ValueError(f"activation {activation!r} needs an activation_fn(output, gate_up)")
        self.activation_fn = None if uses_fused_silu(activation) else activation_fn
        self._buffers: dict[tuple[int, int], serving.MoEBuffers] = {}

    def workspace_shapes(self, num_tokens: int) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        """Buffers `apply` needs for `num_tokens` tokens (experts x capacity rows for a masked layer)."""
        return serving.moe_buffer_specs(self.prepared, num_tokens, unfused_activation=self.activation_fn is not None)

    def _buffers_for(self, num_tokens: int, device: torch.device) -> serving.MoEBuffers:
        key = (num_tokens, device.index)
        if key not in self._buffers:
            specs = self.workspace_shapes(num_tokens)
            self._buffers[key] = {name: torch.empty(shape, dtype=dtype, device=device) for name, (shape, dtype) in specs.items()}
        return self._buffers[key]

    def apply(self, output: torch.Tensor, hidden_states: torch.Tensor, topk_weights: torch.Tensor | None,
              topk_ids: torch.Tensor | None, *, expert_map: torch.Tensor | None = None,
              a1q_scale: torch.Tensor | None = None, expert_num_tokens: torch.Tensor | None = None,
              buffers: serving.MoEBuffers | None = None) -> torch.Tensor:
        moe = self.prepared
        if moe.layout == "masked":
            if expert_num_tokens is None:
                raise ValueError("a masked layer needs expert_num_tokens")
            experts, capacity, hidden = hidden_states.shape
            buffers = buffers or self._buffers_for(capacity, hidden_states.device)
            buffers = dict(buffers, output=output.view(-1, output.size(-1)))
            routes = experts * capacity if topk_ids is None else topk_ids.numel() * moe.dispatch_ranks
            serving.moe_forward_masked(moe, hidden_states.view(-1, hidden), MaskedRouting(expert_num_tokens), buffers, a1q_scale,
                                       routes, activation_fn=self.activation_fn, activated_buffer=buffers.get("activated"))
            return output
        if topk_ids is None or topk_weights is None:
            raise ValueError("indexed and contiguous layers need topk_ids and topk_weights")
        hidden = hidden_states.view(-1, hidden_states.size(-1))
        tokens = hidden.size(0)
        buffers = buffers or self._buffers_for(tokens, hidden.device)
        local_ids = topk_ids if expert_map is None else expert_map[topk_ids.to(torch.int64)]
        experts = moe.w13.shape[0]
        if moe.layout == "indexed":
            rows_hint = serving.moe_rows(moe, tokens * moe.top_k)
            bm13, bm2 = serving.moe_block_sizes(moe, rows_hint)
            first = align_routes(local_ids, experts, bm13)
            second = first if bm2 == bm13 else align_routes(local_ids, experts, bm2)
            routing2 = IndexedRouting(second.sorted_ids, second.expert_ids, second.num_tokens_padded, bm2, 1)
            routed = serving.moe_forward_indexed(moe, hidden, first, routing2, buffers, a1q_scale, local_rows_hint=rows_hint,
                                                 activation_fn=self.activation_fn, activated_buffer=buffers.get("activated"))
            # routes of experts this rank does not hold were never written: they must not enter the sum
            index = None
            if expert_map is not None:
                flat = local_ids.reshape(-1)
                index = torch.where((flat >= 0) & (flat < experts), torch.arange(flat.numel(), device=flat.device), -1)
            return combine_routes(routed, topk_weights, index, out=output)
        offsets, scatter = prepare_scatter(local_ids, experts)
        rows_hint = serving.moe_post_dispatch_rows(moe, tokens)
        scales = None if a1q_scale is None else a1q_scale.view(tokens, -1)
        routed = serving.moe_forward_contiguous(moe, hidden, scatter, ContiguousRouting(offsets), buffers, scales,
                                                local_rows_hint=rows_hint, activation_fn=self.activation_fn,
                                                activated_buffer=buffers.get("activated"))
        return combine_routes(routed, topk_weights, scatter.reshape(-1), out=output)


def make_experts(prepared: serving.NVFP4MoE, activation: str = "silu",
                 activation_fn: serving.ActivationFn | None = None) -> TensorBridgeExperts:
    """The experts object for a prepared layer (`tensorbridge/vllm_moe.py:238-242`)."""
    return TensorBridgeExperts(prepared, activation, activation_fn)


class TensorBridgeMoEMethod:
    """Quantisation method of one MoE layer (`tensorbridge/vllm_moe.py:101-227`): prepares the checkpoint tensors the
    loader left on the layer, then serves `apply`.

    `checkpoint` names the format: "compressed-tensors" layers carry `w13_weight_packed`, `w13_weight_scale`,
    `w13_weight_global_scale` (and the w2 three) with inverse global scales; "modelopt" layers carry `w13_weight`,
    `w13_weight_scale`, `w13_weight_scale_2` with multiplier scales."""

    def __init__(self, top_k: int, num_global_experts: int, ep_size: int = 1, bridge: str = "exact",
                 layout: Literal["indexed", "contiguous", "masked"] = "indexed", checkpoint: str = "compressed-tensors",
                 gate_up_quant: str = "per_token", down_quant: str = "per_token", is_gated: bool = True,
                 activation: str = "silu", activation_fn: serving.ActivationFn | None = None, layer_name: str = "MoE"):
        if checkpoint not in ("compressed-tensors", "modelopt"):
            raise ValueError(f"unknown checkpoint format {checkpoint!r}")
        self.top_k, self.num_global_experts, self.ep_size = top_k, num_global_experts, ep_size
        self.bridge, self.layout, self.checkpoint = bridge, layout, checkpoint
        self.gate_up_quant, self.down_quant, self.is_gated = gate_up_quant, down_quant, is_gated
        self.activation, self.activation_fn, self.layer_name = activation, activation_fn, layer_name
        self.experts: TensorBridgeExperts | None = None

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        if getattr(layer, "apply_router_weight_on_input", False):
            raise ValueError(f"{self.layer_name}: TensorBridge MoE applies router weights to expert outputs")
        if self.checkpoint == "compressed-tensors":
            names = ("w13_weight_packed", "w13_weight_scale", "w13_weight_global_scale",
                     "w2_weight_packed", "w2_weight_scale", "w2_weight_global_scale")
            convention = "inverse"
        else:
            names = ("w13_weight", "w13_weight_scale", "w13_weight_scale_2", "w2_weight", "w2_weight_scale", "w2_weight_scale_2")
            convention = "multiplier"
        tensors = [getattr(layer, name) for name in names]
        prepared = serving.prepare_moe(*[t.data if isinstance(t, torch.nn.Parameter) else t for t in tensors], self.top_k,
                                       self.num_global_experts, self.ep_size, self.bridge, layout=self.layout,
                                       scale_convention=convention, gate_up_quant=self.gate_up_quant,
                                       down_quant=self.down_quant, is_gated=self.is_gated, layer_name=self.layer_name)
        for name in names:
            delattr(layer, name)
        for stale in ("w13_input_global_scale", "w2_input_global_scale", "w13_input_scale", "w2_input_scale"):
            if hasattr(layer, stale):
                delattr(layer, stale)
        layer.w13_weight = torch.nn.Parameter(prepared.w13.weight, requires_grad=False)
        layer.w2_weight = torch.nn.Parameter(prepared.w2.weight, requires_grad=False)
        layer.w13_weight_scale = torch.nn.Parameter(prepared.w13.scale, requires_grad=False)
        layer.w2_weight_scale = torch.nn.Parameter(prepared.w2.scale, requires_grad=False)
        layer.register_buffer("tensorbridge_w13_global_scale", prepared.w13.global_scale)
        layer.register_buffer("tensorbridge_w2_global_scale", prepared.w2.global_scale)
        layer.register_buffer("tensorbridge_w13_locks", prepared.w13.locks)
        layer.register_buffer("tensorbridge_w2_locks", prepared.w2.locks)
        self.experts = make_experts(prepared, self.activation, self.activation_fn)

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, *,
              expert_map: torch.Tensor | None = None) -> torch.Tensor:
        if self.experts is None:
            raise RuntimeError(f"{self.layer_name}: process_weights_after_loading has not run")
        if self.layout == "masked":
            raise ValueError("a masked layer is driven by its dispatcher: call experts.apply with the received buffers")
        hidden = x.view(-1, x.size(-1))
        output = torch.empty((hidden.size(0), self.experts.prepared.w2.shape[1]), dtype=torch.bfloat16, device=x.device)
        self.experts.apply(output, hidden, topk_weights, topk_ids,
                           expert_map=expert_map if expert_map is not None else getattr(layer, "expert_map", None))
        return output.view(*x.shape[:-1], output.size(-1))


def workspace_bytes(experts: TensorBridgeExperts, num_tokens: int) -> int:
    """Bytes of all the buffers `experts.apply` uses for `num_tokens` tokens."""
    return sum(math.prod(shape) * dtype.itemsize for shape, dtype in experts.workspace_shapes(num_tokens).values())
