"""`D = A @ W.T` with FP8 activations and NVFP4 weights on B200: one dense entry point, one grouped by expert.

The public names, argument order and error behaviour are those of the reference's `tensorbridge/gemm.py:12-114`;
the work is done by `tb_gemm_dense` / `tb_gemm_grouped` in libtensorbridge_b200.so.
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch

from tensorbridge import _native
from tensorbridge.jit import runtime
from tensorbridge.jit.codegen import GemmConfig, pad_to_unit
from tensorbridge.quant.nvfp4 import NVFP4Experts, NVFP4Weight


@dataclasses.dataclass(frozen=True)
class IndexedRouting:
    """Route ids sorted by expert and padded per expert to `block_m`; route `r` reads input row `r // top_k` and
    writes output row `r`.  Padding slots hold ids >= `M * top_k`."""

    sorted_ids: torch.Tensor  # int32 [padded route capacity]
    expert_ids: torch.Tensor  # int32, one expert per `block_m` block
    num_tokens_padded: torch.Tensor  # int32 [1], padded routes actually in use (device side)
    block_m: int
    top_k: int


@dataclasses.dataclass(frozen=True)
class ContiguousRouting:
    """Rows of `a` grouped by expert without padding: expert `e` owns rows `expert_offsets[e]:expert_offsets[e+1]`."""

    expert_offsets: torch.Tensor  # int64 [E + 1], first 0, last the row count


@dataclasses.dataclass(frozen=True)
class MaskedRouting:
    """`E` equal blocks of `a.size(0) // E` rows; expert `e` owns the first `expert_counts[e]` rows of block `e`."""

    expert_counts: torch.Tensor  # int32 [E]


Routing = IndexedRouting | ContiguousRouting | MaskedRouting


@dataclasses.dataclass(frozen=True)
class PeerScatter:
    """Where a masked or contiguous grouped launch of an expert-parallel step sends its output rows: `row_target` int32
    `[rows]` names, for every row of `a`, the rank and route it belongs to (`rank << 26 | route`, -1 = nobody's), and
    `peer_out` holds every rank's BF16 route buffer as mapped into this process.  The epilogue stores each row straight
    into the owner's buffer, so no combine pass follows the GEMM (`tensorbridge.parallel.PeerMaskedExchange` builds one)."""

    row_target: torch.Tensor
    peer_out: object  # ctypes array of device pointers, one per rank
    world: int

# FP32 scratch per (device, stream, kind of launch): distinct streams never share partial sums, and launches with K
# splits never share a buffer with launches that give every CTA an even share of K blocks (`use_stream_k = 1`), whose
# partial sums a K-split launch could mistake for tags.
_workspaces: dict[tuple[int, int, bool], torch.Tensor] = {}
# Buffers that were replaced by larger ones.  A CUDA graph captured earlier on the stream still launches with the old
# pointer, so the old buffer must stay allocated for as long as the process may replay that graph: buffers only ever
# grow by appending, nothing is handed back to the allocator.
_retired: list[torch.Tensor] = []


def _workspace(device: torch.device, nbytes: int, stream: int, even_shares: bool = False) -> torch.Tensor | None:
    """A scratch buffer of at least `nbytes` for `stream`, or None when one would have to be allocated while the
    stream is being captured into a CUDA graph."""
    key = (device.index, stream, even_shares)
    have = _workspaces.get(key)
    if have is not None and have.numel() * 4 >= nbytes:
        return have
    if torch.cuda.is_current_stream_capturing():
        return None
    if have is not None:
        _retired.append(have)
    # zeros: the head of the buffer holds the launch sequence the tagged split-K partial sums are matched against
    _workspaces[key] = torch.zeros(max(nbytes, 8 << 20) // 4, dtype=torch.float32, device=device)
    return _workspaces[key]


def reset_workspaces(device: int | None = None) -> None:
    """Zero the split-K scratch of `device` (all devices when None).  Needed only after `check_status()` reported a
    kernel that gave up waiting, if the same CUDA graph is to be replayed: eager launches number themselves afresh."""
    for (index, _, _), buffer in _workspaces.items():
        if device is None or index == device:
            buffer.zero_()


_native.error_hooks.append(reset_workspaces)


# Indexed launches first gather their routed rows into scratch (then the GEMM loads tiles by TMA); set to False to let
# the GEMM fetch rows itself, as it does when scratch cannot be allocated (inside a CUDA-graph capture).
USE_GATHER_PASS = True

# Gathered activation rows of indexed launches, per (device, stream).
_gather_buffers: dict[tuple[int, int], torch.Tensor] = {}


def _gather_buffer(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """Scratch for the row gather of an indexed launch, or None when it would have to be allocated during a CUDA-graph
    capture (the kernel then gathers rows itself, which is slower)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    have = _gather_buffers.get(key)
    if have is not None and have.numel() >= nbytes:
        return have
    if torch.cuda.is_current_stream_capturing():
        return None
    if have is not None:
        _retired.append(have)
    _gather_buffers[key] = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    return _gather_buffers[key]


def _config_struct(config: GemmConfig) -> _native.Config:
    return _native.Config(*config.to_list())


def _require(cond: bool, message: str) -> None:
    if not cond:
        raise ValueError(message)


def _check_common(a: torch.Tensor, a_scale: torch.Tensor, k: int, group_scales: bool) -> tuple[int, int]:
    _require(a.is_cuda and a.dtype == torch.float8_e4m3fn and a.dim() == 2 and a.is_contiguous(),
             "a must be a contiguous FP8 E4M3 CUDA matrix")
    _require(a.size(1) == k, f"a has {a.size(1)} columns, the weight has K = {k}")
    _require(a_scale.is_cuda and a_scale.dtype == torch.float32 and a_scale.device == a.device,
             "a_scale must be FP32 on the device of a")
    rows = a.size(0)
    if group_scales:
        groups = pad_to_unit(k) // 128
        if a_scale.dim() == 3:  # masked [E, capacity, K/128]
            _require(a_scale.size(0) * a_scale.size(1) == rows and a_scale.size(2) == groups,
                     "masked scales must be [E, capacity, K/128]")
            _require(a_scale.stride(0) == a_scale.size(1) * a_scale.stride(1), "masked scales must have uniform row stride")
            return a_scale.stride(1), a_scale.stride(2)
        _require(a_scale.dim() == 2 and tuple(a_scale.shape) == (rows, groups), "a_scale must have shape [M, K / 128]")
        return a_scale.stride(0), a_scale.stride(1)
    _require(a_scale.numel() == rows and a_scale.is_contiguous(), "a_scale must be a contiguous [M, 1] tensor")
    return 1, 0


def _output(out: torch.Tensor | None, rows: int, n: int, like: torch.Tensor) -> torch.Tensor:
    if out is None:
        return torch.empty((rows, n), dtype=torch.bfloat16, device=like.device)
    _require(out.is_cuda and out.device == like.device and out.dtype == torch.bfloat16 and out.is_contiguous()
             and tuple(out.shape) == (rows, n), f"out must be a contiguous BF16 [{rows}, {n}] tensor on the device of a")
    return out


# `enable_pdl` value: programmatic dependent launch, and the weights are not written by any kernel still in flight.
PDL_STATIC_WEIGHTS = 2


class _Call:
    """The argument structs of one (weight, shape, config, launch mode): built once, patched per call."""

    __slots__ = ("args", "cfg", "routing", "args_ref", "cfg_ref", "routing_ref", "need", "unsplit_cfg_ref", "unsplit_cfg")

    def __init__(self, args, cfg, routing, need):
        self.args, self.cfg, self.routing, self.need = args, cfg, routing, need
        self.args_ref, self.cfg_ref = ctypes.byref(args), ctypes.byref(cfg)
        self.routing_ref = None if routing is None else ctypes.byref(routing)
        self.unsplit_cfg = self.unsplit_cfg_ref = None
        if need > 0:
            self.unsplit_cfg = _native.Config.from_buffer_copy(cfg)
            self.unsplit_cfg.use_stream_k = 0
            self.unsplit_cfg_ref = ctypes.byref(self.unsplit_cfg)


_dense_calls: dict[tuple, _Call] = {}
# Argument structs of dense calls whose every pointer is fixed (see `fp8_nvfp4_gemm`).
_repeat_calls: dict[tuple, tuple] = {}


def _relaunch(call: _Call, device: torch.device) -> None:
    """Launch `call` again as it stands: only the stream, its split-K scratch and the status words are looked up."""
    lib = _native.load()
    args = call.args
    index = device.index
    args.status = _native.status_words(index).data_ptr()
    stream = _native.stream_ptr(index)
    cfg_ref = call.cfg_ref
    if call.need > 0:
        workspace = _workspace(device, call.need, stream, call.cfg.use_stream_k == 1)
        if workspace is None:
            cfg_ref = call.unsplit_cfg_ref
            args.workspace, args.workspace_bytes = None, 0
        else:
            args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel() * 4
    if torch.cuda.current_device() == index:
        code = lib.tb_gemm_dense(stream, call.args_ref, cfg_ref)
    else:
        with torch.cuda.device(device):
            code = lib.tb_gemm_dense(stream, call.args_ref, cfg_ref)
    if code:
        _native.check(code)



def _launch(a, a_scale, strides, weight_t, scale_t, global_scale, locks, out, rows, n, k, bridge, group_scales,
            enable_pdl, config, routing_struct, call: _Call | None = None, scatter: PeerScatter | None = None) -> _Call:
    """One launch through the C ABI.  `call` carries the structs of an earlier launch with the same weight, shape,
    config and mode: only the activation, scale, output, workspace and status pointers are patched."""
    device = a.device
    lib = _native.load()
    if call is None:
        cfg = _config_struct(config)
        need = lib.tb_workspace_bytes(rows, n, ctypes.byref(cfg)) if routing_struct is None else 0
        args = _native.GemmArgs(
            0, 0, strides[0], strides[1], weight_t.data_ptr(), scale_t.data_ptr(), global_scale.data_ptr(),
            locks.data_ptr(), None, 0, 0, rows, n, k, _native.BRIDGE_IDS[bridge], int(group_scales), int(enable_pdl), 0,
            _native.status_words(device.index).data_ptr())
        call = _Call(args, cfg, routing_struct, need)
    args = call.args
    args.a, args.a_scale, args.d = a.data_ptr(), a_scale.data_ptr(), out.data_ptr()
    args.a_scale_stride_m, args.a_scale_stride_k = strides
    if scatter is not None:
        args.row_target, args.peer_out, args.peer_count = scatter.row_target.data_ptr(), scatter.peer_out, scatter.world
    args.status = _native.status_words(device.index).data_ptr()
    current = torch.cuda.current_device() == device.index
    stream = _native.stream_ptr(device.index)
    cfg_ref = call.cfg_ref
    if call.need > 0:
        workspace = _workspace(device, call.need, stream, call.cfg.use_stream_k == 1)
        if workspace is None:  # capturing without a buffer: run unsplit rather than allocate inside the capture
            cfg_ref = call.unsplit_cfg_ref
            args.workspace, args.workspace_bytes = None, 0
        else:
            args.workspace, args.workspace_bytes = workspace.data_ptr(), workspace.numel() * 4
    if current:
        code = (lib.tb_gemm_dense(stream, call.args_ref, cfg_ref) if call.routing is None else
                lib.tb_gemm_grouped(stream, call.args_ref, call.routing_ref, cfg_ref))
    else:
        with torch.cuda.device(device):
            code = (lib.tb_gemm_dense(stream, call.args_ref, cfg_ref) if call.routing is None else
                    lib.tb_gemm_grouped(stream, call.args_ref, call.routing_ref, cfg_ref))
    if code:
        _native.check(code)
    return call


def fp8_nvfp4_gemm(a: torch.Tensor, a_scale: torch.Tensor, weight: NVFP4Weight, out: torch.Tensor | None = None,
                   config: GemmConfig | None = None, enable_pdl: bool | int = False, *, group_scales: bool = False
                   ) -> torch.Tensor:
    """BF16 `[M, N]` = `(a * a_scale) @ dequant(weight).T`.

    `a` is FP8 E4M3 `[M, K]` with FP32 per-token scales `[M, 1]` (`tensorbridge.quant.fp8.quantize`); `weight` comes
    from `tensorbridge.quant.nvfp4.prepare` and `(N, K) = weight.shape`.  The kernel instance is chosen from the
    shape (`select_config`) unless `config` pins it.  `enable_pdl` launches with programmatic dependent launch: the
    kernel may start its set-up before the previous kernel on the stream ends and waits for it before reading any
    input, weights included, so the result is the same either way.  `enable_pdl=PDL_STATIC_WEIGHTS` additionally lets
    the kernel stream `weight` before the previous kernel has finished: for weights no kernel in flight still writes
    (anything `prepare` returned), which is how the serving layers launch.  `group_scales` (keyword only, used by
    `tensorbridge.experimental`) selects `[1,128]` activation scales `[M, K/128]` and the `[K/128, N, 8]` scale layout.
    """
    n, k = weight.shape
    repeat_key = None
    config_in = config
    if out is not None:
        # A call that repeats an earlier one pointer for pointer (a serving loop over static buffers) skips the checks
        # it has passed before and relaunches with the argument structs of that call.
        repeat_key = (weight.weight.data_ptr(), weight.scale.data_ptr(), n, k, weight.bridge, a.data_ptr(), a_scale.data_ptr(),
                      out.data_ptr(), a.size(0), a.dtype, out.dtype, int(enable_pdl), id(config), group_scales)
        again = _repeat_calls.get(repeat_key)
        if (again is not None and again[1] is config and a.is_contiguous() and out.is_contiguous()
                and a_scale.size(0) == a.size(0)):
            _relaunch(again[0], a.device)
            return out
    strides = _check_common(a, a_scale, k, group_scales)
    m = a.size(0)
    d = _output(out, m, n, a)
    if m == 0:
        return d
    if config is None:
        config = runtime.select_config(m, n, k, device=a.get_device(), bridge=weight.bridge, group_scales=group_scales)
    key = (weight.weight.data_ptr(), weight.scale.data_ptr(), weight.global_scale.data_ptr(), weight.locks.data_ptr(), m, n, k,
           weight.bridge, group_scales, int(enable_pdl), config, a.get_device())
    call = _dense_calls.get(key)
    if call is None:
        n_pad, k_pad = pad_to_unit(n), pad_to_unit(k)
        _require(weight.weight.dtype == torch.int32 and tuple(weight.weight.shape) == (n_pad, k_pad // 8)
                 and weight.weight.is_contiguous(), f"weight.weight must be contiguous int32 [{n_pad}, {k_pad // 8}]")
        want_scale = (k_pad // 128, n_pad, 8) if group_scales else (k_pad // 16, n_pad)
        _require(tuple(weight.scale.shape) == want_scale and weight.scale.is_contiguous(),
                 f"weight.scale must be contiguous {want_scale}")
        _require(weight.global_scale.numel() == 1 and weight.global_scale.dtype == torch.float32, "global_scale must be FP32 [1]")
        _require(weight.locks.dtype == torch.int32 and weight.locks.numel() >= 1024, "locks must be int32 [1024]")
        if len(_dense_calls) > 4096:
            _dense_calls.clear()
    call = _dense_calls[key] = _launch(a, a_scale, strides, weight.weight, weight.scale, weight.global_scale, weight.locks, d,
                                       m, n, k, weight.bridge, group_scales, enable_pdl, config, None, call)
    if repeat_key is not None:
        if len(_repeat_calls) > 4096:
            _repeat_calls.clear()
        # (keyed by the identity of `config`: the entry keeps the object alive, so the id cannot be reused while it is here)
        _repeat_calls[repeat_key] = (_Call(_native.GemmArgs.from_buffer_copy(call.args), _native.Config.from_buffer_copy(call.cfg),
                                           None, call.need), config_in)
    return d


def fp8_nvfp4_grouped_gemm(a: torch.Tensor, a_scale: torch.Tensor, experts: NVFP4Experts, routing: Routing, m: int,
                           out: torch.Tensor | None = None, config: GemmConfig | None = None, enable_pdl: bool = False,
                           *, group_scales: bool = False, scatter: PeerScatter | None = None) -> torch.Tensor:
    """Each expert's `(a_e * a_scale_e) @ dequant(experts.expert(e)).T` in one launch, BF16 out.

    `a_scale` is `[rows, 1]`, or `[rows, K/128]` (masked: optionally `[E, capacity, K/128]`) with `group_scales=True`,
    in which case `experts.scale` is `[E, K/128, N, 8]`.  `m` only hints the routed row count to config selection.
    Routing metadata stays on the device: nothing is read back, K is never split and tiles are dealt to CTAs in a
    fixed order, so the launch is CUDA-graph capturable and bit-identical from run to run.  Rows no route owns are
    left unwritten."""
    num_experts, n, k = experts.shape
    strides = _check_common(a, a_scale, k, group_scales)
    rows = a.size(0)
    top_k = 1
    r = _native.Routing()
    r.num_experts = num_experts
    if isinstance(routing, IndexedRouting):
        layout = "indexed"
        top_k = int(routing.top_k)
        _require(top_k >= 1, "top_k must be positive")
        for name in ("sorted_ids", "expert_ids", "num_tokens_padded"):
            t = getattr(routing, name)
            _require(t.is_cuda and t.device == a.device and t.dtype == torch.int32 and t.is_contiguous(),
                     f"{name} must be a contiguous int32 tensor on the device of a")
        _require(routing.num_tokens_padded.numel() == 1, "num_tokens_padded must have one element")
        r.layout = _native.LAYOUT_INDEXED
        r.sorted_ids, r.expert_ids = routing.sorted_ids.data_ptr(), routing.expert_ids.data_ptr()
        r.num_tokens_padded = routing.num_tokens_padded.data_ptr()
        r.sorted_capacity = routing.sorted_ids.numel()
        r.top_k = top_k
    elif isinstance(routing, ContiguousRouting):
        layout = "contiguous"
        t = routing.expert_offsets
        _require(t.is_cuda and t.device == a.device and t.dtype == torch.int64 and t.is_contiguous()
                 and t.numel() == num_experts + 1, f"expert_offsets must be contiguous int64 [{num_experts + 1}]")
        r.layout, r.expert_offsets = _native.LAYOUT_CONTIGUOUS, t.data_ptr()
    elif isinstance(routing, MaskedRouting):
        layout = "masked"
        t = routing.expert_counts
        _require(t.is_cuda and t.device == a.device and t.dtype == torch.int32 and t.is_contiguous()
                 and t.numel() == num_experts, f"expert_counts must be contiguous int32 [{num_experts}]")
        _require(rows % num_experts == 0, "masked activation rows must divide into equal expert capacities")
        r.layout, r.expert_counts = _native.LAYOUT_MASKED, t.data_ptr()
    else:
        raise ValueError(f"unknown routing {type(routing).__name__}")
    _require(experts.weight.dtype == torch.int32 and experts.weight.is_contiguous(), "experts.weight must be contiguous int32")
    want_scale = (num_experts, k // 128, n, 8) if group_scales else (num_experts, k // 16, n)
    _require(tuple(experts.scale.shape) == want_scale and experts.scale.is_contiguous(),
             f"experts.scale must be contiguous {want_scale}")
    _require(experts.global_scale.numel() == num_experts and experts.global_scale.dtype == torch.float32,
             f"global_scale must be FP32 [{num_experts}]")
    out_rows = rows * top_k if layout == "indexed" else rows
    d = _output(out, out_rows, n, a)
    if rows == 0:
        return d
    if config is None:
        config = runtime.select_config(m, n, k, num_experts, layout, device=a.get_device(), bridge=experts.bridge,
                                       top_k=top_k, group_scales=group_scales)
    if isinstance(routing, IndexedRouting):
        if routing.block_m != config.block_m:
            raise ValueError("indexed routing must be aligned to the selected block_m")
        blocks = -(-routing.sorted_ids.numel() // config.block_m)
        _require(routing.expert_ids.numel() >= blocks, "indexed routing must provide one expert per aligned block")
        scratch = _gather_buffer(a.device, routing.sorted_ids.numel() * k) if USE_GATHER_PASS else None
        if scratch is not None:
            r.gather_scratch, r.gather_scratch_bytes = scratch.data_ptr(), scratch.numel()
    if scatter is not None:
        _require(layout in ("masked", "contiguous"), "scattered output rows go with masked or contiguous routing")
        t = scatter.row_target
        _require(t.is_cuda and t.device == a.device and t.dtype == torch.int32 and t.is_contiguous() and t.numel() >= rows,
                 f"scatter.row_target must be a contiguous int32 tensor of at least {rows} entries on the device of a")
    _launch(a, a_scale, strides, experts.weight, experts.scale, experts.global_scale, experts.locks, d, rows, n, k,
            experts.bridge, group_scales, enable_pdl, config, r, scatter=scatter)
    return d
