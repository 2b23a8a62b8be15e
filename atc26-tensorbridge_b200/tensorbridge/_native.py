"""ctypes binding of libtensorbridge_b200.so (C ABI in include/tensorbridge_b200.h).

There is no fallback: if the library is missing or a call fails, the caller gets an exception.  The library is
looked up next to this package (`atc26-tensorbridge_b200/libtensorbridge_b200.so`), or at `TENSORBRIDGE_B200_LIB`.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_LIB_NAME = "libtensorbridge_b200.so"
_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE = range(5)
LAYOUT_DENSE, LAYOUT_INDEXED, LAYOUT_CONTIGUOUS, LAYOUT_MASKED = range(4)
BRIDGE_IDS = {"fpma": 0, "exact": 1}
DTYPE_IDS = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
QUANT_PER_TOKEN, QUANT_GROUP_128 = 0, 1


class Config(ctypes.Structure):
    """`tb_config`: the nine GemmConfig fields in wire order."""

    _fields_ = [(name, ctypes.c_int32) for name in (
        "block_m", "num_stages", "use_stream_k", "m_fast_tile_order", "block_k", "block_n", "ctas_per_sm",
        "stream_k_aligned", "math_warpgroups")]


class Problem(ctypes.Structure):
    _fields_ = [("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64), ("num_sms", ctypes.c_int32),
                ("num_experts", ctypes.c_int32), ("layout", ctypes.c_int32), ("group_scales", ctypes.c_int32),
                ("split_k_override", ctypes.c_int32)]


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p), ("a_scale", ctypes.c_void_p), ("a_scale_stride_m", ctypes.c_int64),
        ("a_scale_stride_k", ctypes.c_int64), ("weight", ctypes.c_void_p), ("scale", ctypes.c_void_p),
        ("global_scale", ctypes.c_void_p), ("locks", ctypes.c_void_p), ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_int64), ("d", ctypes.c_void_p), ("rows", ctypes.c_int64), ("n", ctypes.c_int64),
        ("k", ctypes.c_int64), ("bridge", ctypes.c_int32), ("group_scales", ctypes.c_int32),
        ("enable_pdl", ctypes.c_int32), ("num_sms", ctypes.c_int32), ("status", ctypes.c_void_p),
        ("wait_us", ctypes.c_int32), ("only_split", ctypes.c_int32), ("row_target", ctypes.c_void_p),
        ("peer_out", ctypes.POINTER(ctypes.c_void_p)), ("peer_count", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class Routing(ctypes.Structure):
    _fields_ = [
        ("layout", ctypes.c_int32), ("num_experts", ctypes.c_int32), ("expert_offsets", ctypes.c_void_p),
        ("expert_counts", ctypes.c_void_p), ("sorted_ids", ctypes.c_void_p), ("expert_ids", ctypes.c_void_p),
        ("num_tokens_padded", ctypes.c_void_p), ("sorted_capacity", ctypes.c_int64), ("top_k", ctypes.c_int32),
        ("gather_scratch", ctypes.c_void_p), ("gather_scratch_bytes", ctypes.c_int64),
    ]


class QuantMoeArgs(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("x_dtype", ctypes.c_int32), ("mode", ctypes.c_int32), ("x_stride", ctypes.c_int64),
        ("rows", ctypes.c_int64), ("width", ctypes.c_int64), ("activation", ctypes.c_int32), ("use_division", ctypes.c_int32),
        ("expert_counts", ctypes.c_void_p), ("num_experts", ctypes.c_int64), ("num_valid_rows", ctypes.c_void_p),
        ("scatter_idx", ctypes.c_void_p), ("top_k", ctypes.c_int32), ("num_valid_rows_int64", ctypes.c_int32),
        ("out_rows", ctypes.c_int64), ("q", ctypes.c_void_p), ("scale", ctypes.c_void_p),
    ]


class PushArgs(ctypes.Structure):
    """`tb_ep_push_args`."""

    _fields_ = [
        ("topk_ids", ctypes.c_void_p), ("ids_int64", ctypes.c_int32), ("top_k", ctypes.c_int32), ("routes", ctypes.c_int64),
        ("x", ctypes.c_void_p), ("scale", ctypes.c_void_p), ("width", ctypes.c_int64), ("groups", ctypes.c_int64),
        ("route_rank", ctypes.c_void_p), ("all_counts", ctypes.c_void_p), ("num_experts", ctypes.c_int32),
        ("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("interleaved", ctypes.c_int32), ("capacity", ctypes.c_int32),
        ("reserved", ctypes.c_int32), ("peer_a", ctypes.POINTER(ctypes.c_void_p)), ("peer_a_scale", ctypes.POINTER(ctypes.c_void_p)),
        ("dest_row", ctypes.c_void_p), ("counts", ctypes.c_void_p), ("peer_row_target", ctypes.POINTER(ctypes.c_void_p)),
        ("out", ctypes.c_void_p), ("out_row_bytes", ctypes.c_int64),
    ]


class KernelKey(ctypes.Structure):
    """`tb_kernel_key`."""

    _fields_ = [(name, ctypes.c_int32) for name in ("device", "block_m", "exact", "group_scales", "bridge_warps", "teams")]


# Every symbol include/tensorbridge_b200.h declares: (restype, argtypes).
SYMBOLS = {
    "tb_last_error": (ctypes.c_char_p, []),
    "tb_version": (ctypes.c_char_p, []),
    "tb_num_sms": (ctypes.c_int, [ctypes.c_int, ctypes.POINTER(ctypes.c_int)]),
    "tb_select_config": (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(Config)]),
    "tb_workspace_bytes": (ctypes.c_int64, [ctypes.c_int64, ctypes.c_int64, ctypes.POINTER(Config)]),
    "tb_quantize_fp8": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int64,
                                       ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_int64]),
    "tb_quantize_moe": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(QuantMoeArgs)]),
    "tb_scatter_fp8": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                      ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int64,
                                      ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "tb_prepare_weight": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                         ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p]),
    "tb_bridge_dump": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "tb_register_kernel": (ctypes.c_int, [ctypes.POINTER(KernelKey), ctypes.c_void_p]),
    "tb_registered_kernels": (ctypes.c_int, []),
    "tb_gemm_dense": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(GemmArgs), ctypes.POINTER(Config)]),
    "tb_gemm_dense_static_scratch": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(GemmArgs), ctypes.POINTER(Config)]),
    "tb_gemm_grouped": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(GemmArgs), ctypes.POINTER(Routing),
                                       ctypes.POINTER(Config)]),
    "tb_ep_plan": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32,
                                  ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "tb_ep_pack": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                  ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]),
    "tb_ep_layout": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                    ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "tb_ep_place": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "tb_gather_rows": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_void_p]),
    "tb_moe_combine": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                      ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p]),
    "tb_peer_alloc": (ctypes.c_int, [ctypes.c_int64, ctypes.POINTER(ctypes.c_void_p)]),
    "tb_peer_free": (ctypes.c_int, [ctypes.c_void_p]),
    "tb_ipc_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "tb_ipc_open": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]),
    "tb_ipc_close": (ctypes.c_int, [ctypes.c_void_p]),
    "tb_peer_barrier": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                       ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                       ctypes.c_int32, ctypes.c_void_p]),
    "tb_ep_push": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(PushArgs)]),
    "tb_ep_pull": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                  ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_void_p]),
}


def library_path() -> str:
    override = os.environ.get("TENSORBRIDGE_B200_LIB")
    if override:
        return override
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), _LIB_NAME)


def load() -> ctypes.CDLL:
    """The loaded library; raises RuntimeError if it has not been built (`python atc26-tensorbridge_b200/build.py`)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = library_path()
            if not os.path.exists(path):
                raise RuntimeError(f"{path} is missing: build it with `python atc26-tensorbridge_b200/build.py`; "
                                   "there is no fallback path")
            lib = ctypes.CDLL(path)
            for name, (restype, argtypes) in SYMBOLS.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = restype, argtypes
            _lib = lib
    return _lib


def check(code: int) -> None:
    """Raise for a non-zero status: ValueError for rejected arguments, RuntimeError otherwise."""
    if code == OK:
        return
    message = load().tb_last_error().decode()
    if code in (ERR_INVALID, ERR_UNSUPPORTED):
        raise ValueError(message)
    raise RuntimeError(message)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device | int) -> int:
    """The `cudaStream_t` of torch's current stream on `device`, as an integer."""
    if _raw_stream is not None:
        return _raw_stream(device if isinstance(device, int) else device.index)
    return torch.cuda.current_stream(device).cuda_stream


def ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


# Per-device status words the GEMM kernels write when a bounded wait gives up.
_status: dict[int, torch.Tensor] = {}
# Called with the device index when check_status() finds an error (the GEMM module zeroes its split-K scratch there).
error_hooks: list = []


def status_words(device: int) -> torch.Tensor:
    words = _status.get(device)
    if words is None:
        words = _status[device] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", device))
    return words


def check_status(device: int | None = None) -> None:
    """Synchronise and raise RuntimeError if a kernel on `device` reported a timed-out wait since the last check."""
    device = torch.cuda.current_device() if device is None else device
    words = _status.get(device)
    if words is None:
        return
    host = words.tolist()
    if host[0] != 0:
        words.zero_()
        for hook in error_hooks:
            hook(device)
        raise RuntimeError(f"tensorbridge kernel gave up waiting (site {host[0]}, block {host[1]}, units {host[2]})")
