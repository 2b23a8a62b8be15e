"""B200-native FP8-activation x NVFP4-weight GEMMs behind the TensorBridge Python API.

Dense and grouped (MoE) GEMMs, the weight layouts they take, the linear layer and config selection.  Weights come from
`tensorbridge.quant.nvfp4`, activations from `tensorbridge.quant.fp8`; `[1,128]` activation scales are in
`tensorbridge.experimental`; checkpoint-facing helpers in `tensorbridge.serving`; multi-GPU sharding in
`tensorbridge.parallel`.  All device work runs in libtensorbridge_b200.so (hand-written sm_100a kernels).
"""
from tensorbridge._native import check_status
from tensorbridge.gemm import (
    PDL_STATIC_WEIGHTS,
    ContiguousRouting,
    IndexedRouting,
    MaskedRouting,
    PeerScatter,
    Routing,
    fp8_nvfp4_gemm,
    fp8_nvfp4_grouped_gemm,
)
from tensorbridge.jit.autotune import autotune, autotune_grouped
from tensorbridge.jit.codegen import Bridge, GemmConfig
from tensorbridge.jit.runtime import select_config
from tensorbridge.linear import NVFP4Linear
from tensorbridge.quant.nvfp4 import NVFP4Experts, NVFP4Weight

__all__ = [
    "Bridge", "ContiguousRouting", "GemmConfig", "IndexedRouting", "MaskedRouting", "NVFP4Experts", "NVFP4Linear",
    "NVFP4Weight", "PDL_STATIC_WEIGHTS", "PeerScatter", "Routing", "autotune", "autotune_grouped", "check_status", "fp8_nvfp4_gemm",
    "fp8_nvfp4_grouped_gemm", "select_config",
]
