"""B200-native (sm_100a) NVFP4 fused-MoE layer behind the operator surface of sm120fp4.

Public names follow the reference package (`sm120fp4/__init__.py:3-22`): quantize_nvfp4, global_scale_for, to_128x4,
from_128x4, padded_sf_shape; the operator lives in `vllm_backend` (Weights, weights_from_vllm_layout, register).
Everything computes on the GPU through the C ABI of include/b200moe.h; there is no CPU fallback."""
__version__ = "0.1.0"

from .layouts import from_128x4, padded_sf_shape, to_128x4  # noqa: E402,F401
from .quant import global_scale_for, quantize_nvfp4, quantize_nvfp4_128x4, quantize_nvfp4_experts  # noqa: E402,F401
from .router import route, route_tables  # noqa: E402,F401
