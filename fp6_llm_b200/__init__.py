"""fp6_llm_b200: the FP6-LLM / Quant-LLM mixed-input linear layer (FP6 e3m2 or FP5 e2m2 weights x FP16
activations) for NVIDIA B200 (sm_100a), behind the reference project's own operator names.

Drop-in for ``import fp6_llm`` on this path: same six operator functions, ``Num_Wave`` and
``HeuristicFuntion_SplitK`` (reference: fp6_llm/__init__.py:1-23).
"""
from ._native import build, lib
from .module import FPxGateUpLinear, FPxLinear
from .ops import (HeuristicFuntion_SplitK, Num_Wave, dequant_packed_cuda, device_status, heuristic_split_k_b200, set_static_weights, static_weights, set_programmatic_launch, quantize_prepack_cuda,
                  linear_forward_cuda, linear_forward_eXmY_cuda, linear_forward_ex, interleave_gate_up, ACT_NONE, ACT_SILU_MUL, linear_forward_host, linear_forward_host_batch, weight_dequant_cpu,
                  weight_dequant_eXmY_cpu, weight_prepacking_cpu, weight_prepacking_eXmY_cpu, native_supported, native_preferred, native_repack,
                  linear_forward_native, NATIVE_MAX_TOKENS, NATIVE_AUTO_MAX)

__all__ = [
    "linear_forward_cuda", "weight_prepacking_cpu", "weight_dequant_cpu", "linear_forward_eXmY_cuda",
    "weight_prepacking_eXmY_cpu", "weight_dequant_eXmY_cpu", "Num_Wave", "HeuristicFuntion_SplitK",
    "heuristic_split_k_b200", "dequant_packed_cuda", "linear_forward_host", "linear_forward_host_batch", "device_status", "set_static_weights", "static_weights", "set_programmatic_launch", "quantize_prepack_cuda", "FPxLinear", "FPxGateUpLinear", "linear_forward_ex", "interleave_gate_up", "ACT_NONE", "ACT_SILU_MUL", "build", "lib", "native_supported", "native_preferred", "native_repack", "linear_forward_native", "NATIVE_MAX_TOKENS", "NATIVE_AUTO_MAX",
]
