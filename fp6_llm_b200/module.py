"""A torch.nn.Module around the FPx linear layer, the form in which inference engines use the reference's kernel
(the reference's README points to DeepSpeed's FP6 linear module, README.md:19,235; the reference itself ships only the
functional operators of fp6_llm/__init__.py).

    layer = FPxLinear.from_linear(torch_linear, e_bits=3, m_bits=2)     # quantise (RTN, per-row scale) + prepack on the GPU
    y = layer(x)                                                        # x [..., IC] fp16 -> [..., OC] fp16
"""
from __future__ import annotations

import torch

from .formats import bit_width, check_format, magnitudes
from .ops import (ACT_NONE, ACT_SILU_MUL, interleave_gate_up, linear_forward_ex, linear_forward_native, native_preferred,
                  native_repack, native_supported, quantize_prepack_cuda)


def _enable_native(layer) -> None:
    rows = layer.weight.shape[0]
    if not native_supported(layer.e_bits, layer.m_bits, rows, layer.in_features, 1):
        raise ValueError("the tile layout needs OC % 256 == 0 and IC % 64 == 0")
    layer.register_buffer("weight_native", native_repack(layer.e_bits, layer.m_bits, layer.weight))


def _forward(layer, flat: torch.Tensor, activation: int) -> torch.Tensor:
    native = getattr(layer, "weight_native", None)
    if native is not None and layer.split_k == 0 and native_preferred(layer.e_bits, layer.m_bits, layer.weight.shape[0],
                                                                      layer.in_features, flat.shape[0]):
        return linear_forward_native(layer.e_bits, layer.m_bits, flat, native, layer.scales, layer.bias, activation)
    # the bias is added inside the kernel's fp32 epilogue, before the one rounding to fp16
    return linear_forward_ex(layer.e_bits, layer.m_bits, flat, layer.weight, layer.scales, layer.split_k, layer.bias, activation)


class FPxLinear(torch.nn.Module):
    """y = x @ dequant(W)^T (+ bias) with W held as prepacked FP6 (e3m2) / FP5 (e2m2) codes and fp16 row scales."""

    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None, e_bits: int = 3,
                 m_bits: int = 2, split_k: int = 0):
        super().__init__()
        check_format(e_bits, m_bits)
        if packed.dtype != torch.int32 or packed.dim() != 2 or scales.dtype != torch.float16:
            raise ValueError("expected prepacked int32 weights [OC, IC/32*bw] and fp16 scales [OC]")
        if scales.numel() != packed.shape[0] or (bias is not None and bias.numel() != packed.shape[0]):
            raise ValueError("scales and bias need one entry per output channel")
        self.e_bits, self.m_bits, self.split_k = e_bits, m_bits, split_k
        self.out_features = packed.shape[0]
        self.in_features = packed.shape[1] * 32 // bit_width(e_bits, m_bits)
        self.register_buffer("weight", packed)
        self.register_buffer("scales", scales)
        self.register_buffer("bias", bias.to(torch.float16) if bias is not None else None)

    @staticmethod
    def row_scales(weight: torch.Tensor, e_bits: int, m_bits: int) -> torch.Tensor:
        """max|w| of each output channel mapped to the format's largest magnitude (28 for e3m2, 7 for e2m2)."""
        top = float(magnitudes(e_bits, m_bits)[-1])
        return (weight.float().abs().amax(dim=1) / top).clamp_min(2.0 ** -24).to(torch.float16)

    @classmethod
    def from_linear(cls, linear: torch.nn.Linear, e_bits: int = 3, m_bits: int = 2, split_k: int = 0) -> "FPxLinear":
        """Quantise a (CUDA) torch.nn.Linear: per-row scale, round to nearest, prepacked by one kernel."""
        w = linear.weight.detach().to(torch.float16).contiguous()
        if not w.is_cuda:
            raise ValueError("the layer must live on a CUDA device: quantisation and packing run there")
        scales = cls.row_scales(w, e_bits, m_bits)
        packed = quantize_prepack_cuda(w, scales, e_bits, m_bits)
        bias = linear.bias.detach() if linear.bias is not None else None
        return cls(packed, scales, bias, e_bits, m_bits, split_k)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.float16 or x.shape[-1] != self.in_features:
            raise ValueError(f"expected fp16 activations [..., {self.in_features}]")
        flat = x.reshape(-1, self.in_features).contiguous()
        y = _forward(self, flat, ACT_NONE)
        return y.reshape(*x.shape[:-1], self.out_features)

    def enable_native(self) -> "FPxLinear":
        """Also keep the weights in the tile layout of the tensor cores' own six-bit inputs (6 more bits per weight,
        whatever the format): batches for which `native_preferred` says so (decode sizes) run on that path, the others as before."""
        _enable_native(self)
        return self

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, format=e{self.e_bits}m{self.m_bits}"


class FPxGateUpLinear(torch.nn.Module):
    """The first half of a LLaMA-style MLP in one launch: y = silu(x @ Wg^T + bg) * (x @ Wu^T + bu), with Wg and Wu held
    as ONE prepacked FPx matrix whose rows alternate gate / up, so that the kernel's epilogue sees both values of an
    output channel side by side and stores only the product ([..., C] instead of [..., 2C])."""

    def __init__(self, packed: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None, e_bits: int = 3,
                 m_bits: int = 2, split_k: int = 0):
        super().__init__()
        check_format(e_bits, m_bits)
        if packed.dtype != torch.int32 or packed.dim() != 2 or scales.dtype != torch.float16 or packed.shape[0] % 2:
            raise ValueError("expected prepacked int32 weights [2C, IC/32*bw] (rows: gate, up, gate, up, ...) and fp16 scales [2C]")
        if scales.numel() != packed.shape[0] or (bias is not None and bias.numel() != packed.shape[0]):
            raise ValueError("scales and bias need one entry per weight row")
        self.e_bits, self.m_bits, self.split_k = e_bits, m_bits, split_k
        self.out_features = packed.shape[0] // 2
        self.in_features = packed.shape[1] * 32 // bit_width(e_bits, m_bits)
        self.register_buffer("weight", packed)
        self.register_buffer("scales", scales)
        self.register_buffer("bias", bias.to(torch.float16) if bias is not None else None)

    @classmethod
    def from_linears(cls, gate: torch.nn.Linear, up: torch.nn.Linear, e_bits: int = 3, m_bits: int = 2,
                     split_k: int = 0) -> "FPxGateUpLinear":
        """Quantise two (CUDA) torch.nn.Linear layers of equal shape into one interleaved, prepacked matrix."""
        w = interleave_gate_up(gate.weight.detach().to(torch.float16), up.weight.detach().to(torch.float16))
        if not w.is_cuda:
            raise ValueError("the layers must live on a CUDA device: quantisation and packing run there")
        scales = FPxLinear.row_scales(w, e_bits, m_bits)
        packed = quantize_prepack_cuda(w, scales, e_bits, m_bits)
        bias = None
        if gate.bias is not None or up.bias is not None:
            zero = torch.zeros(gate.out_features, dtype=torch.float16, device=w.device)
            bias = interleave_gate_up(gate.bias.detach().half() if gate.bias is not None else zero,
                                      up.bias.detach().half() if up.bias is not None else zero)
        return cls(packed, scales, bias, e_bits, m_bits, split_k)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.float16 or x.shape[-1] != self.in_features:
            raise ValueError(f"expected fp16 activations [..., {self.in_features}]")
        flat = x.reshape(-1, self.in_features).contiguous()
        y = _forward(self, flat, ACT_SILU_MUL)
        return y.reshape(*x.shape[:-1], self.out_features)

    def enable_native(self) -> "FPxGateUpLinear":
        """See :meth:`FPxLinear.enable_native`."""
        _enable_native(self)
        return self

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features} (gate and up fused), format=e{self.e_bits}m{self.m_bits}"
