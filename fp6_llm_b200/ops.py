"""Python operators with the reference's names, argument order and meaning (fp6_llm/__init__.py:1-23,
fp6_llm/csrc/pybind.cpp:9-15), implemented on the C interface of libfp6_b200.so.

torch is used for device memory and streams only.  All compute runs in the library's CUDA kernels;
there is no CPU implementation behind these functions, so a machine without a CUDA device raises.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _native
from .formats import bit_width, check_format


# ----------------------------------------------------------------------------- reference heuristic
def Num_Wave(M, N, SplitK, Num_GPU_SMs):
    """Same formula as the reference (fp6_llm/__init__.py:6-8): waves of its 256-row, 2-CTA/SM kernel."""
    return math.ceil(M / 512) * math.ceil(N / 64) * SplitK / Num_GPU_SMs


def HeuristicFuntion_SplitK(M, N, Num_GPU_SMs):
    """The reference's split-K choice, unchanged (fp6_llm/__init__.py:13-23): the first k in 1..99 whose
    last wave is at least 80 % full, else 1.  M = weight rows, N = batch.  The name keeps the reference's
    spelling.  For this library's own kernel on B200 use :func:`heuristic_split_k_b200`."""
    split_k = 1
    for i in range(1, 100):
        waves = Num_Wave(M, N, i, Num_GPU_SMs)
        if waves / math.ceil(waves) >= 0.8:
            split_k = i
            break
    return split_k


def heuristic_split_k_b200(M: int, N: int, K: int, num_sms: int = 148) -> int:
    """Split-K for the sm_100a kernel: 128-row tiles, one CTA per SM, K-aware (C: fp6b200_choose_split_k)."""
    return int(_native.lib().fp6b200_choose_split_k(M, N, K, num_sms))


# ----------------------------------------------------------------------------- helpers
def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("fp6_llm_b200 needs a CUDA device (sm_100a); there is no CPU implementation")


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


_workspaces: dict = {}
_retired: list = []


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Grow-only fp32 split-K workspace per (device, stream) (the reference allocates one per call,
    fp6_llm/csrc/fp6_linear.cu:185-187): calls on one stream run in order and may share it, calls on different
    streams get their own.  A buffer that is outgrown is kept alive until the process ends, because work already
    queued (or captured in a CUDA graph) may still use it."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() * 4 < nbytes:
        if ws is not None:
            _retired.append(ws)
        ws = torch.empty(max(nbytes // 4, 1 << 20), dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def _in_channels(weights: torch.Tensor, e_bits: int, m_bits: int) -> int:
    bw = bit_width(e_bits, m_bits)
    if weights.dim() != 2 or (weights.shape[1] * 32) % bw:
        raise ValueError(f"weight tensor of shape {tuple(weights.shape)} is not [OC, IC/32*{bw}]")
    return weights.shape[1] * 32 // bw


# ----------------------------------------------------------------------------- linear layer
ACT_NONE, ACT_SILU_MUL = 0, 1


def _linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK, bias, activation):
    _require_cuda()
    check_format(EXPONENT, MANTISSA)
    if _in_feats.dtype != torch.float16 or _scales.dtype != torch.float16 or _weights.dtype != torch.int32:
        raise ValueError("expected fp16 activations, int32 packed weights and fp16 scales")
    if not (_in_feats.is_cuda and _weights.is_cuda and _scales.is_cuda):
        raise ValueError("all tensors must be CUDA tensors")
    if not (_in_feats.device == _weights.device == _scales.device):
        raise ValueError("all tensors must be on the same device")
    if _in_feats.dim() != 2:
        raise ValueError("activations must be [B, IC]")
    if not (_in_feats.is_contiguous() and _weights.is_contiguous() and _scales.is_contiguous()):
        raise ValueError("tensors must be contiguous")
    B, IC = _in_feats.shape
    OC = _weights.shape[0]
    if _in_channels(_weights, EXPONENT, MANTISSA) != IC:
        raise ValueError(f"K mismatch: activations have IC={IC}, weights encode IC={_in_channels(_weights, EXPONENT, MANTISSA)}")
    if IC % 64 or OC % 256 or B < 1:
        raise ValueError("need IC % 64 == 0, OC % 256 == 0 and B >= 1")
    if _scales.numel() != OC:
        raise ValueError("scales must have OC elements")
    if splitK < 0:
        raise ValueError("splitK must be >= 0")
    if activation not in (ACT_NONE, ACT_SILU_MUL):
        raise ValueError("activation must be ACT_NONE or ACT_SILU_MUL")
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != OC or bias.device != _in_feats.device
                             or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous fp16 tensor with OC elements on the layer's device")
    dev = _in_feats.device
    L = _native.lib()
    with torch.cuda.device(dev):
        nbytes = L.fp6b200_workspace_bytes(OC, B, IC, splitK)
        ws = _workspace(dev, nbytes) if nbytes else None
        out = torch.empty((B, OC // 2 if activation == ACT_SILU_MUL else OC), dtype=torch.float16, device=dev)
        if bias is None and activation == ACT_NONE:
            rc = L.fp6b200_linear(EXPONENT, MANTISSA, _stream_ptr(dev), _ptr(_weights), _ptr(_scales), _ptr(_in_feats),
                                  _ptr(out), OC, B, IC, _ptr(ws) if ws is not None else None, splitK)
        else:
            rc = L.fp6b200_linear_ex(EXPONENT, MANTISSA, _stream_ptr(dev), _ptr(_weights), _ptr(_scales), _ptr(_in_feats),
                                     _ptr(out), OC, B, IC, _ptr(ws) if ws is not None else None, splitK,
                                     _ptr(bias) if bias is not None else None, activation)
    _native.check(rc, "fp6b200_linear")
    return out


def linear_forward_eXmY_cuda(EXPONENT: int, MANTISSA: int, _in_feats: torch.Tensor, _weights: torch.Tensor,
                             _scales: torch.Tensor, splitK: int = 1) -> torch.Tensor:
    """Out[B, OC] = In[B, IC] @ dequant(W)[OC, IC]^T  (fp_eXmY_linear_forward_cuda,
    fp6_llm/csrc/fp6_linear.cu:269-313).

    _in_feats  fp16 [B, IC] cuda;  _weights  int32 [OC, IC/32*(1+E+M)] cuda, prepacked;
    _scales    fp16 [OC] cuda;     splitK >= 1 as in the reference, 0 = let the library choose.
    Runs on the current torch stream (the reference uses the legacy default stream)."""
    return _linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK, None, ACT_NONE)


def linear_forward_ex(EXPONENT: int, MANTISSA: int, _in_feats: torch.Tensor, _weights: torch.Tensor, _scales: torch.Tensor,
                      splitK: int = 0, bias: torch.Tensor | None = None, activation: int = ACT_NONE) -> torch.Tensor:
    """The layer with the epilogue fused into the kernel (C: fp6b200_linear_ex; the reference has no such entry): an fp16
    bias [OC] added in fp32 before the one rounding, and optionally ACT_SILU_MUL, for which the weight rows come in
    (gate, up) pairs - see :func:`interleave_gate_up` - and the result is [B, OC/2] = silu(gate) * up."""
    return _linear(EXPONENT, MANTISSA, _in_feats, _weights, _scales, splitK, bias, activation)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Row order ACT_SILU_MUL expects: row 2c = gate[c], row 2c+1 = up[c].  Works on weights [C, IC], scales [C] or biases
    [C]; apply it to the fp16 weights BEFORE quantising and packing (or to the unpacked code tensor before prepacking)."""
    if gate.shape != up.shape:
        raise ValueError("gate and up must have the same shape")
    return torch.stack([gate, up], dim=1).reshape(gate.shape[0] * 2, *gate.shape[1:]).contiguous()


# ----------------------------------------------------------------------------- the tensor cores' own six-bit inputs
NATIVE_MAX_TOKENS = 64     # what linear_forward_native takes
NATIVE_AUTO_MAX = 32       # the largest batch for which it is ever chosen automatically (see native_preferred)


def native_supported(EXPONENT: int, MANTISSA: int, OC: int, IC: int, B: int) -> bool:
    """Whether :func:`linear_forward_native` takes this format and shape (OC % 256 == 0, IC % 64 == 0, 1 <= B <= 64)."""
    return bool(_native.lib().fp6b200_native_supported(EXPONENT, MANTISSA, OC, B, IC))


def native_preferred(EXPONENT: int, MANTISSA: int, OC: int, IC: int, B: int) -> bool:
    """Whether :func:`linear_forward_native` measured faster than the fp16-pattern kernel for this shape (at most 32
    tokens): the rule the modules and the sharded layer choose by."""
    return bool(_native.lib().fp6b200_native_preferred(EXPONENT, MANTISSA, OC, B, IC))


def native_repack(EXPONENT: int, MANTISSA: int, _weights: torch.Tensor) -> torch.Tensor:
    """Prepacked weights (int32 [OC, IC/32*bw], the output of the packer) -> the tile layout :func:`linear_forward_native`
    reads (uint8, 128 x 128 tiles of 12 KB, six-bit codes in little-endian bit order; codes narrower than six bits are
    widened to the tensor-core format with the same exponent field, which holds their values exactly).  Once per weight
    tensor, on the GPU (C: fp6b200_native_repack; the reference has no counterpart)."""
    _require_cuda()
    if not _weights.is_cuda or _weights.dtype != torch.int32 or not _weights.is_contiguous():
        raise ValueError("expected a contiguous int32 CUDA tensor of prepacked weights")
    OC, IC = _weights.shape[0], _in_channels(_weights, EXPONENT, MANTISSA)
    L = _native.lib()
    if not L.fp6b200_native_supported(EXPONENT, MANTISSA, OC, 1, IC):
        raise ValueError("the native path needs OC % 256 == 0 and IC % 64 == 0")
    dev = _weights.device
    with torch.cuda.device(dev):
        out = torch.empty(L.fp6b200_native_weight_bytes(OC, IC), dtype=torch.uint8, device=dev)
        rc = L.fp6b200_native_repack(EXPONENT, MANTISSA, _stream_ptr(dev), _ptr(_weights), _ptr(out), OC, IC)
    _native.check(rc, "fp6b200_native_repack")
    return out


def linear_forward_native(EXPONENT: int, MANTISSA: int, _in_feats: torch.Tensor, _weights_native: torch.Tensor,
                          _scales: torch.Tensor, bias: torch.Tensor | None = None, activation: int = ACT_NONE) -> torch.Tensor:
    """Out[B, OC] = In[B, IC] @ dequant(W)[OC, IC]^T with the weights in the layout of :func:`native_repack`, for up to
    64 tokens (C: fp6b200_linear_native).  Same result as :func:`linear_forward_ex` up to fp32 summation order: the
    activations enter the tensor cores as four exact e5m2 planes and the six-bit codes as they are."""
    _require_cuda()
    if _in_feats.dtype != torch.float16 or _scales.dtype != torch.float16 or _weights_native.dtype != torch.uint8:
        raise ValueError("expected fp16 activations, uint8 native weights and fp16 scales")
    if not (_in_feats.is_cuda and _weights_native.is_cuda and _scales.is_cuda):
        raise ValueError("all tensors must be CUDA tensors")
    if not (_in_feats.device == _weights_native.device == _scales.device):
        raise ValueError("all tensors must be on the same device")
    if _in_feats.dim() != 2 or not (_in_feats.is_contiguous() and _weights_native.is_contiguous() and _scales.is_contiguous()):
        raise ValueError("activations must be a contiguous [B, IC]; weights and scales contiguous")
    B, IC = _in_feats.shape
    OC = _scales.numel()
    L = _native.lib()
    if not L.fp6b200_native_supported(EXPONENT, MANTISSA, OC, B, IC):
        raise ValueError("the native path takes OC % 256 == 0, IC % 64 == 0 and 1 <= B <= 64")
    if _weights_native.numel() != L.fp6b200_native_weight_bytes(OC, IC):
        raise ValueError("native weight tensor does not match OC (from the scales) and IC (from the activations)")
    if activation not in (ACT_NONE, ACT_SILU_MUL):
        raise ValueError("activation must be ACT_NONE or ACT_SILU_MUL")
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != OC or bias.device != _in_feats.device
                             or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous fp16 tensor with OC elements on the layer's device")
    dev = _in_feats.device
    with torch.cuda.device(dev):
        ws = _workspace(dev, L.fp6b200_native_workspace_bytes(B, IC))
        out = torch.empty((B, OC // 2 if activation == ACT_SILU_MUL else OC), dtype=torch.float16, device=dev)
        rc = L.fp6b200_linear_native(EXPONENT, MANTISSA, _stream_ptr(dev), _ptr(_weights_native), _ptr(_scales),
                                     _ptr(_in_feats), _ptr(out), OC, B, IC, _ptr(ws),
                                     _ptr(bias) if bias is not None else None, activation)
    _native.check(rc, "fp6b200_linear_native")
    return out


def linear_forward_cuda(*args) -> torch.Tensor:
    """FP6 (e3m2) linear layer (fp6_linear_forward_cuda, fp6_llm/csrc/fp6_linear.cu:161-201).

    Code order, as bound by the reference (fp6_llm/csrc/pybind.cpp:9): (activation, packed_weight, scale, splitK).
    The order printed in the reference's README, (packed_weight, scale, activation, splitK), is accepted too and
    told apart by the dtype of the first argument."""
    if len(args) == 3:
        args = (*args, 1)
    if len(args) != 4:
        raise TypeError("linear_forward_cuda(activation, packed_weight, scale, splitK)")
    a, b, c, split_k = args
    if isinstance(a, torch.Tensor) and a.dtype == torch.int32:   # README order
        a, b, c = c, a, b
    return linear_forward_eXmY_cuda(3, 2, a, b, c, int(split_k))


# ----------------------------------------------------------------------------- prepacking
def weight_prepacking_eXmY_cpu(EXPONENT: int, MANTISSA: int, fpx_tensor: torch.Tensor) -> torch.Tensor:
    """Unpacked int32 [OC, IC/32*bw] -> prepacked tensor of the same shape, bit-identical to the reference's
    weight_matrix_prepacking_fp_eXmY_cpu (fp6_llm/csrc/fp6_linear.cu:323-341).

    A CPU tensor (the reference's case) is staged through the GPU and a CPU tensor comes back; a CUDA tensor is
    packed on its device into a NEW tensor (the device kernel gathers from all over the matrix and cannot work in
    place).  Either way the packing itself runs in the CUDA kernel."""
    _require_cuda()
    check_format(EXPONENT, MANTISSA)
    if fpx_tensor.dtype != torch.int32 or fpx_tensor.dim() != 2:
        raise ValueError("expected an int32 [OC, IC/32*bw] tensor")
    IC = _in_channels(fpx_tensor, EXPONENT, MANTISSA)
    OC = fpx_tensor.shape[0]
    if OC % 256 or IC % 64:
        raise ValueError("need OC % 256 == 0 and IC % 64 == 0")
    src = fpx_tensor.contiguous()
    out = torch.empty_like(src)
    L = _native.lib()
    if src.is_cuda:
        with torch.cuda.device(src.device):
            rc = L.fp6b200_prepack(EXPONENT, MANTISSA, _stream_ptr(src.device), _ptr(src), _ptr(out), OC, IC)
    else:
        rc = L.fp6b200_prepack_host(EXPONENT, MANTISSA, _ptr(out), _ptr(src), OC, IC)
    _native.check(rc, "fp6b200_prepack")
    return out


def quantize_prepack_cuda(weights: torch.Tensor, scales: torch.Tensor, EXPONENT: int = 3, MANTISSA: int = 2) -> torch.Tensor:
    """fp16 CUDA weights [OC, IC] and fp16 row scales [OC] -> prepacked int32 [OC, IC/32*bw] in one kernel: round to
    nearest (ties to the even code, saturating) and the reference's packed layout
    (fp6_llm/csrc/utils/weight_prepacking.h:118-196).  Same bits as quantising with formats.quantize_rtn, packing the
    codes and prepacking them.  The reference has no bound quantiser (fp6_llm/csrc/utils/weight_quant.h is unused)."""
    _require_cuda()
    check_format(EXPONENT, MANTISSA)
    if weights.dtype != torch.float16 or scales.dtype != torch.float16 or not (weights.is_cuda and scales.is_cuda):
        raise ValueError("expected fp16 CUDA weights and scales")
    if weights.dim() != 2 or scales.numel() != weights.shape[0]:
        raise ValueError("expected weights [OC, IC] and one scale per output channel")
    OC, IC = weights.shape
    if OC % 256 or IC % 64:
        raise ValueError("need OC % 256 == 0 and IC % 64 == 0")
    src, sc = weights.contiguous(), scales.contiguous()
    out = torch.empty((OC, IC * bit_width(EXPONENT, MANTISSA) // 32), dtype=torch.int32, device=weights.device)
    with torch.cuda.device(weights.device):
        rc = _native.lib().fp6b200_quantize_prepack(EXPONENT, MANTISSA, _stream_ptr(weights.device), _ptr(src), _ptr(sc),
                                                    _ptr(out), OC, IC)
    _native.check(rc, "fp6b200_quantize_prepack")
    return out


def weight_prepacking_cpu(fp6_tensor: torch.Tensor) -> torch.Tensor:
    """FP6 case of :func:`weight_prepacking_eXmY_cpu` (weight_matrix_prepacking_cpu, fp6_llm/csrc/fp6_linear.cu:211-223)."""
    return weight_prepacking_eXmY_cpu(3, 2, fp6_tensor)


# ----------------------------------------------------------------------------- dequantisation
def weight_dequant_eXmY_cpu(EXPONENT: int, MANTISSA: int, fpx_tensor: torch.Tensor, fp16_scale: torch.Tensor) -> torch.Tensor:
    """UNPACKED int32 [OC, IC/32*bw] + fp16 scale [OC] -> fp16 [OC, IC], bit-identical to the reference's
    weight_matrix_dequant_fp_eXmY_cpu (fp6_llm/csrc/fp6_linear.cu:352-375).  CPU tensors are staged through
    the GPU; CUDA tensors stay on their device."""
    _require_cuda()
    check_format(EXPONENT, MANTISSA)
    if fpx_tensor.dtype != torch.int32 or fp16_scale.dtype != torch.float16:
        raise ValueError("expected int32 weights and fp16 scales")
    IC = _in_channels(fpx_tensor, EXPONENT, MANTISSA)
    OC = fpx_tensor.shape[0]
    if fp16_scale.numel() != OC:
        raise ValueError("scales must have OC elements")
    if OC % 64 or IC % 64:
        raise ValueError("need OC % 64 == 0 and IC % 64 == 0")
    if fpx_tensor.device != fp16_scale.device:
        raise ValueError("weights and scales must be on the same device")
    src, sc = fpx_tensor.contiguous(), fp16_scale.contiguous()
    out = torch.empty((OC, IC), dtype=torch.float16, device=src.device)
    L = _native.lib()
    if src.is_cuda:
        with torch.cuda.device(src.device):
            rc = L.fp6b200_dequant(EXPONENT, MANTISSA, _stream_ptr(src.device), _ptr(src), _ptr(sc), _ptr(out), OC, IC)
    else:
        rc = L.fp6b200_dequant_host(EXPONENT, MANTISSA, _ptr(out), _ptr(src), OC, IC, _ptr(sc))
    _native.check(rc, "fp6b200_dequant")
    return out


def weight_dequant_cpu(fp6_tensor: torch.Tensor, fp16_scale: torch.Tensor) -> torch.Tensor:
    """FP6 case of :func:`weight_dequant_eXmY_cpu` (weight_matrix_dequant_cpu, fp6_llm/csrc/fp6_linear.cu:234-251)."""
    return weight_dequant_eXmY_cpu(3, 2, fp6_tensor, fp16_scale)


def dequant_packed_cuda(EXPONENT: int, MANTISSA: int, packed: torch.Tensor, fp16_scale: torch.Tensor) -> torch.Tensor:
    """PREPACKED int32 weights (cuda) + scales -> fp16 [OC, IC]: the matrix the GEMM multiplies by.  Not in the
    reference (its GPU dequantiser only exists fused in the GEMM); used for fp16-GEMM comparisons."""
    _require_cuda()
    check_format(EXPONENT, MANTISSA)
    if not packed.is_cuda or packed.dtype != torch.int32 or fp16_scale.dtype != torch.float16:
        raise ValueError("expected cuda int32 packed weights and fp16 scales")
    IC = _in_channels(packed, EXPONENT, MANTISSA)
    OC = packed.shape[0]
    out = torch.empty((OC, IC), dtype=torch.float16, device=packed.device)
    with torch.cuda.device(packed.device):
        rc = _native.lib().fp6b200_dequant_packed(EXPONENT, MANTISSA, _stream_ptr(packed.device), _ptr(packed.contiguous()),
                                                  _ptr(fp16_scale.contiguous()), _ptr(out), OC, IC)
    _native.check(rc, "fp6b200_dequant_packed")
    return out


def linear_forward_host(EXPONENT: int, MANTISSA: int, act_host: torch.Tensor, packed_dev: torch.Tensor,
                        scales_dev: torch.Tensor, out_host: torch.Tensor, splitK: int = 0) -> torch.Tensor:
    """The layer with HOST activations/output (ideally pinned) and device-resident weights: host->device copy,
    kernels, device->host copy, synchronise (C: fp6b200_linear_host_io)."""
    _require_cuda()
    B, IC = act_host.shape
    OC = packed_dev.shape[0]
    with torch.cuda.device(packed_dev.device):
        rc = _native.lib().fp6b200_linear_host_io(EXPONENT, MANTISSA, _ptr(packed_dev), _ptr(scales_dev), _ptr(act_host),
                                                  _ptr(out_host), OC, B, IC, splitK)
    _native.check(rc, "fp6b200_linear_host_io")
    return out_host


def linear_forward_host_batch(calls) -> None:
    """Several host-buffer layers as one pipelined batch (C: fp6b200_linear_host_io_batch): `calls` is a sequence of
    (EXPONENT, MANTISSA, act_host, packed_dev, scales_dev, out_host, splitK[, native_dev]); host tensors should be pinned.
    The copy of the next call's activations and of the previous call's result overlap the current call's kernels; returns
    when every output has arrived.  With native_dev (the weights in the layout of :func:`native_repack`) calls of up to
    NATIVE_AUTO_MAX tokens with splitK == 0 run on the tensor cores' own six-bit inputs."""
    _require_cuda()
    calls = list(calls)
    if not calls:
        return
    arr = (_native.HostCall * len(calls))()
    dev = calls[0][3].device
    for i, call in enumerate(calls):
        e, m, act, packed, scales, out, split_k = call[:7]
        native = call[7] if len(call) > 7 else None
        check_format(e, m)
        if native is not None and (native.device != dev or native.dtype != torch.uint8 or not native.is_contiguous()):
            raise ValueError("native weights must be a contiguous uint8 tensor on the batch's device")
        if packed.device != dev or scales.device != dev:
            raise ValueError("all layers of a batch must live on one device")
        if act.is_cuda or out.is_cuda or act.dtype != torch.float16 or out.dtype != torch.float16:
            raise ValueError("activations and outputs of the host entry points are fp16 CPU tensors")
        B, IC = act.shape
        OC = packed.shape[0]
        if _in_channels(packed, e, m) != IC or tuple(out.shape) != (B, OC) or not (act.is_contiguous() and out.is_contiguous()):
            raise ValueError("shape mismatch between activations, packed weights and output")
        arr[i] = _native.HostCall(e, m, packed.data_ptr(), scales.data_ptr(), act.data_ptr(), out.data_ptr(), OC, B, IC, split_k,
                                  native.data_ptr() if native is not None else None)
    with torch.cuda.device(dev):
        rc = _native.lib().fp6b200_linear_host_io_batch(arr, len(calls))
    _native.check(rc, "fp6b200_linear_host_io_batch")


def set_static_weights(on: bool) -> None:
    """Promise (or withdraw the promise) that packed weights are prepacked ahead of time and only read afterwards:
    no work still in flight on a stream writes the weights of a linear layer launched on that stream.  The GEMM then
    requests and unpacks its first weight stages while the previous kernel of the stream is still finishing.
    After a prepack, synchronise (or wait on an event) before the first layer that uses the result."""
    _native.check(_native.lib().fp6b200_set_option(1, 1 if on else 0), "fp6b200_set_option")


def set_programmatic_launch(on: bool) -> None:
    """Let (default) or do not let a GEMM start while the previous kernel of its stream is finishing."""
    _native.check(_native.lib().fp6b200_set_option(2, 1 if on else 0), "fp6b200_set_option")


def static_weights() -> bool:
    return _native.lib().fp6b200_get_option(1) == 1


def device_status() -> int:
    """Synchronise and return (then clear) the time-out code a GEMM CTA may have recorded; 0 = healthy."""
    code = ctypes.c_int(0)
    _native.check(_native.lib().fp6b200_device_status(ctypes.byref(code)), "fp6b200_device_status")
    return code.value
