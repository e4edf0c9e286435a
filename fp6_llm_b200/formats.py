"""FPx number formats and the unpacked weight stream.

FPx code = [sign | E exponent bits | M mantissa bits], no inf/NaN.  The reference dequantises a code by
moving it into fp16 bit positions (sign kept, the rest shifted right by 5-E) and multiplying by
2^(16 - 2^(E-1)) (fp6_llm/csrc/utils/weight_dequant.h:30-43), so e3m2 covers 0..28 and e2m2 covers 0..7.
The reference dispatches e3m2 and e2m2; its templates are generic, and this library also takes e2m1 (4-bit, 0..6),
e3m1 (5-bit, 0..24) and e2m3 (6-bit, 0..7.5).

The *unpacked* weight tensor of the reference is int32 [OC, IC*bw/32]; viewed as bytes each row is an
MSB-first stream of bw-bit codes (fp6_llm/csrc/utils/common.h:9-17, fp6_llm/csrc/utils/weight_quant.h:74-76).

Everything here is tensor plumbing for building inputs (synthetic weights, quantisation to codes,
bit-stream packing); it works on CPU or CUDA tensors and is not on the timed path.
"""
from __future__ import annotations

import torch

SUPPORTED = ((3, 2), (2, 2), (2, 1), (3, 1), (2, 3))


def bit_width(e_bits: int, m_bits: int) -> int:
    return 1 + e_bits + m_bits


def check_format(e_bits: int, m_bits: int) -> None:
    if (e_bits, m_bits) not in SUPPORTED:
        raise ValueError(f"unsupported FPx format e{e_bits}m{m_bits}; supported: e3m2, e2m2, e2m1, e3m1, e2m3")


def magnitudes(e_bits: int, m_bits: int) -> torch.Tensor:
    """Values of the non-negative codes 0 .. 2^(E+M)-1 at scale 1, as float32."""
    check_format(e_bits, m_bits)
    n = 1 << (e_bits + m_bits)
    code = torch.arange(n, dtype=torch.int32)
    h = (code << (10 - m_bits)).to(torch.int16)          # exponent+mantissa in fp16 bit positions
    val = h.view(torch.float16).to(torch.float32)
    return val * float(1 << (16 - (1 << (e_bits - 1))))


def code_values(e_bits: int, m_bits: int) -> torch.Tensor:
    """Value of every code 0 .. 2^bw-1 (the upper half are the negatives; code 2^(bw-1) is -0)."""
    mag = magnitudes(e_bits, m_bits)
    return torch.cat([mag, -mag])


def quantize_rtn(w: torch.Tensor, scale: torch.Tensor, e_bits: int, m_bits: int) -> torch.Tensor:
    """Round-to-nearest FPx codes (uint8 [OC, IC]) of w / scale[:, None]; ties go to the even code,
    magnitudes beyond the largest value saturate.  The reference ships no such quantiser (its
    fp6_llm/csrc/utils/weight_quant.h truncates and is not exposed); inputs for benchmarks need one."""
    mag = magnitudes(e_bits, m_bits).to(w.device)
    q = w.to(torch.float32) / scale.to(torch.float32)[:, None]
    a = q.abs()
    mid = (mag[:-1] + mag[1:]) * 0.5
    lo = torch.bucketize(a, mid, right=False)            # tie -> lower code
    hi = torch.bucketize(a, mid, right=True)             # tie -> upper code
    idx = torch.where(lo % 2 == 0, lo, hi)               # they differ only on exact ties
    sign = (torch.signbit(q)).to(torch.int64) << (e_bits + m_bits)
    return (idx + sign).to(torch.uint8)


def pack_codes(codes: torch.Tensor, e_bits: int, m_bits: int) -> torch.Tensor:
    """uint8 codes [OC, IC] -> unpacked int32 [OC, IC*bw/32] (MSB-first bit stream per row)."""
    check_format(e_bits, m_bits)
    bw = bit_width(e_bits, m_bits)
    oc, ic = codes.shape
    if ic % 32:
        raise ValueError("IC must be a multiple of 32")
    g = codes.reshape(oc, ic // 8, 8).to(torch.int64)
    word = torch.zeros(oc, ic // 8, dtype=torch.int64, device=codes.device)
    for i in range(8):                                    # 8 codes -> bw bytes
        word |= g[:, :, i] << (bw * (7 - i))
    out = torch.empty(oc, ic // 8, bw, dtype=torch.uint8, device=codes.device)
    for b in range(bw):
        out[:, :, b] = ((word >> (8 * (bw - 1 - b))) & 0xFF).to(torch.uint8)
    return out.reshape(oc, ic * bw // 8).view(torch.int32)


def unpack_codes(w_unpacked: torch.Tensor, e_bits: int, m_bits: int) -> torch.Tensor:
    """Inverse of pack_codes: int32 [OC, IC*bw/32] -> uint8 codes [OC, IC]."""
    check_format(e_bits, m_bits)
    bw = bit_width(e_bits, m_bits)
    oc = w_unpacked.shape[0]
    by = w_unpacked.contiguous().view(torch.uint8).reshape(oc, -1, bw).to(torch.int64)
    word = torch.zeros(by.shape[:2], dtype=torch.int64, device=w_unpacked.device)
    for b in range(bw):
        word |= by[:, :, b] << (8 * (bw - 1 - b))
    codes = torch.stack([(word >> (bw * (7 - i))) & ((1 << bw) - 1) for i in range(8)], dim=-1)
    return codes.reshape(oc, -1).to(torch.uint8)


def synth_layer(oc: int, ic: int, e_bits: int, m_bits: int, seed: int, device="cpu", std: float = 0.02):
    """Seeded stand-in for a checkpoint layer: fp16 N(0, std) weights, per-row scale max|w| / (28 for e3m2,
    7.5 for e2m2, the largest magnitude for the other formats), round-to-nearest codes.  Returns (unpacked int32 [OC, IC*bw/32], scale fp16 [OC])."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    w = (torch.randn(oc, ic, generator=gen, device=device, dtype=torch.float32) * std).to(torch.float16)
    # the row maximum lands on the largest magnitude; e2m2 keeps the 7.5 the benchmark configuration names (it saturates to 7)
    denom = 7.5 if (e_bits, m_bits) == (2, 2) else float(magnitudes(e_bits, m_bits)[-1])
    scale = (w.abs().amax(dim=1).to(torch.float32) / denom).to(torch.float16)
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    codes = quantize_rtn(w, scale, e_bits, m_bits)
    return pack_codes(codes, e_bits, m_bits), scale


def random_codes_layer(oc: int, ic: int, e_bits: int, m_bits: int, seed: int, device="cpu",
                       scale_lo: float = 1e-3, scale_hi: float = 1e-2):
    """Uniformly random codes and U(scale_lo, scale_hi) fp16 row scales."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    bw = bit_width(e_bits, m_bits)
    codes = torch.randint(0, 1 << bw, (oc, ic), generator=gen, device=device, dtype=torch.int32).to(torch.uint8)
    scale = (torch.rand(oc, generator=gen, device=device) * (scale_hi - scale_lo) + scale_lo).to(torch.float16)
    return pack_codes(codes, e_bits, m_bits), scale
