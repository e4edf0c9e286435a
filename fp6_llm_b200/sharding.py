"""Output-channel (column-parallel) sharding of one FPx linear layer across the GPUs of a node.

Rank r owns a contiguous range of output channels, computes Out[:, r0:r1] with the single-GPU kernel and
the ranks exchange their column slabs with ONE all-gather (torch.distributed; NCCL over NVLink on GPUs, gloo
in the CPU tests).  The reference has no multi-GPU code at all; the one thing that comes from it is the packed
layout, which decides how a shard must be cut:

    the packed tensor is [1-bit region][2-bit region][4-bit region] over the WHOLE matrix
    (fp6_llm/csrc/utils/weight_prepacking.h:126-133), and inside a region the bytes of one 64-row block are
    contiguous (8*w*K bytes for the w-bit region).  So prepack(W[r0:r1]) is the concatenation, region by
    region, of bytes [r0/64 * 8wK, r1/64 * 8wK) -- never packed[r0:r1, :].
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from .formats import bit_width, check_format

ROW_UNIT = 256   # the kernel's row constraint (reference: fp6_llm/csrc/fp6_linear.cu:56)


def plan_rows(out_channels: int, world_size: int) -> List[Tuple[int, int]]:
    """[r0, r1) per rank: multiples of 256 rows, as even as possible, earlier ranks take the remainder."""
    if out_channels % ROW_UNIT:
        raise ValueError(f"OC={out_channels} is not a multiple of {ROW_UNIT}")
    units = out_channels // ROW_UNIT
    if world_size < 1 or units < world_size:
        raise ValueError(f"cannot cut {units} row units over {world_size} ranks")
    base, extra = divmod(units, world_size)
    plan, r0 = [], 0
    for r in range(world_size):
        n = (base + (1 if r < extra else 0)) * ROW_UNIT
        plan.append((r0, r0 + n))
        r0 += n
    return plan


def shard_packed(packed: torch.Tensor, in_channels: int, e_bits: int, m_bits: int, r0: int, r1: int) -> torch.Tensor:
    """The prepacked tensor of rows [r0, r1) cut out of the prepacked tensor of the whole matrix."""
    check_format(e_bits, m_bits)
    bw = bit_width(e_bits, m_bits)
    oc = packed.shape[0]
    if r0 % 64 or r1 % 64 or not (0 <= r0 < r1 <= oc):
        raise ValueError("shard rows must be multiples of 64 inside the matrix")
    flat = packed.contiguous().view(torch.uint8).reshape(-1)
    pieces, off = [], 0
    for w in (1, 2, 4):
        if not bw & w:
            continue
        block = 8 * w * in_channels                     # bytes of one 64-row block in this region
        pieces.append(flat[off + (r0 // 64) * block: off + (r1 // 64) * block])
        off += oc * in_channels * w // 8
    out = torch.cat(pieces)
    return out.view(torch.int32).reshape(r1 - r0, in_channels * bw // 32)


def gather_columns(local: torch.Tensor, plan: Sequence[Tuple[int, int]], rank: int, group=None) -> torch.Tensor:
    """All-gather of the per-rank column slabs [B, r1-r0] into the full [B, OC] on every rank.

    One collective on a [world, B, widest] buffer (slabs narrower than the widest are padded), then the slabs
    are laid side by side."""
    import torch.distributed as dist
    world = len(plan)
    batch = local.shape[0]
    widths = [b - a for a, b in plan]
    widest = max(widths)
    if local.shape[1] != widths[rank]:
        raise ValueError("local slab width does not match the plan")
    if widths[rank] == widest:
        send = local.contiguous()
    else:
        send = local.new_zeros((batch, widest))
        send[:, : widths[rank]] = local
    flat = local.new_empty((world * batch, widest))          # rank-major concatenation along dim 0
    dist.all_gather_into_tensor(flat, send, group=group)
    gathered = flat.view(world, batch, widest)
    if all(w == widest for w in widths):
        return gathered.permute(1, 0, 2).reshape(batch, world * widest)
    return torch.cat([gathered[r, :, : widths[r]] for r in range(world)], dim=1)


class ShardedFPxLinear:
    """One rank's part of an OC-sharded FPx linear layer.  `packed_shard`/`scale_shard` live on this rank's GPU."""

    def __init__(self, packed_shard: torch.Tensor, scale_shard: torch.Tensor, plan: Sequence[Tuple[int, int]],
                 rank: int, e_bits: int = 3, m_bits: int = 2, group=None):
        self.packed, self.scale, self.plan, self.rank = packed_shard, scale_shard, list(plan), rank
        self.e_bits, self.m_bits, self.group = e_bits, m_bits, group

    def forward_local(self, x: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        from .ops import linear_forward_eXmY_cuda
        return linear_forward_eXmY_cuda(self.e_bits, self.m_bits, x, self.packed, self.scale, split_k)

    def forward(self, x: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        y = self.forward_local(x, split_k)
        if len(self.plan) == 1:
            return y
        return gather_columns(y, self.plan, self.rank, self.group)
