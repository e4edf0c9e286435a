"""Output-channel (column-parallel) sharding of one FPx linear layer across the GPUs of a node.

Rank r owns a contiguous range of output channels and computes Out[:, r0:r1] with the single-GPU kernel.  The
column slabs reach the other ranks in one of two ways:

  * fused (PeerExchange): the kernel's epilogue stores every finished tile straight into the output buffer of
    EVERY rank (peer-mapped symmetric memory, plain stores over NVLink) and a one-warp kernel ends the layer with
    an arrival barrier between the GPUs.  No separate collective, no staging copy.
  * ONE all-gather (torch.distributed; NCCL over NVLink on GPUs, gloo in the CPU tests) of the per-rank slabs.

The reference has no multi-GPU code at all; the one thing that comes from it is the packed
layout, which decides how a shard must be cut:

    the packed tensor is [1-bit region][2-bit region][4-bit region] over the WHOLE matrix
    (fp6_llm/csrc/utils/weight_prepacking.h:126-133), and inside a region the bytes of one 64-row block are
    contiguous (8*w*K bytes for the w-bit region).  So prepack(W[r0:r1]) is the concatenation, region by
    region, of bytes [r0/64 * 8wK, r1/64 * 8wK) -- never packed[r0:r1, :].
"""
from __future__ import annotations

import ctypes
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


class PeerExchange:
    """What the ranks of one process group share for the fused exchange: a flag word per pair of ranks, this rank's
    call counter, and three rotating output buffers per (batch, out_channels) shape, all but the counter in symmetric
    memory (torch.distributed._symmetric_memory: every rank's allocation is mapped into every process).

    Lifetime of a result.  Every call ends with the arrival barrier, so a rank runs at most one call ahead of a peer,
    and a peer stores into a buffer as soon as it starts the call that uses it.  With three buffers per shape the
    tensor returned by call k is overwritten by call k+3 of that shape, which a peer may start once THIS rank has
    issued call k+2: a result is safe while this rank issues one more call of the shape (h1 = L1(x); h2 = L2(h1);
    y = h1 + h2 is fine), and must be consumed or copied, in stream order, before the second next one is issued.

    CUDA graphs.  The buffer is chosen on the host when the call is made, so a captured graph always uses the buffers
    it was captured with: capture a multiple of three calls per shape, or make sure that in every replay order two
    calls that share a buffer are at least three layer calls (of any shape: each ends with the barrier) apart.

    Multicast is switched off for the symmetric allocations (the kernels use plain peer stores only): call close()
    - after a barrier between the ranks - before the process group is destroyed."""

    MAX_WORLD = 8
    BUFFERS = 3

    def __init__(self, group=None):
        import os
        import torch.distributed as dist
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # before the first rendezvous of the process
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > self.MAX_WORLD:
            raise ValueError(f"the fused exchange handles at most {self.MAX_WORLD} ranks")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._symm = symm
        self.flags = symm.empty(64, dtype=torch.int32, device=self.device)
        self._flags_handle = symm.rendezvous(self.flags, self.group)
        self.flags.zero_()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)          # nobody signals before every rank has cleared its flags
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in self._flags_handle.buffer_ptrs])
        self._buffers = {}

    def close(self) -> None:
        """Drops the exchange buffers and their peer mappings.  Collective in spirit: every rank must have finished its
        calls (synchronise, then a barrier between the ranks) before any rank closes."""
        torch.cuda.synchronize(self.device)
        self._buffers = {}
        self._flag_ptrs = None
        self._flags_handle = None
        self.flags = None

    def _next_buffer(self, batch: int, out_channels: int):
        key = (batch, out_channels)
        slot = self._buffers.get(key)
        if slot is None:
            ring = []
            for _ in range(self.BUFFERS):
                t = self._symm.empty((batch, out_channels), dtype=torch.float16, device=self.device)
                h = self._symm.rendezvous(t, self.group)
                ring.append((t, h, (ctypes.c_void_p * self.world)(*[int(p) for p in h.buffer_ptrs])))
            slot = {"ring": ring, "next": 0}
            self._buffers[key] = slot
        entry = slot["ring"][slot["next"]]
        slot["next"] = (slot["next"] + 1) % self.BUFFERS
        return entry

    def reserve(self, batch: int, out_channels: int) -> None:
        """Creates the output buffers of a shape now (a collective call: every rank, same order)."""
        key = (batch, out_channels)
        if key not in self._buffers:
            self._next_buffer(batch, out_channels)
            self._buffers[key]["next"] = 0

    def linear(self, layer: "ShardedFPxLinear", x: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        """The whole [B, OC] result of the sharded layer on this rank (a view of an exchange buffer)."""
        from . import _native
        from .ops import _ptr, _stream_ptr, _workspace
        if split_k not in (0, 1):
            raise ValueError("the fused exchange takes split_k 0 or 1")
        if x.dtype != torch.float16 or not x.is_cuda or x.dim() != 2 or not x.is_contiguous():
            raise ValueError("activations must be a contiguous fp16 CUDA tensor [B, IC]")
        if len(layer.plan) != self.world or layer.rank != self.rank:
            raise ValueError("the layer's plan does not match this process group")
        batch, ic = x.shape
        r0, r1 = layer.plan[self.rank]
        oc = layer.plan[-1][1]
        if layer.packed.shape[0] != r1 - r0 or layer.packed.shape[1] * 32 != ic * bit_width(layer.e_bits, layer.m_bits):
            raise ValueError("packed shard does not match the plan or the activations")
        out, _handle, out_ptrs = self._next_buffer(batch, oc)
        L = _native.lib()
        with torch.cuda.device(self.device):
            if layer.use_native(batch, split_k):
                ws = _workspace(self.device, L.fp6b200_native_workspace_bytes(batch, ic))
                rc = L.fp6b200_linear_native_gather(layer.e_bits, layer.m_bits, _stream_ptr(self.device), _ptr(layer.native),
                                                    _ptr(layer.scale), _ptr(x), out_ptrs, self._flag_ptrs, _ptr(self.epoch),
                                                    self.world, self.rank, oc, r0, r1 - r0, batch, ic, _ptr(ws))
            else:
                nbytes = L.fp6b200_workspace_bytes(r1 - r0, batch, ic, split_k)
                ws = _workspace(self.device, nbytes) if nbytes else None
                rc = L.fp6b200_linear_gather(layer.e_bits, layer.m_bits, _stream_ptr(self.device), _ptr(layer.packed),
                                             _ptr(layer.scale), _ptr(x), out_ptrs, self._flag_ptrs, _ptr(self.epoch),
                                             self.world, self.rank, oc, r0, r1 - r0, batch, ic,
                                             _ptr(ws) if ws is not None else None, split_k)
        _native.check(rc, "fp6b200_linear_gather")
        return out


class ShardedFPxLinear:
    """One rank's part of an OC-sharded FPx linear layer.  `packed_shard`/`scale_shard` live on this rank's GPU.
    With `exchange` (a PeerExchange) the slabs are exchanged by the kernel itself, otherwise by one all-gather."""

    def __init__(self, packed_shard: torch.Tensor, scale_shard: torch.Tensor, plan: Sequence[Tuple[int, int]],
                 rank: int, e_bits: int = 3, m_bits: int = 2, group=None, exchange: "PeerExchange | None" = None,
                 native: bool = False):
        self.packed, self.scale, self.plan, self.rank = packed_shard, scale_shard, list(plan), rank
        self.e_bits, self.m_bits, self.group, self.exchange = e_bits, m_bits, group, exchange
        # native=True: the shard is also kept in the tile layout of the tensor cores' own six-bit inputs, and the batches for
        # which ops.native_preferred says so run there
        self.native = None
        if native:
            from .ops import native_repack, native_supported
            ic = packed_shard.shape[1] * 32 // bit_width(e_bits, m_bits)
            if native_supported(e_bits, m_bits, packed_shard.shape[0], ic, 1):
                self.native = native_repack(e_bits, m_bits, packed_shard)

    def use_native(self, batch: int, split_k: int) -> bool:
        from .ops import native_preferred
        if self.native is None or split_k != 0:
            return False
        ic = self.packed.shape[1] * 32 // bit_width(self.e_bits, self.m_bits)
        return native_preferred(self.e_bits, self.m_bits, self.packed.shape[0], ic, batch)

    def forward_local(self, x: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        from .ops import linear_forward_eXmY_cuda, linear_forward_native
        if self.use_native(x.shape[0], split_k):
            return linear_forward_native(self.e_bits, self.m_bits, x, self.native, self.scale)
        return linear_forward_eXmY_cuda(self.e_bits, self.m_bits, x, self.packed, self.scale, split_k)

    def forward(self, x: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        if len(self.plan) == 1:
            return self.forward_local(x, split_k)
        if self.exchange is not None:
            return self.exchange.linear(self, x, split_k)
        return gather_columns(self.forward_local(x, split_k), self.plan, self.rank, self.group)


# ------------------------------------------------------------------------------------------------ IC-sharded (row-parallel)
COL_UNIT = 64   # the kernel's K granularity (reference: fp6_llm/csrc/fp6_linear.cu:57)


def plan_cols(in_channels: int, world_size: int) -> List[Tuple[int, int]]:
    """[k0, k1) per rank: multiples of 64 input channels, as even as possible, earlier ranks take the remainder."""
    if in_channels % COL_UNIT:
        raise ValueError(f"IC={in_channels} is not a multiple of {COL_UNIT}")
    units = in_channels // COL_UNIT
    if world_size < 1 or units < world_size:
        raise ValueError(f"cannot cut {units} column units over {world_size} ranks")
    base, extra = divmod(units, world_size)
    plan, k0 = [], 0
    for r in range(world_size):
        n = (base + (1 if r < extra else 0)) * COL_UNIT
        plan.append((k0, k0 + n))
        k0 += n
    return plan


def slice_unpacked_cols(w_unpacked: torch.Tensor, e_bits: int, m_bits: int, k0: int, k1: int) -> torch.Tensor:
    """Input channels [k0, k1) of the UNPACKED int32 [OC, IC*bw/32] tensor (64 codes are 2*bw whole words, so a multiple
    of 64 columns is a plain column slice); prepack the result to get the rank's weights.  The packed tensor cannot be
    cut along K by slicing: every region interleaves the K blocks of a 64-row block."""
    check_format(e_bits, m_bits)
    bw = bit_width(e_bits, m_bits)
    if k0 % COL_UNIT or k1 % COL_UNIT or not (0 <= k0 < k1 <= w_unpacked.shape[1] * 32 // bw):
        raise ValueError("column shards must be multiples of 64 inside the matrix")
    return w_unpacked[:, k0 * bw // 32: k1 * bw // 32].contiguous()


def reduce_partials(partial: torch.Tensor, mode: str = "all_reduce", group=None) -> torch.Tensor:
    """Sums the ranks' [B, OC] partial results.  "all_reduce": every rank gets the whole [B, OC].  "reduce_scatter": rank r
    gets output channels [r*OC/world, (r+1)*OC/world) as [B, OC/world] (what a following column-parallel layer, or a
    sequence-parallel region, consumes).  One collective either way; the sum is taken in the tensor's dtype (fp16), as
    tensor-parallel inference engines do."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if mode == "all_reduce":
        out = partial.contiguous()
        dist.all_reduce(out, group=group)
        return out
    if mode != "reduce_scatter":
        raise ValueError("mode must be all_reduce or reduce_scatter")
    batch, oc = partial.shape
    if oc % world:
        raise ValueError("OC must divide by the number of ranks for reduce_scatter")
    send = partial.view(batch, world, oc // world).permute(1, 0, 2).contiguous()     # [world, B, OC/world]
    out = partial.new_empty((batch, oc // world))
    try:
        dist.reduce_scatter_tensor(out, send, group=group)
    except (RuntimeError, NotImplementedError):   # a backend without reduce-scatter (gloo): all-reduce, keep the own slab
        dist.all_reduce(send, group=group)
        out = send[dist.get_rank(group)].contiguous()
    return out


class RowParallelFPxLinear:
    """One rank's part of an IC-sharded (row-parallel) FPx linear layer, the form the O and down projections take behind
    a column-parallel layer: the rank holds the prepacked weights of its input channels [k0, k1) for ALL output channels
    and receives the matching activation columns; the partial results are summed over the ranks by one collective.
    The bias, if any, is added by rank 0 only (inside its kernel), so the sum carries it once."""

    def __init__(self, packed_cols: torch.Tensor, scale: torch.Tensor, plan: Sequence[Tuple[int, int]], rank: int,
                 e_bits: int = 3, m_bits: int = 2, bias: "torch.Tensor | None" = None, group=None, mode: str = "all_reduce"):
        self.packed, self.scale, self.plan, self.rank = packed_cols, scale, list(plan), rank
        self.e_bits, self.m_bits, self.group, self.mode = e_bits, m_bits, group, mode
        self.bias = bias if rank == 0 else None
        k0, k1 = self.plan[rank]
        if packed_cols.shape[1] * 32 != (k1 - k0) * bit_width(e_bits, m_bits):
            raise ValueError("packed shard does not match the column plan")

    def forward_local(self, x_cols: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        from .ops import ACT_NONE, linear_forward_ex
        return linear_forward_ex(self.e_bits, self.m_bits, x_cols, self.packed, self.scale, split_k, self.bias, ACT_NONE)

    def forward(self, x_cols: torch.Tensor, split_k: int = 0) -> torch.Tensor:
        """x_cols: this rank's activation columns [B, k1-k0] (the output slab of the column-parallel layer before it)."""
        local = self.forward_local(x_cols, split_k)
        if len(self.plan) == 1:
            return local
        return reduce_partials(local, self.mode, self.group)
