"""Batch x head partition of one attention call over the GPUs of a node.

Every kernel of the path is indexed by the flattened (batch, head) unit and no term crosses units,
so the call shards with no collective on the data path (the reference indexes everything by `bh`:
kernels/hip/sk1_t6i.hip:82, kernels/hip/h34_prologue.hip:108-110).  One process per GPU; each rank
runs prologue + attention on its contiguous range of units.  A collective (all-gather over
NCCL/NVLink) is used only when the caller asks for the whole output on every rank.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def partition_units(n_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, stop) range of flattened (batch, head) units for `rank`; the first
    `n_units % world_size` ranks take one extra unit."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("bad world_size/rank")
    base, extra = divmod(int(n_units), world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def _flatten_units(t: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    """(B,H,N,D) or (B,N,H,D) -> a logical (1, B*H, N, D) view without copying when possible."""
    if tensor_layout == "NHD":
        t = t.transpose(1, 2)
    b, h, n, d = t.shape
    return t.reshape(1, b * h, n, d)


def sageattn_sharded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, is_causal: bool = False,
                     sm_scale: Optional[float] = None, smooth_k: bool = True,
                     group: Optional[dist.ProcessGroup] = None, gather: bool = False,
                     attn_fn: Optional[Callable] = None) -> torch.Tensor:
    """Attention over this rank's units.  `q, k, v` are this rank's shard, shaped
    (1, units, N, 128) in HND layout (use `partition_units` to slice a replicated tensor).  With
    `gather=False` (the hot path) the local output is returned and nothing is communicated; with
    `gather=True` the outputs of all ranks are all-gathered along the unit axis and every rank
    returns (1, total_units, N, 128).  `attn_fn` defaults to `sageattn`.

    With grouped-query heads, partition the key/value units and give each rank the matching
    `g = Hq / Hkv` times as many query units: q is (1, g*units, Nq, D), k and v are
    (1, units, Nk, D); query unit u reads key/value unit u // g, so a contiguous range of
    key/value units [a, b) goes with the query range [g*a, g*b)."""
    if attn_fn is None:
        from .core import sageattn as attn_fn
    out = attn_fn(q, k, v, tensor_layout="HND", is_causal=is_causal, sm_scale=sm_scale,
                  smooth_k=smooth_k)
    if not gather:
        return out
    return gather_units(out, group=group)


def gather_units(out_local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather per-rank outputs (1, units_r, N, D) along the unit axis.  Ranks may hold
    different unit counts (when world_size does not divide B*H): shards are padded to the largest
    count for the collective and trimmed afterwards."""
    if not (dist.is_available() and dist.is_initialized()):
        return out_local
    world = dist.get_world_size(group)
    if world == 1:
        return out_local
    units = torch.tensor([out_local.shape[1]], dtype=torch.int64, device=out_local.device)
    all_units = [torch.zeros_like(units) for _ in range(world)]
    dist.all_gather(all_units, units, group=group)
    counts = [int(u.item()) for u in all_units]
    umax = max(counts)
    _, _, n, d = out_local.shape
    send = out_local
    if out_local.shape[1] != umax:
        send = out_local.new_zeros((1, umax, n, d))
        send[:, : out_local.shape[1]] = out_local
    buf = out_local.new_empty((world * umax, n, d))
    dist.all_gather_into_tensor(buf, send.reshape(umax, n, d).contiguous(), group=group)
    buf = buf.view(world, umax, n, d)
    parts = [buf[r, : counts[r]] for r in range(world)]
    return torch.cat(parts, dim=0).unsqueeze(0)
