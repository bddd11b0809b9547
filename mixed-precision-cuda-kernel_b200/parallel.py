"""Column-parallel sharding of a CherryQ quantized linear over the GPUs of one node.

The layer shards along N (output rows): every output element is an independent dot product, so a
rank that holds `qweight[:, n0:n1]`, `scales[:, n0:n1]`, `cherry_weight[:, n0:n1]` and the full
`cherry_indices` computes `y[:, n0:n1]` with exactly the single-GPU arithmetic.  The only
exchange is one all-gather of the (M, N/P) fp16 slices (NCCL over NVLink).  The reference has no
multi-GPU path (its `utils.simple_dispatch_model`, utils.py:28-55, only places whole layers).

Host-side safety net (tested on CPU with gloo): before any GPU work the ranks compare the layer's
metadata (shape, bits, group size, a hash of the cherry list) and fail together if they disagree.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass

import torch
import torch.distributed as dist

ROW_ALIGN = 16      # shards are whole 16-row sub-tiles (and multiples of 8, as the layer requires)


def shard_bounds(n_rows: int, world: int, rank: int, align: int = ROW_ALIGN):
    """[n0, n1) of `rank`: whole `align`-row blocks, as even as possible, the remainder spread over
    the first ranks; the last rank also takes a ragged tail (n_rows need only be a multiple of 8)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    blocks = n_rows // align
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    n0, n1 = b0 * align, b1 * align
    if rank == world - 1:
        n1 = n_rows
    return n0, n1


def shard_buffers(qweight, scales, cherry_weight, cherry_indices, world, rank):
    """This rank's slice of the reference-format buffers (N is their contiguous axis)."""
    n0, n1 = shard_bounds(qweight.shape[1], world, rank)
    return (qweight[:, n0:n1].contiguous(), scales[:, n0:n1].contiguous(),
            cherry_weight[:, n0:n1].contiguous(), cherry_indices.clone())


@dataclass
class ShardMeta:
    bits: int
    group_size: int
    in_features: int
    out_features: int
    num_cherries: int
    cherry_hash: str

    @staticmethod
    def of(bits, group_size, in_features, out_features, cherry_indices) -> "ShardMeta":
        h = hashlib.sha256(cherry_indices.detach().cpu().to(torch.int32).numpy().tobytes()).hexdigest()[:16]
        return ShardMeta(int(bits), int(group_size), int(in_features), int(out_features),
                         int(cherry_indices.numel()), h)


def check_shard_agreement(meta: ShardMeta, group=None):
    """Every rank must describe the same layer.  Raises RuntimeError on ALL ranks when they do not
    (each rank sees the full list, so no rank is left waiting in a later collective)."""
    world = dist.get_world_size(group)
    metas = [None] * world
    dist.all_gather_object(metas, meta, group=group)
    bad = [r for r, m in enumerate(metas) if m != metas[0]]
    if bad:
        raise RuntimeError(f"shard metadata differs on ranks {bad}: {[metas[r] for r in bad]} vs rank 0 {metas[0]}")
    return metas[0]


class ColumnParallelQuantLinear(torch.nn.Module):
    """One rank's shard of a quantized linear plus the all-gather of the outputs.

    `local` is a module (normally `cherryq_b200.qlinear.QuantLinear` built on this rank's slice of
    the buffers) mapping (..., K) -> (..., n1 - n0)."""

    def __init__(self, local: torch.nn.Module, out_features: int, group=None, meta: ShardMeta | None = None):
        super().__init__()
        self.local = local
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.out_features = out_features
        self.bounds = [shard_bounds(out_features, self.world, r) for r in range(self.world)]
        if meta is not None:
            check_shard_agreement(meta, group)

    @torch.inference_mode()
    def forward(self, x):
        y_local = self.local(x)
        sizes = [b - a for a, b in self.bounds]
        width = max(sizes)
        if y_local.shape[-1] != width:           # ragged shards: pad to the widest, gather, cut
            pad = torch.zeros(*y_local.shape[:-1], width, dtype=y_local.dtype, device=y_local.device)
            pad[..., :y_local.shape[-1]] = y_local
        else:
            pad = y_local.contiguous()
        flat = torch.empty(self.world * pad.numel(), dtype=pad.dtype, device=pad.device)
        dist.all_gather_into_tensor(flat, pad.reshape(-1), group=self.group)
        out = flat.view(self.world, *pad.shape)
        return torch.cat([out[r][..., :sizes[r]] for r in range(self.world)], dim=-1)
