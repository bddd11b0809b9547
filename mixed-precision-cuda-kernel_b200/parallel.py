"""Column-parallel sharding of a CherryQ quantized linear over the GPUs of one node.

The layer shards along N (output rows): every output element is an independent dot product, so a
rank that holds `qweight[:, n0:n1]`, `scales[:, n0:n1]`, `cherry_weight[:, n0:n1]` and the full
`cherry_indices` computes `y[:, n0:n1]` with exactly the single-GPU arithmetic.  The only
exchange is one all-gather of the (M, N/P) fp16 slices: `PeerAllGather` (one kernel of this library
over mapped peer memory) or NCCL.  The reference has no
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


class PeerAllGather:
    """All-gather of equal (rows, cols_local) fp16 slices through mapped peer memory: one small
    kernel of this library per call and rank (`cq_peer_allgather`) instead of a library collective.

    Set-up is collective over `group`: every rank creates its region, the 64-byte IPC handles
    travel through `all_gather_object`, every rank maps the others' regions.  If any rank fails to
    map a peer (no peer access between the devices, IPC closed in the container) all ranks raise
    together.  `__call__` enqueues one launch on the current stream and can be captured in a CUDA
    graph; every rank must make the same sequence of calls.  A peer that never delivers shows up
    as a timeout bit in `status` (a device word), read with `check()`; the output of that call is
    then filled with NaN.  One rank per GPU.
    """

    def __init__(self, group, device, capacity_bytes: int = 4 << 20, timeout_ms: int = 2000):
        import ctypes as C

        from . import _cabi
        self._C, self._cabi, self.lib = C, _cabi, _cabi.lib()
        self.group, self.device = group, torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.capacity, self.timeout_ms = int(capacity_bytes) // 16 * 16, int(timeout_ms)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._opened = []
        self.own = None
        with torch.cuda.device(self.device):
            own = C.c_void_p()
            rc = self.lib.cq_peer_region_create(self.capacity, C.byref(own))
            handle = C.create_string_buffer(64)
            if rc == 0:
                self.own = own.value
                rc = self.lib.cq_peer_region_export(own, handle)
            handles = [None] * self.world
            dist.all_gather_object(handles, (rc, handle.raw), group=group)
            ptrs, failed = [], any(h[0] != 0 for h in handles)
            if not failed:
                for r, (_, raw) in enumerate(handles):
                    if r == self.rank:
                        ptrs.append(self.own)
                        continue
                    p = C.c_void_p()
                    rc = self.lib.cq_peer_region_open(raw, C.byref(p))
                    if rc != 0:
                        failed = True
                        break
                    self._opened.append(p.value)
                    ptrs.append(p.value)
            oks = [None] * self.world
            dist.all_gather_object(oks, not failed, group=group)
            if not all(oks):
                self.close()
                raise RuntimeError("peer memory could not be mapped on every rank "
                                   f"(per-rank success: {oks}); use the NCCL all-gather instead")
            self.regions = (C.c_void_p * self.world)(*ptrs)
            self._region_ints = [int(v) for v in ptrs]
        dist.barrier(group=group)          # every region is zeroed and mapped before the first launch

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 2:
            raise ValueError("x must be a (rows, cols_local) fp16 CUDA tensor")
        out = torch.empty(x.shape[0], self.world * x.shape[1], dtype=torch.float16, device=x.device)
        return self.gather_into(x, out)

    gather = __call__

    def gather_into(self, x: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
        """out (rows, world * cols_local) <- the slices x (rows, cols_local) of all ranks, in rank order."""
        if x.dim() != 2 or x.dtype != torch.float16 or not x.is_cuda or not x.is_contiguous():
            raise ValueError("x must be a contiguous (rows, cols_local) fp16 CUDA tensor")
        rows, cols = x.shape
        if out.dtype != torch.float16 or not out.is_contiguous() or out.numel() != rows * cols * self.world:
            raise ValueError("out must be a contiguous fp16 tensor of rows * world * cols_local elements")
        stream = stream if stream is not None else torch.cuda.current_stream(x.device)
        cv = self._C.c_void_p
        self._cabi.check(self.lib.cq_peer_allgather(self.regions, self.world, self.rank, self.capacity,
                                                    cv(x.data_ptr()), cv(out.data_ptr()), rows, cols, self.timeout_ms,
                                                    cv(self.status.data_ptr()), cv(stream.cuda_stream)), "peer all-gather")
        return out

    def matvec_gather(self, row_layer, x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        """This rank's shard of a layer (a `quant_cuda.RowLayer`) applied to x (rows <= 4, K) AND the exchange of
        the ranks' output slices, in one launch: returns (rows, world * N_local).  Counts as one call of the
        exchange sequence (every rank makes the same calls in the same order)."""
        rows, n = x.shape[0], row_layer.out_features
        y_local = torch.empty(rows, n, dtype=torch.float16, device=x.device)
        if out is None:
            out = torch.empty(rows, self.world * n, dtype=torch.float16, device=x.device)
        row_layer.matvec_gather(x, y_local, out, self._region_ints, self.rank,
                                self.capacity, self.timeout_ms, self.status)
        return out

    # The exchange is one CTA per rank: made for the latency of decode-sized slices.  Beyond this many bytes per
    # rank a bandwidth-oriented collective (NCCL) is the better tool (measured: 32 x 3584 fp16 per rank on 8 GPUs
    # took about 100 us here).
    MAX_SLICE_BYTES = 64 * 1024

    def fits(self, rows: int, cols_local: int) -> bool:
        return (cols_local % 8 == 0 and rows * cols_local * 2 <= self.MAX_SLICE_BYTES
                and rows * cols_local * 4 * self.world <= self.capacity)    # twice the payload on the wire

    def check(self) -> None:
        """Host read of the status word (synchronises): raises if a wait for a peer ran out."""
        if int(self.status.item()) != 0:
            self.status.zero_()
            raise RuntimeError("a peer did not deliver its slice within the time limit")

    def close(self) -> None:
        """Unmap the peers' regions and free the own one.  Call on every rank, with no gather in flight."""
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.lib.cq_peer_region_close(self._C.c_void_p(p))
            self._opened = []
            if dist.is_initialized():
                try:
                    dist.barrier(group=self.group)     # nobody still has a peer's region mapped
                except Exception:
                    pass
            if self.own is not None:
                self.lib.cq_peer_region_destroy(self._C.c_void_p(self.own))
                self.own = None
