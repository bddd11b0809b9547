"""Host-side logic of the column-parallel path, on CPU with gloo (world_size 2)."""
import datetime
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_bounds_cover_rows_exactly():
    from cherryq_b200.parallel import shard_bounds
    for n in (8, 16, 40, 1024, 4096, 11008, 4744, 28672):
        for world in (1, 2, 4, 8):
            b = [shard_bounds(n, world, r) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == n
            for (a0, a1), (b0, b1) in zip(b, b[1:]):
                assert a1 == b0
            for a0, a1 in b[:-1]:
                assert a0 % 16 == 0 and a1 % 16 == 0
            assert all((a1 - a0) % 8 == 0 for a0, a1 in b)


def _worker(rank, world, port, mode, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from conftest import load_golden
        from cherryq_b200.parallel import (ColumnParallelQuantLinear, ShardMeta, check_shard_agreement,
                                           shard_bounds, shard_buffers)
        from oracle import cherryq_oracle as O
        g = load_golden("k256_n40_b3_g64_f16")
        bufs = [torch.from_numpy(g[k]) for k in ("qweight", "scales", "cherry_weight", "cherry_indices")]
        if mode == "forward":
            qs, ss, cs, idx = shard_buffers(*bufs, world, rank)
            n0, n1 = shard_bounds(g["N"], world, rank)
            dense = O.unpack(qs.numpy(), ss.numpy(), cs.numpy(), idx.numpy(), g["bits"], g["G"], g["K"])

            class Local(torch.nn.Module):          # CPU stand-in for the rank's GPU layer
                def forward(self, x):
                    return torch.from_numpy(O.forward_dense_fp64(x.numpy(), dense)).to(torch.float16)

            meta = ShardMeta.of(g["bits"], g["G"], g["K"], g["N"], idx)
            layer = ColumnParallelQuantLinear(Local(), g["N"], meta=meta)
            y = layer(torch.from_numpy(g["x"]))
            ref = g["y"].astype(np.float64)
            err = float(np.abs(y.numpy().astype(np.float64) - ref).max() / np.abs(ref).max())
            # the slices of the full-layer oracle, reassembled, equal the sharded computation
            full = O.unpack(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["G"], g["K"])
            same = bool(np.array_equal(full[n0:n1], dense))
            q.put((rank, "ok", err, same, tuple(y.shape)))
        elif mode == "mismatch":
            idx = bufs[3].clone()
            if rank == 1:
                idx[0] += 1                     # one rank holds a different cherry list
            try:
                check_shard_agreement(ShardMeta.of(g["bits"], g["G"], g["K"], g["N"], idx))
                q.put((rank, "no-error"))
            except RuntimeError as e:
                q.put((rank, "raised", "differs" in str(e)))
        elif mode == "absent":
            # rank 1 never joins the check: rank 0 must get an error from the timeout, not hang
            if rank == 0:
                try:
                    pg = dist.new_group(timeout=datetime.timedelta(seconds=3))
                    check_shard_agreement(ShardMeta.of(g["bits"], g["G"], g["K"], g["N"], bufs[3]), group=pg)
                    q.put((rank, "no-error"))
                except Exception as e:
                    q.put((rank, "raised", type(e).__name__))
            else:
                dist.new_group(timeout=datetime.timedelta(seconds=3))
                q.put((rank, "skipped"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(mode, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return sorted(out)


def test_column_parallel_forward_matches_full_layer():
    out = _run("forward")
    for rank, status, err, same, shape in out:
        assert status == "ok" and same
        assert shape == (5, 40)
        assert err <= 2e-3


def test_metadata_mismatch_raises_on_every_rank():
    out = _run("mismatch")
    assert all(o[1] == "raised" and o[2] for o in out), out


def test_absent_rank_times_out_instead_of_hanging():
    out = _run("absent")
    r0 = [o for o in out if o[0] == 0][0]
    assert r0[1] == "raised", out
