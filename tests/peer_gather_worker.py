"""Worker of tests/test_gpu_peer_gather.py: one rank (one GPU) of a two-rank exchange.  Compares the
peer-memory all-gather kernel with NCCL's all-gather on the same slices: single calls of several
shapes, a burst of back-to-back calls (landing areas re-used), and replays of a CUDA graph."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def nccl_gather(x, world):
    t, nl = x.shape
    out = torch.empty(world, t, nl, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous())
    return out.permute(1, 0, 2).reshape(t, world * nl)


def main():
    out_path = sys.argv[1]
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    world, rank = dist.get_world_size(), dist.get_rank()
    from cherryq_b200.parallel import PeerAllGather
    peer = PeerAllGather(dist.group.WORLD, dev, capacity_bytes=1 << 20, timeout_ms=5000)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    ok = True
    for rows, cols in [(1, 1376), (1, 8), (4, 2048), (16, 5504), (3, 24), (1, 1376)]:
        x = torch.randn(rows, cols, device=dev, generator=g).half()
        ok &= torch.equal(peer(x), nccl_gather(x, world))
    # back-to-back calls without host synchronisation
    xs = [torch.randn(2, 512, device=dev, generator=g).half() for _ in range(64)]
    got = [peer(x) for x in xs]
    want = [nccl_gather(x, world) for x in xs]
    ok &= all(torch.equal(a, b) for a, b in zip(got, want))
    # inside a CUDA graph: the same graph replayed with changing inputs
    x = torch.zeros(1, 1376, dtype=torch.float16, device=dev)
    out = torch.zeros(1, world * 1376, dtype=torch.float16, device=dev)
    s = torch.cuda.Stream(device=dev)
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        peer.gather_into(x, out, s)
        s.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            for _ in range(3):
                peer.gather_into(x, out, s)
        for i in range(20):
            x.copy_(torch.randn(1, 1376, device=dev, generator=g).half())
            graph.replay()
            s.synchronize()
            ok &= torch.equal(out, nccl_gather(x, world))
    # the matvec that ends with the exchange (one launch) against matvec + NCCL, mixed with plain exchanges
    import math
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    for K, N, bits in [(4096, 1376, 4), (11008, 512, 3), (2048, 40, 4)]:
        gw = torch.Generator(device=dev).manual_seed(7)            # same full layer on every rank
        c = math.ceil(K / 256) // 8 * 8
        w = (torch.randn(N * world, K, device=dev, generator=gw) * 0.02).half()
        idx = torch.randperm(K, device=dev, generator=gw)[:c].to(torch.int32)
        q, sc, cw, ci = qc.pack(w[rank * N:(rank + 1) * N].contiguous(), idx.contiguous(), bits, 128)
        row = qc.RowLayer(q, sc, cw, ci, bits, K, 128)
        for rows in (1, 3, 4):
            xa = torch.randn(rows, K, device=dev, generator=gw).half()   # the same activations on every rank
            y = torch.empty(rows, N, dtype=torch.float16, device=dev)
            row.matvec(xa, y, False)
            want_all = nccl_gather(y, world)
            for _ in range(3):
                ok &= torch.equal(peer.matvec_gather(row, xa), want_all)
                ok &= torch.equal(peer(y), want_all)                      # a plain exchange in between
    peer.check()
    peer.close()                      # collective: unmap the peers, meet, free the own region
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    if rank == 0:
        with open(out_path, "w") as f:
            f.write("ok" if int(flag.item()) == 1 else "mismatch")
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
