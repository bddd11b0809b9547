#!/usr/bin/env python
"""Benchmark of the CherryQ quantized-linear hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the layer the headline target is quoted on): one
LLaMA-7B gate/up projection, 4096 -> 11008, 4-bit, group 128, cherry ratio 1/256 (16 fp16
columns), fp16 activations ~N(0,1), batch 1.  Weights are synthetic with the configuration's
distributions (dense ~N(0, 0.02), cherry columns ~N(0, 0.2)), quantised and packed by the GPU
pack kernel.  A "step" is one matvec of that layer.  To keep the 23.5 MB layer from living in
the 126 MB L2, consecutive steps walk over enough distinct copies of the layer to exceed 3x L2.

metric  : algorithmic bytes of the reference format (qweight + scales + cherry values + indices
          + x + y) per second, in GB/s - the number the HBM roofline is judged against.
value   : inputs resident in HBM, the one-row decode kernel through the C ABI (cq_rlayer_matvec), every launch
          of the timed region a CUDA-graph node; the region is timed --repeats times, the median is reported.
e2e     : the same metric with HOST buffers, one synchronous call per step: x comes from pinned host memory and
          y is complete in pinned host memory when the call returns.  At N = 1 through the C ABI's
          cq_rlayer_matvec_host; the record also holds the same through the drop-in torch op
          `quant_cuda.vecquant4matmul_cherryq` (copy x in, zero-fill the output because the operator
          accumulates as the reference's does, run the op, read y back), which is the path at N > 1.
N > 1   : the layer is sharded column-parallel (N/P output rows per GPU), every rank runs its
          shard and the slices are exchanged (peer-memory kernel, or NCCL): strong scaling of one layer.
          Rank 0 checks the gathered vector bit for bit against the unsharded layer before timing.
model_70b : LLaMA-2-70B-architecture 3-bit greedy decode on the same GPUs, tokens/s (every N).
--impl reference : the reference's CPU path (unpack to dense fp16 + F.linear per call, restated
          in oracle/torch_port.py because the Python reference does not travel) on the host cores.
"""
import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K_IN, N_OUT, BITS, GROUP = 4096, 11008, 4, 128
WORKLOAD = "llama7b_gate_proj_4096x11008_4bit_g128_cherry1/256_batch1"
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(k, n, bits, group, m, c):
    kc = k - c
    return kc // 8 * bits * n + math.ceil(kc / group) * n * 2 + c * n * 2 + c * 2 + m * k * 2 + m * n * 2


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[1]) for r in self.rows if len(r) > 2 and r[1].isdigit())
        mx = [int(r[2]) for r in self.rows if len(r) > 2 and r[2].isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_layer_gpu(qc, torch, k, n, bits, group, seed, device):
    """Synthetic layer with the configuration's distributions, packed on the GPU."""
    g = torch.Generator(device=device).manual_seed(seed)
    c = math.ceil(k / 256) // 8 * 8
    w = torch.randn(n, k, device=device, generator=g) * 0.02
    idx = torch.randperm(k, device=device, generator=g)[:c].to(torch.int32)
    w[:, idx.long()] = torch.randn(n, c, device=device, generator=g) * 0.2
    q, s, cw, ci = qc.pack(w.half().contiguous(), idx.contiguous(), bits, group)
    return q, s, cw, ci, c


def reference_inputs(torch):
    """Buffers of the reference format with the workload's shapes (the CPU path's cost does not depend on the values)."""
    from oracle import cherryq_oracle as O
    torch.manual_seed(0)
    c = O.num_cherries(K_IN, 1 / 256)
    kc = K_IN - c
    q = torch.randint(0, 256, (kc // 8 * BITS, N_OUT), dtype=torch.uint8)
    s = (torch.rand(math.ceil(kc / GROUP), N_OUT) * 0.01 + 0.001).half()
    cw = (torch.randn(c, N_OUT) * 0.2).half()
    ci = torch.sort(torch.randperm(K_IN)[:c]).values.to(torch.int16)
    x = torch.randn(1, K_IN).half()
    return x, q, s, cw, ci, c


def host_threads():
    """Threads the CPU legs use: every core this process may run on (torchrun sets OMP_NUM_THREADS=1,
    which would otherwise leave the reference arm on one core), at most 32."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, 32))


def cpu_baseline(seconds=12.0):
    """The reference's dequantize-then-matmul CPU path on a bounded sample: repeated calls on the
    full-size layer for about `seconds`."""
    import torch
    from oracle import torch_port as TP
    torch.set_num_threads(host_threads())
    x, q, s, cw, ci, c = reference_inputs(torch)
    TP.forward_dequantize_then_matmul(x, q, s, cw, ci, BITS, GROUP)
    calls, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < seconds or calls < 3:
        TP.forward_dequantize_then_matmul(x, q, s, cw, ci, BITS, GROUP)
        calls += 1
    dt = (time.perf_counter() - t0) / calls
    nbytes = algorithmic_bytes(K_IN, N_OUT, BITS, GROUP, 1, c)
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{calls} calls of unpack()+F.linear on the full 4096x11008 layer, {dt * 1e3:.1f} ms per call",
            "ms_per_call": dt * 1e3}


def workload_config(**extra):
    """Keys both arms print, so that their `config` objects name the same workload."""
    cfg = {"workload": WORKLOAD, "bits": BITS, "group": GROUP, "K": K_IN, "N": N_OUT, "batch": 1}
    cfg.update(extra)
    return cfg


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import torch_port as TP
    torch.set_num_threads(host_threads())
    x, q, s, cw, ci, c = reference_inputs(torch)
    for _ in range(max(args.warmup, 1)):
        TP.forward_dequantize_then_matmul(x, q, s, cw, ci, BITS, GROUP)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        TP.forward_dequantize_then_matmul(x, q, s, cw, ci, BITS, GROUP)
    dt = (time.perf_counter() - t0) / args.steps
    nbytes = algorithmic_bytes(K_IN, N_OUT, BITS, GROUP, 1, c)
    v = nbytes / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "matvec_algorithmic_GBps_batch1", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": workload_config(path="reference CPU path: unpack() to dense fp16 + F.linear per call"),
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{args.steps} full-layer calls per run"},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# dram__bytes_read.sum + dram__bytes_write.sum of one cq_rowvec_kernel launch on this workload (one ncu capture,
# --clock-control none, two launches, the layer rotated over 17 copies)
NCU_DRAM_BYTES_PER_LAUNCH = 23_673_200
PREFILL_TOKENS = 2048


def median(v):
    v = sorted(v)
    return v[len(v) // 2]


class Region:
    """`steps` launches as CUDA graphs: every launch of the timed region is a graph node, none comes from
    Python.  The launches walk round-robin over the layer copies; when `steps` exceeds the number of copies
    a graph of one round is replayed and a second graph holds the remainder."""

    def __init__(self, torch, stream, launch, steps, ncopies):
        self.torch, self.stream = torch, stream
        self.rounds, rem = divmod(steps, ncopies)
        self.g_round = self._capture(launch, range(ncopies)) if self.rounds else None
        self.g_rem = self._capture(launch, range(rem)) if rem else None
        self.what = (f"CUDA graphs only: {self.rounds} replays of a graph of {ncopies} launches" if self.rounds else
                     "CUDA graphs only:") + (f" + one graph of {rem} launches" if rem else "")

    def _capture(self, launch, idx):
        g = self.torch.cuda.CUDAGraph()
        with self.torch.cuda.graph(g, stream=self.stream):
            for i in idx:
                launch(i)
        return g

    def run(self):
        for _ in range(self.rounds):
            self.g_round.replay()
        if self.g_rem is not None:
            self.g_rem.replay()

    def time(self, repeats):
        """Device time (ms) of `repeats` back-to-back runs of the region, one pair of events each."""
        ev = [(self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
        for e0, e1 in ev:
            e0.record(self.stream)
            self.run()
            e1.record(self.stream)
        self.stream.synchronize()
        return [e0.elapsed_time(e1) for e0, e1 in ev]


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import cherryq_b200
    from cherryq_b200 import _cabi
    qc = cherryq_b200.load_quant_cuda()
    lib = _cabi.lib()

    if N_OUT % (16 * world):
        raise RuntimeError(f"{world} ranks do not divide the layer's 16-row tiles")
    n_local = N_OUT // world
    # every rank draws the whole layer (same seed) and keeps its rows: rank 0 can check the gathered vector
    g = torch.Generator(device=dev).manual_seed(1234)
    c = math.ceil(K_IN / 256) // 8 * 8
    w = torch.randn(N_OUT, K_IN, device=dev, generator=g) * 0.02
    idx = torch.randperm(K_IN, device=dev, generator=g)[:c].to(torch.int32)
    w[:, idx.long()] = torch.randn(N_OUT, c, device=dev, generator=g) * 0.2
    w = w.half()
    q, s, cw, ci = qc.pack(w[rank * n_local:(rank + 1) * n_local].contiguous(), idx.contiguous(), BITS, GROUP)
    alg = algorithmic_bytes(K_IN, N_OUT, BITS, GROUP, 1, c)          # whole layer, all ranks
    alg_local = algorithmic_bytes(K_IN, n_local, BITS, GROUP, 1, c)

    def ptr(t):
        return C.c_void_p(t.data_ptr())

    def prepared(qq, ss, cc, ii, n):
        L = _cabi.rlayer_init(BITS, K_IN, n, c, GROUP)
        _cabi.check(lib.cq_rlayer_check(C.byref(L)), "cq_rlayer_check")
        b = torch.empty(L.blob_bytes, dtype=torch.uint8, device=dev)
        L.blob = b.data_ptr()
        # on the stream the buffers were packed on (torch's current one), then everything is awaited
        cur = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        _cabi.check(lib.cq_rlayer_prepare(C.byref(L), ptr(qq), ptr(ss), ptr(cc), ptr(ii), cur), "prepare")
        torch.cuda.synchronize()
        return L, b

    # distinct copies of the prepared layer: > 3x L2 in total
    L0, blob0 = prepared(q, s, cw, ci, n_local)
    ncopies = max(2, math.ceil(3 * L2_BYTES / L0.blob_bytes))
    layers, blobs = [L0], [blob0]
    for i in range(1, ncopies):
        L = _cabi.rlayer_init(BITS, K_IN, n_local, c, GROUP)
        b = blob0.clone()
        L.blob = b.data_ptr()
        layers.append(L)
        blobs.append(b)
    torch.cuda.synchronize()

    x = torch.randn(1, K_IN, device=dev, generator=g).half()
    y = torch.zeros(1, n_local, dtype=torch.float16, device=dev)
    y_all = torch.zeros(1, N_OUT, dtype=torch.float16, device=dev) if world > 1 else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.Stream(device=dev)
    sp = C.c_void_p(stream.cuda_stream)

    # the exchange step of the column-parallel layer: this library's peer-memory kernel, or NCCL when
    # asked for (--gather nccl) or when the peers' memory cannot be mapped (recorded in the line)
    peer, gather_kind = None, "none"
    if world > 1:
        gather_kind = "NCCL all-gather"
        if args.gather == "peer":
            from cherryq_b200.parallel import PeerAllGather
            try:
                peer = PeerAllGather(dist.group.WORLD, dev, capacity_bytes=1 << 20)
                gather_kind = "peer-memory exchange by the matvec's last CTA, same launch (cq_rlayer_matvec_gather)"
            except RuntimeError as exc:
                if rank == 0:
                    print(f"peer memory unavailable, using NCCL: {exc}", file=sys.stderr)

    def matvec(i):
        _cabi.check(lib.cq_rlayer_matvec(C.byref(layers[i % ncopies]), ptr(x), ptr(y), 0, ptr(status), sp), "matvec")

    def gather():
        if peer is not None:
            peer.gather_into(y, y_all, stream)
        elif world > 1:
            dist.all_gather_into_tensor(y_all.view(-1), y.view(-1))

    def step(i):
        if peer is not None:         # the matvec and the exchange of the slices in one launch
            _cabi.check(lib.cq_rlayer_matvec_gather(C.byref(layers[i % ncopies]), ptr(x), K_IN, ptr(y), 1, peer.regions, world,
                                                    rank, peer.capacity, ptr(y_all), peer.timeout_ms, ptr(peer.status), sp),
                        "matvec_gather")
        else:
            matvec(i)
            gather()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    repeats = max(1, args.repeats)
    gather_checked = None
    own_kernels_per_step = 1       # the matvec (at N > 1 its last CTA runs the exchange; NCCL's kernel is not counted)
    torch.cuda.synchronize()       # the inputs above were written on the default stream
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):          # warm-up: also sets kernel attributes before any capture
            step(i)
        stream.synchronize()
        if world > 1:
            barrier()        # every stream of the device (a library collective may run on one of its own), every rank
            # rank 0 computes the whole vector from the unsharded layer with the same kernel: every output element
            # is the same arithmetic whichever rank owns its row, so the gathered vector must match bit for bit
            ok = torch.ones(1, dtype=torch.int32, device=dev)
            if rank == 0:
                qf, sf, cwf, cif = qc.pack(w.contiguous(), idx.contiguous(), BITS, GROUP)
                Lf, bf = prepared(qf, sf, cwf, cif, N_OUT)
                yf = torch.zeros(1, N_OUT, dtype=torch.float16, device=dev)
                _cabi.check(lib.cq_rlayer_matvec(C.byref(Lf), ptr(x), ptr(yf), 0, ptr(status), sp), "matvec")
                stream.synchronize()
                ok[0] = int(torch.equal(yf.view(torch.int16), y_all.view(torch.int16)))
            # a second look after one more step and a full synchronisation, so that a collective still in flight on a
            # library's own stream cannot fail the check; a wrong result stays wrong
            dist.broadcast(ok, src=0)
            if not int(ok.item()):
                step(0)
                barrier()
                if rank == 0:
                    ok[0] = int(torch.equal(yf.view(torch.int16), y_all.view(torch.int16)))
            if rank == 0:
                if not int(ok.item()):
                    bad = (yf.view(torch.int16) != y_all.view(torch.int16)).view(-1).nonzero().view(-1)
                    print(f"gathered vector: {bad.numel()} of {N_OUT} elements differ, first at {bad[:4].tolist()}, last at "
                          f"{bad[-4:].tolist()} (rows per rank {n_local}); zeros in the gathered vector: "
                          f"{int((y_all == 0).sum())}; values {y_all.view(-1)[bad[:4]].tolist()} against {yf.view(-1)[bad[:4]].tolist()}; "
                          f"own slice equal: {torch.equal(y.view(-1), yf.view(-1)[:n_local])}", file=sys.stderr)
                del qf, sf, cwf, cif, bf, yf
            dist.broadcast(ok, src=0)
            gather_checked = bool(int(ok.item()))
            if not gather_checked:
                raise RuntimeError("the gathered output differs from the unsharded layer's")
        del w
        region = Region(torch, stream, step, args.steps, ncopies)
        region.run()                                   # one untimed pass of the graphs
        stream.synchronize()
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        times = region.time(repeats)
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        # the kernel alone (N == 1: the region holds nothing else)
        kern_times = times
        if world > 1:
            kregion = Region(torch, stream, matvec, args.steps, ncopies)
            kregion.run()
            stream.synchronize()
            kern_times = kregion.time(repeats)
    if world > 1:
        t = torch.tensor([times, kern_times], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)       # per repeat, the slowest rank
        times, kern_times = t[0].tolist(), t[1].tolist()
    if int(status.item()) != 0 or (peer is not None and int(peer.status.item()) != 0):
        raise RuntimeError("a device-side wait timed out during the benchmark")
    ms_step = median(times) / args.steps
    kern_ms = median(kern_times) / args.steps
    value = alg / (ms_step * 1e-3) / 1e9

    # ---------------------------------------------------------------- end to end through the drop-in op
    xh = torch.randn(1, K_IN).half().pin_memory()
    yh = torch.empty(1, N_OUT if rank == 0 else n_local, dtype=torch.float16).pin_memory()
    xd = torch.empty(1, K_IN, dtype=torch.float16, device=dev)
    out = torch.empty(1, n_local, dtype=torch.float16, device=dev)
    out_all = torch.empty(1, N_OUT, dtype=torch.float16, device=dev) if world > 1 else None
    refs = []
    for i in range(ncopies):                 # the op's own weight buffers (reference format), > 3x L2 in total
        refs.append((q, cw, ci, s) if i == 0 else tuple(t.clone() for t in (q, cw, ci, s)))

    def e2e_step(i):
        qq, cc, ii, ss = refs[i % ncopies]
        xd.copy_(xh, non_blocking=True)
        out.zero_()
        if BITS == 4:
            qc.vecquant4matmul_cherryq(xd, qq, cc, ii, ss, out, GROUP)
        else:
            qc.vecquant3matmul_cherryq(xd, qq, cc, ii, ss, out, GROUP, True)
        if world > 1:
            if peer is not None:
                peer.gather_into(out, out_all)
            else:
                dist.all_gather_into_tensor(out_all.view(-1), out.view(-1))
            if rank == 0:
                yh.copy_(out_all, non_blocking=True)      # the whole output vector reaches the host on rank 0
        else:
            yh.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed_host_loop(fn, n):
        """ms per call of n synchronous host-side calls (each returns with its result in host memory)."""
        for i in range(ncopies + 3):
            fn(i)
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(n):
            fn(i)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / n
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    e2e_steps = min(args.steps, 2000)
    op_ms = timed_host_loop(e2e_step, e2e_steps)
    qc.poll()
    op_path = (f"quant_cuda.vecquant{BITS}matmul_cherryq with pinned host x per rank" +
               (f", {gather_kind}, the whole y read back on rank 0" if world > 1 else " and y"))
    if world == 1:
        # the C ABI's host-buffer call: x from pinned host memory, y in pinned host memory when it returns
        xhp, yhp = C.c_void_p(xh.data_ptr()), C.c_void_p(yh.data_ptr())

        def host_step(i):
            _cabi.check(lib.cq_rlayer_matvec_host(C.byref(layers[i % ncopies]), xhp, yhp, ptr(xd), ptr(out), ptr(status),
                                                  None), "matvec_host")
        e2e_ms = timed_host_loop(host_step, e2e_steps)
        e2e_path = "cq_rlayer_matvec_host (C ABI): pinned host x in, pinned host y out, one call per step"
    else:
        e2e_ms, e2e_path = op_ms, op_path
    e2e = {"value": alg / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": K_IN * 2,
           "d2h_bytes_per_step": N_OUT * 2, "ms_per_step": e2e_ms, "steps": e2e_steps, "path": e2e_path,
           "through_the_torch_op": {"ms_per_step": op_ms, "value": alg / (op_ms * 1e-3) / 1e9, "path": op_path}}

    # the reference project's own CUDA kernel on the same layer copies (built by oracle/build_ref.py;
    # information only: batch 1, device-resident inputs, CUDA events)
    ref_gpu = None
    if world == 1 and rank == 0:
        try:
            from oracle import build_ref
            rmod = build_ref.load()
        except Exception:
            rmod = None
        if rmod is not None:
            rsteps = 10 * ncopies
            def ref_call(qq, cc, ii, ss):
                if BITS == 4:
                    rmod.vecquant4matmul_cherryq(xd, qq, cc, ii, ss, out, GROUP)
                else:
                    rmod.vecquant3matmul_cherryq(xd, qq, cc, ii, ss, out, GROUP, True)
            for i in range(ncopies):
                qq, cc, ii, ss = refs[i]
                ref_call(qq, cc, ii, ss)
            torch.cuda.synchronize()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record()
            for i in range(rsteps):
                qq, cc, ii, ss = refs[i % ncopies]
                ref_call(qq, cc, ii, ss)
            r1.record()
            torch.cuda.synchronize()
            rms = r0.elapsed_time(r1) / rsteps
            ref_gpu = {"kernel": f"VecQuant{BITS}MatMulKernelCherryQBatchedHalf (reference csrc/quant_cuda_kernel.cu, unmodified, sm_100a)",
                       "us_per_call": rms * 1e3, "GBps": alg / (rms * 1e-3) / 1e9, "steps": rsteps}

    region_what = region.what
    del layers, blobs, refs, region
    if world > 1:
        del kregion
    torch.cuda.empty_cache()

    # the other half of the path, same layer: the 2048-token prefill GEMM (single-GPU runs only)
    prefill = None
    if world == 1 and not args.no_cpu:
        prefill = prefill_measure(torch, dist, dev, world, rank, local, 60, 5)

    # the model-level number the metric names: LLaMA-2-70B-architecture 3-bit decode, tokens/s on these GPUs
    model70 = None
    if not args.no_model:
        if peer is not None:
            peer.close()
            peer = None
        try:
            model70 = model_measure(args, torch, dist, dev, world, rank, local, "70b", gen=64)
        except Exception as exc:          # the record says why it is missing; the headline line still prints
            model70 = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = alg_local / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": "matvec_algorithmic_GBps_batch1", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(
                l2_defeat=f"{ncopies} distinct layer copies ({ncopies * L0.blob_bytes / 1e6:.0f} MB) walked "
                          "round-robin, inputs larger than L2",
                parallelism="single GPU" if world == 1 else f"column-parallel over {world} GPUs + {gather_kind}",
                launch=region_what,
                timing=f"median of {repeats} back-to-back timed regions of {args.steps} steps each (CUDA events on the "
                       "launching stream, max over ranks per region)"),
            "pct_of_nominal_8TBps": value / world / 8000.0 * 100.0 if world == 1 else None,
            "region_ms": {"median": median(times), "min": min(times), "max": max(times), "repeats": repeats},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_DRAM_BYTES_PER_LAUNCH * alg_local / alg if NCU_DRAM_BYTES_PER_LAUNCH and not args.shape else None,
                         "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json)",
                         "kernel": "cq_rowvec_kernel<4,1,16,2,1>" if (K_IN, BITS) == (4096, 4) else "cq_rowvec_kernel", "alg_bytes_per_launch": alg_local,
                         "launch_us": kern_ms * 1e3},
            "e2e": e2e, "gpu_launches": args.steps * world * own_kernels_per_step,
            "clocks": clocks,
        }
        if gather_checked is not None:
            line["gather_checked"] = gather_checked
        line["cpu_baseline"] = cpu_baseline() if world == 1 and not args.no_cpu else None
        line["reference_gpu_kernel"] = ref_gpu
        if ref_gpu is not None:
            line["speedup_vs_reference_gpu_kernel"] = ref_gpu["us_per_call"] / (ms_step * 1e3)
        if prefill is not None:
            line["prefill"] = {k: prefill[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "roofline", "e2e")}
            line["prefill"]["workload"] = prefill["config"]["workload"]
        line["model_70b"] = model70
        print(json.dumps(line))
    leave(torch, dist, world)


def leave(torch, dist, world):
    """End of a multi-rank run.  The decode graphs of the model leg hold NCCL or peer-memory kernels; destroying
    the process group under live graphs blocked in the communicator's teardown when it was tried, so the ranks
    meet once more and leave the process without it."""
    if world <= 1:
        return
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def measured_tensor_peak():
    """Dense 16-bit tensor TFLOP/s measured on this pool (burst figure: the kernel is timed alone)."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def run_prefill(args):
    """Prefill of PREFILL_TOKENS tokens through one layer: the tensor-core GEMM of the path.  Same layer
    as the decode workload; the line reports dense TFLOP/s against the measured 16-bit tensor peak."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = prefill_measure(torch, dist, dev, world, rank, local, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def prefill_measure(torch, dist, dev, world, rank, local, steps_arg, warmup_arg):
    """Times the prefill GEMM (and its end-to-end leg) and returns the JSON line as a dict (rank 0)."""
    import cherryq_b200
    from cherryq_b200 import _cabi
    qc = cherryq_b200.load_quant_cuda()
    lib = _cabi.lib()
    M = PREFILL_TOKENS
    n_local = N_OUT
    if world > 1:
        # equal shards of whole 128-row tiles (the last tiles of the last rank are padding rows)
        n_local = math.ceil(N_OUT / 128 / world) * 128
    q, s, cw, ci, c = make_layer_gpu(qc, torch, K_IN, n_local, BITS, GROUP, 1234 + rank, dev)

    def ptr(t):
        return C.c_void_p(t.data_ptr())

    ncopies = 6                                      # 6 x 23 MB of weights + 62 MB of x / y per step > L2
    layers, blobs = [], []
    for i in range(ncopies):
        L = _cabi.tlayer_init(BITS, K_IN, n_local, c, GROUP)
        b = torch.empty(L.blob_bytes, dtype=torch.uint8, device=dev)
        L.blob = b.data_ptr()
        if i == 0:
            _cabi.check(lib.cq_tlayer_prepare(C.byref(L), ptr(q), ptr(s), ptr(cw), ptr(ci), None), "prepare")
            torch.cuda.synchronize()
        else:
            b.copy_(blobs[0])
        layers.append(L)
        blobs.append(b)
    x = torch.randn(M, K_IN, device=dev).half()
    y = torch.zeros(M, n_local, dtype=torch.float16, device=dev)
    ws = torch.empty(lib.cq_tlayer_gemm_workspace_bytes(C.byref(layers[0]), M), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.Stream(device=dev)
    sp = C.c_void_p(stream.cuda_stream)
    y_all = torch.empty(world, M, n_local, dtype=torch.float16, device=dev) if world > 1 else None

    def launch(i):
        _cabi.check(lib.cq_tlayer_gemm(C.byref(layers[i % ncopies]), ptr(x), K_IN, ptr(y), n_local, M, 0, ptr(ws),
                                       ptr(status), sp), "gemm")
        if world > 1:
            dist.all_gather_into_tensor(y_all, y)

    steps = min(steps_arg, 200)
    torch.cuda.synchronize()       # the inputs above were written on the default stream
    with torch.cuda.stream(stream):
        for i in range(max(warmup_arg, 3)):
            launch(i)
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            launch(i)
        e1.record(stream)
        stream.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if int(status.item()) != 0:
        raise RuntimeError("a device-side wait timed out during the benchmark")
    ms_step = ms / steps
    flops = 2.0 * M * K_IN * N_OUT
    value = flops / (ms_step * 1e-3) / 1e12

    # end to end through the drop-in op: host activations in, host outputs back
    xh = torch.randn(M, K_IN).half().pin_memory()
    yh = torch.empty(M, n_local, dtype=torch.float16).pin_memory()
    xd = torch.empty(M, K_IN, dtype=torch.float16, device=dev)
    out = torch.empty(M, n_local, dtype=torch.float16, device=dev)

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        out.zero_()
        qc.vecquant4matmul_cherryq(xd, q, cw, ci, s, out, GROUP)
        yh.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    e2e_steps = min(steps, 30)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    qc.poll()
    if rank == 0:
        peak, kind = measured_tensor_peak()
        achieved = flops / world / (ms_step * 1e-3) / 1e12
        line = {
            "metric": "prefill_dense_TFLOPs", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": max(warmup_arg, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"llama7b_gate_proj_4096x11008_4bit_g128_cherry1/256_prefill{M}", "bits": BITS,
                       "group": GROUP, "K": K_IN, "N": N_OUT, "tokens": M,
                       "l2_defeat": f"{ncopies} distinct layer copies + x, y, staged activations per step "
                                    f"({(ncopies * layers[0].blob_bytes + x.numel() * 2 + y.numel() * 2 + ws.numel()) / 1e6:.0f} MB) "
                                    "larger than L2",
                       "parallelism": "single GPU" if world == 1 else f"column-parallel over {world} GPUs + NCCL all-gather",
                       "launch": "stream launches (activation pre-pass + GEMM kernel per step)"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": kind + " cuBLAS bf16 burst (MEASURED_PEAKS.json)",
                         "kernel": "cq_prefill_kernel<4,1> (+ prefill_stage_x_kernel, inside the timed step)",
                         "flops_per_launch": flops / world, "launch_us": ms_step * 1e3},
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K_IN * 2,
                    "d2h_bytes_per_step": M * n_local * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "path": "quant_cuda.vecquant4matmul_cherryq with pinned host x / y per rank"},
            "gpu_launches": 2 * steps * world, "clocks": clocks, "cpu_baseline": None,
        }
        return line
    return None


def run_model(args):
    """Greedy decode of 256 tokens after a 128-token random prompt on a LLaMA-2 architecture with random-init
    CherryQ weights (batch 1): decode tokens/s, with the share of the quantized linears."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = model_measure(args, torch, dist, dev, world, rank, local, args.model, gen=args.gen, prompt_len=args.prompt,
                         batch=args.batch, max_seq=args.max_seq)
    if rank == 0:
        print(json.dumps(line))
    leave(torch, dist, world)


def model_measure(args, torch, dist, dev, world, rank, local, name, gen=256, prompt_len=128, batch=1, max_seq=512):
    """Builds the model, decodes `gen` tokens greedily after a `prompt_len`-token random prompt (one CUDA graph
    per decode step, as benchmark_perplexity.py:92-113 of the reference times its per-token loop) and returns
    the JSON record (rank 0; None elsewhere)."""
    from cherryq_b200 import decoder as D
    base = {"7b": D.LLAMA2_7B, "13b": D.LLAMA2_13B, "70b": D.LLAMA2_70B}[name]
    cfg = D.DecoderConfig(**{**base.__dict__, "max_seq": max_seq})
    t_build = time.time()
    model = D.CherryDecoder(cfg, device=dev, seed=1234, tp_group=dist.group.WORLD if world > 1 else None,
                            tp_gather=args.gather, release_reference_buffers=True, batch=batch)
    torch.cuda.synchronize()
    t_build = time.time() - t_build
    prompt = torch.randint(0, cfg.vocab, (batch, prompt_len), device=dev, generator=torch.Generator(device=dev).manual_seed(0))

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), r

    model.prefill(prompt)                       # first use: re-packs, workspaces
    prefill_ms, _ = timed(lambda: model.prefill(prompt))
    model.capture()
    model.prefill(prompt)
    model.generate(8)                           # warm the graph
    model.prefill(prompt)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    gen_ms, toks = timed(lambda: model.generate(gen))
    clocks = sampler.stop() if rank == 0 else None
    ranks_agree = None
    if world > 1:
        tt = torch.tensor([gen_ms, prefill_ms], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        gen_ms, prefill_ms = float(tt[0]), float(tt[1])
        same = toks.clone()
        dist.broadcast(same, src=0)
        agree = torch.tensor([int(torch.equal(same, toks))], device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        ranks_agree = bool(int(agree.item()))
        if not ranks_agree:
            raise RuntimeError("the ranks generated different tokens")
    tok_s = gen * batch / (gen_ms * 1e-3)

    # the quantized projections alone, same call sequence, captured the same way
    xin = {k: torch.randn(batch, k, device=dev).half() for k in {kk for kk, _ in model.shapes.values()}}
    s = torch.cuda.Stream(device=dev)
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s), torch.inference_mode():
        def all_linears():            # the decoder's own call pattern: q/k/v and gate/up share a launch
            for lay in model.layers:
                model._lins(lay, ("q", "k", "v"), xin[model.shapes["q"][0]])
                lay["o"](xin[model.shapes["o"][0]])
                model._lins(lay, ("gate", "up"), xin[model.shapes["gate"][0]])
                lay["down"](xin[model.shapes["down"][0]])
        all_linears()
        s.synchronize()
        gl = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gl, stream=s):
            all_linears()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    gl.replay()
    lin_ms, _ = timed(lambda: [gl.replay() for _ in range(20)])
    lin_ms /= 20
    with torch.inference_mode():
        h = torch.randn(batch, cfg.hidden, device=dev).half()
        for _ in range(3):
            torch.nn.functional.linear(h, model.lm_head)
        torch.cuda.synchronize()
        head_ms, _ = timed(lambda: [torch.nn.functional.linear(h, model.lm_head) for _ in range(50)])
    head_ms /= 50

    qbytes, hbytes = model.quantized_bytes_per_token() * world, model.lm_head_bytes()
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    ms_tok = gen_ms / gen
    return {
        "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": gen, "warmup": 8,
        "ms_per_step": ms_tok, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": f"llama2_{name}_arch_{cfg.bits}bit_g128_cherry1/256_prompt{prompt_len}_greedy{gen}_batch{batch}",
                   "batch": batch, "max_seq": max_seq,
                   "layers": cfg.n_layers, "kv_heads": cfg.n_kv_heads,
                   "hidden": cfg.hidden, "ffn": cfg.ffn, "vocab": cfg.vocab, "bits": cfg.bits,
                   "l2_defeat": f"{qbytes / 1e9:.1f} GB of quantized weights + {hbytes / 1e6:.0f} MB lm_head per token, "
                                "far larger than L2",
                   "parallelism": "single GPU" if world == 1 else
                                  f"column-parallel over {world} GPUs, 4 all-gathers per layer inside the graph "
                                  f"({'peer-memory exchange, for the o and down projections inside their own launch' if model.peer is not None else 'NCCL'})",
                   "launch": f"one CUDA graph per decode step ({cfg.n_layers * 7} quantized projections, attention, "
                             "norms, lm_head, argmax)"},
        "roofline": {"bound": "hbm", "achieved": (qbytes + hbytes) / (ms_tok * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": (qbytes + hbytes * world) / world / (ms_tok * 1e-3) / 1e9 / peak, "traffic": None,
                     "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json)",
                     "bytes_per_token": qbytes + hbytes},
        "split": {"quantized_linears_ms": lin_ms, "lm_head_ms": head_ms, "rest_ms": ms_tok - lin_ms - head_ms,
                  "quantized_linears_GBps": qbytes / (lin_ms * 1e-3) / 1e9},
        "prefill": {"tokens": prompt_len, "ms": prefill_ms, "tokens_per_s": prompt_len / (prefill_ms * 1e-3)},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the decode loop lives on the device (token ids are read back once at the end: "
                        f"{gen * 8} bytes); prompt upload {prompt_len * 8} bytes once"},
        "gpu_launches": gen * (cfg.n_layers * 7) * world, "clocks": clocks, "cpu_baseline": None,
        "build_s": t_build, "first_tokens": [int(t) for t in toks.reshape(gen, -1)[:8, 0].tolist()], "ranks_agree": ranks_agree,
    }


def run_sweep(args):
    """The three LLaMA-7B linear shapes x {4, 3} bits x batch {1, 4, 16} through the drop-in ops
    (`quant_cuda.vecquant{3,4}matmul_cherryq`, device-resident inputs, every call a CUDA-graph node, the
    layer rotated over more than 3x L2 of distinct copies), and the reference's own micro-benchmark case
    (benchmark_speed.py of the reference project: fp32 activations / scales / cherries / output, int32
    indices, 4096 -> 13824, 3-bit, batch 16, 100 calls)."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    peak, peak_kind = measured_peak()
    try:
        from oracle import build_ref
        rmod = build_ref.load()
    except Exception:
        rmod = None
    stream = torch.cuda.Stream(device=dev)
    repeats = max(3, min(args.repeats, 20))
    rows = []
    for (k, n) in ((4096, 4096), (4096, 11008), (11008, 4096)):
        for bits in (4, 3):
            q, s, cw, ci, c = make_layer_gpu(qc, torch, k, n, bits, GROUP, 1234, dev)
            nbytes = q.numel() + 2 * s.numel() + 2 * cw.numel()
            ncopies = max(2, math.ceil(3 * L2_BYTES / nbytes))
            copies = [(q, cw, ci, s)] + [tuple(t.clone() for t in (q, cw, ci, s)) for _ in range(ncopies - 1)]
            for m in (1, 4, 16):
                x = torch.randn(m, k, device=dev).half()
                out = torch.zeros(m, n, dtype=torch.float16, device=dev)

                def call(i, mod=qc):
                    qq, cc, ii, ss = copies[i % ncopies]
                    if bits == 4:
                        mod.vecquant4matmul_cherryq(x, qq, cc, ii, ss, out, GROUP)
                    else:
                        mod.vecquant3matmul_cherryq(x, qq, cc, ii, ss, out, GROUP, True)

                torch.cuda.synchronize()               # the buffers above were written on the default stream
                with torch.cuda.stream(stream):
                    for i in range(ncopies + 2):       # first use builds the re-packed copies (not capturable)
                        call(i)
                    stream.synchronize()
                    region = Region(torch, stream, call, 4 * ncopies, ncopies)
                    region.run()
                    stream.synchronize()
                    us = median(region.time(repeats)) * 1e3 / (4 * ncopies)
                alg = algorithmic_bytes(k, n, bits, GROUP, m, c)
                row = {"K": k, "N": n, "bits": bits, "batch": m, "us_per_call": us, "GBps": alg / us / 1e3,
                       "frac_of_measured_hbm": alg / us / 1e3 / peak,
                       "route": (f"row-tile kernel, {(m + 3) // 4} launch(es)" + (", tiles shared by 2 CTAs" if k - c > 8192 else ""))
                                if m <= (8 if k - c > 8192 else 12) else "tensor-core tile GEMM"}
                if rmod is not None and m == 1:        # the reference's kernels race in shared memory beyond batch 1
                    torch.cuda.synchronize()
                    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    for i in range(ncopies):
                        call(i, rmod)
                    r0.record()
                    for i in range(2 * ncopies):
                        call(i, rmod)
                    r1.record()
                    torch.cuda.synchronize()
                    row["reference_kernel_us"] = r0.elapsed_time(r1) * 1e3 / (2 * ncopies)
                rows.append(row)
            del copies
            qc.cache_clear()
            torch.cuda.empty_cache()

    # the reference's micro-benchmark, with its tensors and its loop of 100 calls
    bs, kk, nn = 16, 4096, 13824
    vec = torch.randn(bs, kk, device=dev)
    qweight = torch.randint(1, 5, (1530, nn), dtype=torch.uint8, device=dev)
    cherry_weight = torch.randn(16, nn, device=dev)
    cherry_indices = torch.randperm(16, dtype=torch.int32).sort().values.to(dev)
    scaling = torch.ones(32, nn, device=dev)
    mul = torch.zeros(bs, nn, device=dev)

    def speed_case(mod):
        mod.vecquant3matmul_cherryq(vec, qweight, cherry_weight, cherry_indices, scaling, mul, 128, False)   # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(100):
            mod.vecquant3matmul_cherryq(vec, qweight, cherry_weight, cherry_indices, scaling, mul, 128, False)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / 100 * 1e6

    fp32_case = {"case": "reference micro-benchmark: 4096 -> 13824, 3-bit, group 128, batch 16, fp32 in / out, 100 calls, "
                         "host clock around the loop as the reference script does",
                 "us_per_call": speed_case(qc)}
    if rmod is not None:
        fp32_case["reference_kernel_us_per_call"] = speed_case(rmod)
    wh = torch.randn(kk, nn, device=dev).half()
    vh = vec.half()
    torch.matmul(vh, wh)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(100):
        torch.matmul(vh, wh)
    torch.cuda.synchronize()
    fp32_case["torch_fp16_matmul_us_per_call"] = (time.perf_counter() - t0) / 100 * 1e6
    print(json.dumps({
        "metric": "matvec_algorithmic_GBps_sweep", "unit": "GB/s", "n_gpus": 1, "higher_is_better": True,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama7b_linear_shapes_x_bits_x_batch_through_the_drop_in_ops", "group": GROUP,
                   "l2_defeat": "distinct layer copies of more than 3x L2 walked round-robin",
                   "timing": f"median of {repeats} regions of 4 rounds over the copies, CUDA graphs only",
                   "peak": peak, "peak_kind": peak_kind + " copy bandwidth"},
        "rows": rows, "fp32_path": fp32_case}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "model", "sweep"],
                    help="decode: batch-1 matvec (the headline line); prefill: 2048-token GEMM of the same layer; "
                         "model: LLaMA-2-7B-architecture greedy decode, tokens/s; sweep: the 7B shapes x bits x batch table "
                         "and the reference's fp32 micro-benchmark case")
    ap.add_argument("--model", default="7b", choices=["7b", "13b", "70b"],
                    help="architecture of the model workload: LLaMA-2 7B (4-bit), 13B (3-bit) or 70B (3-bit, GQA)")
    ap.add_argument("--batch", type=int, default=1, help="model workload: sequences decoded in lockstep")
    ap.add_argument("--max-seq", type=int, default=512, help="model workload: positions of the KV cache")
    ap.add_argument("--prompt", type=int, default=128, help="model workload: prompt tokens per sequence")
    ap.add_argument("--gen", type=int, default=256, help="model workload: tokens generated per sequence")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="exchange step at N > 1: this library's peer-memory kernel (default) or NCCL")
    ap.add_argument("--repeats", type=int, default=50,
                    help="timed regions of --steps steps run back to back; the median is reported")
    ap.add_argument("--no-model", action="store_true", help="skip the 70B-architecture decode leg")
    ap.add_argument("--shape", default=None, metavar="KxNxBITS",
                    help="decode workload on another layer than the headline one, e.g. 28672x8192x3 (the 70B down "
                         "projection); for profiling: the line then names that layer as its workload")
    args = ap.parse_args()
    if args.shape:
        global K_IN, N_OUT, BITS, WORKLOAD
        K_IN, N_OUT, BITS = (int(v) for v in args.shape.lower().split("x"))
        WORKLOAD = f"linear_{K_IN}x{N_OUT}_{BITS}bit_g128_cherry1/256_batch1"
    if args.impl == "reference":
        if args.steps > 200:
            args.steps = 200        # each step is a full-layer CPU call (tens of ms): keep the run within minutes
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "model":
        run_model(args)
    elif args.workload == "sweep":
        run_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
