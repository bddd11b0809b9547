"""Peer-memory all-gather kernel (cq_peer_allgather).  On one device: the degenerate one-rank
exchange over several calls (landing-area parity, call counter), argument checks, and the bounded
wait: a second rank that does not exist never raises its flag, the kernel gives up after the time
limit, sets the status bit, fills the output with NaN and stays usable.  On two devices: worker
processes compare the kernel with NCCL's all-gather, eagerly and inside a CUDA graph."""
import ctypes as C
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CAP = 1 << 20


@pytest.fixture()
def region():
    from cherryq_b200 import _cabi
    lib = _cabi.lib()
    p = C.c_void_p()
    _cabi.check(lib.cq_peer_region_create(CAP, C.byref(p)), "create")
    yield lib, _cabi, p
    torch.cuda.synchronize()
    _cabi.check(lib.cq_peer_region_destroy(p), "destroy")


def _gather(lib, regions, world, rank, x, out, status, timeout_ms=500):
    cv = C.c_void_p
    return lib.cq_peer_allgather(regions, world, rank, CAP, cv(x.data_ptr()), cv(out.data_ptr()), x.shape[0], x.shape[1],
                                 timeout_ms, cv(status.data_ptr()), cv(torch.cuda.current_stream().cuda_stream))


def test_one_rank_exchange_over_many_calls(region):
    lib, _cabi, p = region
    regions = (C.c_void_p * 1)(p.value)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for i, (rows, cols) in enumerate([(1, 1376), (1, 8), (4, 512), (16, 4096), (1, 1376), (3, 24), (37, 128)]):
        x = torch.randn(rows, cols, device="cuda").half()
        out = torch.zeros(rows, cols, dtype=torch.float16, device="cuda")
        _cabi.check(_gather(lib, regions, 1, 0, x, out, status), "gather")
        assert torch.equal(out, x), (i, rows, cols)
    assert int(status.item()) == 0


def test_argument_checks(region):
    lib, _cabi, p = region
    regions = (C.c_void_p * 1)(p.value)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.zeros(1, 12, dtype=torch.float16, device="cuda")
    assert _gather(lib, regions, 1, 0, x, x.clone(), status) == 4            # cols_local not a multiple of 8
    big = torch.zeros(64, 16384, dtype=torch.float16, device="cuda")          # 2 MB, 4 MB on the wire > capacity
    assert _gather(lib, regions, 1, 0, big, big.clone(), status) == 5
    ok = torch.zeros(1, 16, dtype=torch.float16, device="cuda")
    assert _gather(lib, regions, 1, 1, ok, ok.clone(), status) == 1           # rank outside the world
    assert _gather(lib, regions, 1, 0, ok, ok.clone(), status, timeout_ms=0) == 1


def test_absent_peer_runs_into_the_time_limit(region):
    lib, _cabi, p = region
    # "two ranks" whose regions are both this one: rank 1 does not exist, its flag is never raised
    regions = (C.c_void_p * 2)(p.value, p.value)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.randn(1, 256, device="cuda").half()
    out = torch.full((1, 512), 7.0, dtype=torch.float16, device="cuda")
    _cabi.check(_gather(lib, regions, 2, 0, x, out, status, timeout_ms=200), "gather")
    torch.cuda.synchronize()
    assert int(status.item()) & 8                                             # CQ_ERR_DEVICE_TIMEOUT
    assert bool(torch.isnan(out).all())                                       # nothing stale can pass for a result
    # the context and the region stay usable: the next one-rank call works
    status.zero_()
    one = (C.c_void_p * 1)(p.value)
    out1 = torch.zeros(1, 256, dtype=torch.float16, device="cuda")
    _cabi.check(_gather(lib, one, 1, 0, x, out1, status), "gather")
    assert torch.equal(out1, x) and int(status.item()) == 0


def test_capacity_mismatch_is_reported(region):
    """A call that states another capacity than the region was created with would address the landing areas
    wrongly: it sends nothing and ends with the time-out status and a NaN output."""
    lib, _cabi, p = region
    regions = (C.c_void_p * 1)(p.value)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.randn(1, 256, device="cuda").half()
    out = torch.zeros(1, 256, dtype=torch.float16, device="cuda")
    cv = C.c_void_p
    rc = lib.cq_peer_allgather(regions, 1, 0, CAP // 2, cv(x.data_ptr()), cv(out.data_ptr()), 1, 256, 200, cv(status.data_ptr()),
                               cv(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & 8 and bool(torch.isnan(out).all())
    status.zero_()
    _cabi.check(_gather(lib, regions, 1, 0, x, out, status), "gather")           # the right capacity works afterwards
    assert torch.equal(out, x) and int(status.item()) == 0


def _one_layer(K=2048, N=264, bits=4):
    import math
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    g = torch.Generator(device="cuda").manual_seed(5)
    c = math.ceil(K / 256) // 8 * 8
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).half()
    idx = torch.randperm(K, device="cuda", generator=g)[:c].to(torch.int32)
    q, s, cw, ci = qc.pack(w, idx.contiguous(), bits, 128)
    return qc, qc.RowLayer(q, s, cw, ci, bits, K, 128)


def test_matvec_with_exchange_in_one_launch_single_rank(region):
    """cq_rlayer_matvec_gather on a world of one: the last CTA of the matvec runs the exchange with itself;
    repeated and mixed with plain exchanges on the same region (one call sequence)."""
    lib, _cabi, p = region
    qc, row = _one_layer()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for rows in (1, 4, 2, 1):
        x = torch.randn(rows, 2048, device="cuda").half()
        want = torch.empty(rows, 264, dtype=torch.float16, device="cuda")
        row.matvec(x, want, False)
        y_local = torch.zeros_like(want)
        y_all = torch.zeros_like(want)
        for _ in range(3):
            row.matvec_gather(x, y_local, y_all, [p.value], 0, CAP, 500, status)
            torch.cuda.synchronize()
            assert torch.equal(y_all, want) and torch.equal(y_local, want)
            regions = (C.c_void_p * 1)(p.value)
            out = torch.zeros_like(want)
            _cabi.check(_gather(lib, regions, 1, 0, want, out, status), "gather")
            assert torch.equal(out, want)
    assert int(status.item()) == 0


def test_matvec_with_exchange_absent_peer_times_out(region):
    lib, _cabi, p = region
    qc, row = _one_layer()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.randn(1, 2048, device="cuda").half()
    want = torch.empty(1, 264, dtype=torch.float16, device="cuda")
    row.matvec(x, want, False)
    y_local = torch.zeros_like(want)
    y_all = torch.full((1, 528), 7.0, dtype=torch.float16, device="cuda")
    # "two ranks" whose regions are both this one: rank 1 does not exist and never delivers
    row.matvec_gather(x, y_local, y_all, [p.value, p.value], 0, CAP, 200, status)
    torch.cuda.synchronize()
    assert int(status.item()) & 8                                             # CQ_ERR_DEVICE_TIMEOUT
    assert torch.equal(y_local, want) and bool(torch.isnan(y_all).all())
    # the context and the region stay usable
    status.zero_()
    y_all1 = torch.zeros_like(want)
    row.matvec_gather(x, y_local, y_all1, [p.value], 0, CAP, 500, status)
    torch.cuda.synchronize()
    assert torch.equal(y_all1, want) and int(status.item()) == 0


def test_two_ranks_match_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "peer_gather_worker.py")
    out = tmp_path / "result.txt"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", worker, str(out)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stderr[-2000:]
    assert out.read_text().strip() == "ok"
