"""The drop-in ops keep a re-packed copy of a layer, found again by the addresses of its four
buffers.  Addresses are re-used: a layer that was freed and another one allocated in its place must
never be served the old copy.  Each case frees layer A, allocates a same-shaped layer B (the caching
allocator hands back the same blocks), calls the op and compares with the dequantised matmul of B."""
import gc

import numpy as np
import pytest

from oracle import cherryq_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

K, N, BITS, G = 512, 256, 4, 128


@pytest.fixture(scope="module")
def qc():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import cherryq_b200
    return cherryq_b200.load_quant_cuda()


def make_layer(qc, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).half()
    c = -(-K // 256) // 8 * 8
    idx = torch.randperm(K, device="cuda", generator=g)[:max(c, 8)].to(torch.int32)
    return qc.pack(w, idx.contiguous(), BITS, G)          # qweight, scales, cherry_weight, cherry_indices


def dense(bufs):
    q, s, cw, ci = (t.cpu().numpy() for t in bufs)
    return O.unpack(q, s, cw, ci, BITS, G, K).astype(np.float64)             # (N, K)


def call(qc, x, bufs):
    q, s, cw, ci = bufs
    out = torch.zeros(x.shape[0], N, dtype=torch.float16, device="cuda")
    qc.vecquant4matmul_cherryq(x, q, cw, ci, s, out, G)
    torch.cuda.synchronize()
    return out.cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("rows", [1, 4, 16])             # the one-row kernel, the few-row kernel, the tile GEMM
def test_freed_layer_is_never_served_to_its_successor(qc, rows):
    qc.cache_clear()
    x = torch.randn(rows, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rows)).half()
    a = make_layer(qc, 100 + rows)
    addr_a = [t.data_ptr() for t in a]
    ya = call(qc, x, a)
    ref_a = x.cpu().numpy().astype(np.float64) @ dense(a).T
    assert np.abs(ya - ref_a).max() <= 2e-3 * np.abs(ref_a).max()
    del a
    gc.collect()
    b = make_layer(qc, 200 + rows)
    addr_b = [t.data_ptr() for t in b]
    if addr_a != addr_b:
        pytest.skip("the allocator did not hand the freed blocks back")
    yb = call(qc, x, b)
    ref_b = x.cpu().numpy().astype(np.float64) @ dense(b).T
    assert np.abs(ref_a - ref_b).max() > 0.1 * np.abs(ref_b).max()          # the two layers really differ
    assert np.abs(yb - ref_b).max() <= 2e-3 * np.abs(ref_b).max()


@pytest.mark.parametrize("rows", [1, 16])
def test_weights_rewritten_in_place_need_an_explicit_clear(qc, rows):
    """Same storages, new contents (load_state_dict into existing buffers): the cache cannot see that;
    cache_clear() is the documented step, after which the new weights are used."""
    qc.cache_clear()
    x = torch.randn(rows, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)).half()
    a = make_layer(qc, 300)
    call(qc, x, a)
    b = make_layer(qc, 301)
    for dst, src in zip(a, b):
        dst.copy_(src)
    qc.cache_clear()
    y = call(qc, x, a)
    ref = x.cpu().numpy().astype(np.float64) @ dense(b).T
    assert np.abs(y - ref).max() <= 2e-3 * np.abs(ref).max()


def test_quantlinear_owns_its_copy():
    """QuantLinear keeps its re-packed copies itself and drops them when its buffers are replaced."""
    import cherryq_b200
    from cherryq_b200.qlinear import QuantLinear
    qc = cherryq_b200.load_quant_cuda()
    x = torch.randn(1, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(11)).half()
    lin = QuantLinear(BITS, G, None, 1 / 64, K, N, bias=False).cuda()
    a, b = make_layer(qc, 400), make_layer(qc, 401)
    for bufs in (a, b):
        q, s, cw, ci = bufs
        lin.load_state_dict({"qweight": q, "scales": s, "cherry_weight": cw, "cherry_indices": ci.to(torch.int16)},
                            strict=False)
        y = lin(x).float().cpu().numpy().astype(np.float64)
        ref = x.cpu().numpy().astype(np.float64) @ dense(bufs).T
        assert np.abs(y - ref).max() <= 2e-3 * np.abs(ref).max()


def test_released_layer_serves_every_batch_size_from_its_own_copies():
    """After release_reference_buffers() the module answers decode batches from its row-tile copy and large
    batches from its own tile-layout copy (built on first use), with the results of the unreleased module."""
    import cherryq_b200
    from cherryq_b200.qlinear import QuantLinear
    qc = cherryq_b200.load_quant_cuda()
    bufs = make_layer(qc, 500)
    lin = QuantLinear(BITS, G, None, 1 / 64, K, N, bias=False).cuda()
    lin.qweight, lin.scales, lin.cherry_weight, lin.cherry_indices = bufs
    xs = {rows: torch.randn(rows, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rows)).half()
          for rows in (1, 4, 7, 16, 64, 300)}
    before = {rows: lin(x).clone() for rows, x in xs.items()}
    ref = dense(bufs)
    lin.release_reference_buffers()
    assert lin.qweight.numel() == 0
    for rows, x in xs.items():
        y = lin(x)
        want = x.cpu().numpy().astype(np.float64) @ ref.T
        assert np.abs(y.float().cpu().numpy() - want).max() <= 2e-3 * np.abs(want).max()
        assert float((y.float() - before[rows].float()).abs().max()) <= 2e-3 * float(before[rows].float().abs().max())
    lin.restore_reference_buffers()
    for got, want in zip((lin.qweight, lin.scales, lin.cherry_weight, lin.cherry_indices), bufs):
        assert torch.equal(got, want)
