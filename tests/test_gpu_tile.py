"""GPU parity tests of the tile layout and the tcgen05 (UMMA + tensor memory) matvec, through
the C ABI."""
import ctypes as C

import numpy as np
import pytest

import stream_model as SM
from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O
from test_gpu_parity import dev, make_case, ptr, rel_err, TIGHT_TOL

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cabi():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cherryq_b200 import _cabi
    _cabi.lib()
    return _cabi


class TilePrepared:
    def __init__(self, cabi, qweight, scales, cw, idx, bits, K, G):
        self.cabi = cabi
        self.t = [dev(qweight), dev(scales), dev(cw), dev(idx)]
        N, Cn = qweight.shape[1], len(idx)
        self.L = cabi.tlayer_init(bits, K, N, Cn, G)
        self.blob = torch.zeros(self.L.blob_bytes, dtype=torch.uint8, device="cuda")
        self.L.blob = self.blob.data_ptr()
        cabi.check(cabi.lib().cq_tlayer_prepare(C.byref(self.L), *[ptr(t) for t in self.t], None), "tprepare")
        torch.cuda.synchronize()
        self.scratch = torch.zeros(cabi.lib().cq_scratch_bytes(), dtype=torch.uint8, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def matvec(self, x, y=None, accumulate=False):
        xd = dev(x) if isinstance(x, np.ndarray) else x
        M = xd.shape[0]
        if y is None:
            y = torch.full((M, self.L.N), float("nan"), dtype=torch.float16, device="cuda")
        self.cabi.check(self.cabi.lib().cq_tlayer_matvec(C.byref(self.L), ptr(xd), self.L.K, ptr(y), self.L.N, M,
                                                         int(accumulate), ptr(self.scratch), ptr(self.status), None),
                        "tmatvec")
        torch.cuda.synchronize()
        assert int(self.status.item()) == 0, f"a device-side wait timed out (status {int(self.status.item())})"
        return y


@pytest.mark.parametrize("name", golden_cases())
def test_tile_prepare_matches_model_and_roundtrips(cabi, name):
    g = load_golden(name)
    p = TilePrepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    model, d = SM.build_tile_blob(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    got = p.blob.cpu().numpy()
    assert d["blob_bytes"] == p.L.blob_bytes
    for sec, nbytes in (("off_stream", d["n_tile"] * d["tile_bytes"]), ("off_cidx", 2 * d["Cp"]),
                        ("off_osh", 4 * (d["Kp"] // 8))):
        o = d[sec]
        assert np.array_equal(got[o:o + nbytes], model[o:o + nbytes]), sec
    outs = [torch.zeros_like(t) for t in p.t]
    cabi.check(cabi.lib().cq_tlayer_unprepare(C.byref(p.L), *[ptr(t) for t in outs], None), "tunprepare")
    torch.cuda.synchronize()
    for a, b in zip(outs, p.t):
        assert torch.equal(a, b)


@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("M", [1, 3, 5])
def test_tile_matvec_golden(cabi, name, M):
    g = load_golden(name)
    p = TilePrepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    x = g["x"][:M]
    y = p.matvec(x).cpu().numpy()
    assert np.isfinite(y).all()
    assert rel_err(y, g["y"][:M].astype(np.float64)) <= TIGHT_TOL
    y2 = p.matvec(x).cpu().numpy()
    assert np.array_equal(y.view(np.uint16), y2.view(np.uint16))


@pytest.mark.parametrize("bits", [4, 3])
@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 11008), (11008, 4096)])
def test_tile_matvec_llama7b_shapes(cabi, K, N, bits):
    w, idx, p, dense = make_case(K, N, bits, 128, seed=K + N + bits)
    prep = TilePrepared(cabi, p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], bits, K, 128)
    rng = np.random.default_rng(5)
    for M in (1, 4, 16):
        x = rng.normal(size=(M, K)).astype(np.float16)
        y = prep.matvec(x).cpu().numpy()
        assert rel_err(y, O.forward_dense_fp64(x, dense)) <= TIGHT_TOL, (K, N, bits, M)


@pytest.mark.parametrize("K,N,bits,G,frac,M", [
    (256, 8, 4, 128, 1 / 16, 1),
    (136, 24, 3, 128, 1 / 17, 3),
    (1024, 4744, 4, 128, 1 / 64, 1),
    (8192, 1024, 3, 128, 1 / 256, 8),
    (2048, 512, 3, 64, 1 / 256, 16),
    (2048, 512, 4, 2048, 1 / 256, 9),
    (512, 64, 4, 128, 0.0, 4),
    (28672, 256, 3, 128, 1 / 256, 2),
])
def test_tile_matvec_edge_shapes(cabi, K, N, bits, G, frac, M):
    w, idx, p, dense = make_case(K, N, bits, G, seed=K * 7 + N, frac=frac)
    prep = TilePrepared(cabi, p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], bits, K, G)
    x = np.random.default_rng(1).normal(size=(M, K)).astype(np.float16)
    y = prep.matvec(x).cpu().numpy()
    assert rel_err(y, O.forward_dense_fp64(x, dense)) <= TIGHT_TOL


def test_tile_matvec_accumulates_and_walks_large_batches(cabi):
    w, idx, p, dense = make_case(2048, 384, 4, 128, seed=9)
    prep = TilePrepared(cabi, p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], 4, 2048, 128)
    x = np.random.default_rng(2).normal(size=(37, 2048)).astype(np.float16)
    base = np.random.default_rng(3).normal(size=(37, 384)).astype(np.float16)
    y = prep.matvec(x, y=dev(base.copy()), accumulate=True).cpu().numpy()
    assert rel_err(y, O.forward_dense_fp64(x, dense) + base.astype(np.float64)) <= TIGHT_TOL
