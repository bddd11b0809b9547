"""GPU parity tests of the tile layout of the prefill GEMM (re-pack against the numpy model, and
back), through the C ABI."""
import ctypes as C

import numpy as np
import pytest

import stream_model as SM
from conftest import golden_cases, load_golden
from test_gpu_parity import dev, ptr

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
