"""cq_layer_matvec_static: the matvec entry point that brings its own scratch (a fixed array in
the library's device image) and allocates nothing.  Called through the C ABI and compared with
cq_layer_matvec on the same inputs, two calls in a row.  This file sorts last on purpose, so that
the shared array is also exercised after everything else has run; it passes on its own too."""
import ctypes as C

import numpy as np
import pytest

from conftest import load_golden
from oracle import cherryq_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CQ_ERR_STATIC_LIMIT = 10


@pytest.fixture(scope="module")
def cabi():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cherryq_b200 import _cabi
    _cabi.lib()
    return _cabi


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr())


class Layer:
    def __init__(self, cabi, p, bits, K, G):
        self.cabi, self.lib = cabi, cabi.lib()
        self.t = [dev(p["qweight"]), dev(p["scales"]), dev(p["cherry_weight"]), dev(p["cherry_indices"])]
        self.L = cabi.layer_init(bits, K, p["qweight"].shape[1], len(p["cherry_indices"]), G)
        self.blob = torch.zeros(self.L.blob_bytes, dtype=torch.uint8, device="cuda")
        self.L.blob = self.blob.data_ptr()
        cabi.check(self.lib.cq_layer_prepare(C.byref(self.L), *[ptr(t) for t in self.t], None), "prepare")
        self.scratch = torch.zeros(self.lib.cq_scratch_bytes(), dtype=torch.uint8, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()

    def with_scratch(self, x, y, accumulate=0):
        self.cabi.check(self.lib.cq_layer_matvec(C.byref(self.L), ptr(x), self.L.K, ptr(y), self.L.N, x.shape[0],
                                                 accumulate, ptr(self.scratch), ptr(self.status), None), "matvec")

    def static(self, x, y, accumulate=0):
        return self.lib.cq_layer_matvec_static(C.byref(self.L), ptr(x), self.L.K, ptr(y), self.L.N, x.shape[0],
                                               accumulate, ptr(self.status), None)


def bits_of(t):
    return t.cpu().numpy().view(np.uint16)


def run_twice_and_compare(layer, x):
    M, N = x.shape[0], layer.L.N
    want = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    layer.with_scratch(x, want)
    torch.cuda.synchronize()
    outs = [torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for y in outs:         # back to back on one stream: the second call reuses the array as the first left it
        assert layer.static(x, y) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory in use changed across the calls"
    assert int(layer.status.item()) == 0
    for y in outs:
        assert np.array_equal(bits_of(y), bits_of(want))
    return want


@pytest.mark.parametrize("name", ["k256_n32_b4_g128_f16", "k2048_n16_b3_g128_f16"])
@pytest.mark.parametrize("M", [1, 5])
def test_static_scratch_matches_on_golden_layers(cabi, name, M):
    g = load_golden(name)
    layer = Layer(cabi, g, int(g["bits"]), int(g["K"]), int(g["G"]))
    y = run_twice_and_compare(layer, dev(g["x"][:M])).cpu().numpy().astype(np.float64)
    ref = g["y"][:M].astype(np.float64)
    assert np.abs(y - ref).max() / np.abs(ref).max() <= 2e-3


@pytest.mark.parametrize("bits,M", [(4, 1), (3, 1), (4, 16)])
def test_static_scratch_matches_at_full_size(cabi, bits, M):
    # 4096 -> 11008: every CTA contributes partial sums to rows it does not finish itself
    K, N, G = 4096, 11008, 128
    w, idx = O.make_layer(K, N, bits, G, 1 / 256, 11, np.float16)
    p = O.pack(w, idx, bits, G)
    layer = Layer(cabi, p, bits, K, G)
    x = dev(np.random.default_rng(5).normal(size=(M, K)).astype(np.float16))
    run_twice_and_compare(layer, x)
    # accumulate mode, and interleaved with the scratch-taking entry point
    base = torch.randn(M, N, device="cuda").half()
    a, b = base.clone(), base.clone()
    layer.with_scratch(x, a, accumulate=1)
    assert layer.static(x, b, accumulate=1) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits_of(a), bits_of(b))


def test_static_scratch_rejects_requests_beyond_its_limits(cabi):
    g = load_golden("k256_n32_b4_g128_f16")
    layer = Layer(cabi, g, 4, int(g["K"]), int(g["G"]))
    x = torch.zeros(17, int(g["K"]), dtype=torch.float16, device="cuda")
    y = torch.full((17, layer.L.N), 3.0, dtype=torch.float16, device="cuda")
    rc = layer.static(x, y)
    assert rc == CQ_ERR_STATIC_LIMIT
    msg = layer.lib.cq_strerror(rc)
    msg = (msg if isinstance(msg, bytes) else C.cast(msg, C.c_char_p).value).decode()
    assert "cq_layer_matvec_static" in msg and "16 rows" in msg
    torch.cuda.synchronize()
    assert bool((y == 3.0).all()), "a rejected call must not launch"
    assert layer.static(x[:0], y[:0]) == 1          # M = 0: bad argument, as for cq_layer_matvec
