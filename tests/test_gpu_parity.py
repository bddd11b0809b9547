"""GPU parity tests: every call goes through the C ABI of libcherryq.so (ctypes, raw
device pointers) or through the `quant_cuda` extension built on top of it, and is
compared with the numpy oracle / the golden fixtures frozen from the reference."""
import ctypes as C

import numpy as np
import pytest

import stream_model as SM
from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-2     # north-star bound: max |y - y_ref| / max |y_ref| against the fp32/fp64 dequantised matmul
TIGHT_TOL = 2e-3   # what fp32 accumulation + one fp16 store actually delivers


@pytest.fixture(scope="module")
def cabi():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cherryq_b200 import _cabi
    _cabi.lib()
    return _cabi


@pytest.fixture(scope="module")
def qc():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import cherryq_b200
    return cherryq_b200.load_quant_cuda()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr())


class Prepared:
    """A layer prepared through the C ABI from reference-format numpy buffers."""

    def __init__(self, cabi, qweight, scales, cw, idx, bits, K, G):
        self.cabi = cabi
        self.t = [dev(qweight), dev(scales), dev(cw), dev(idx)]
        N, Cn = qweight.shape[1], len(idx)
        self.L = cabi.layer_init(bits, K, N, Cn, G)
        self.blob = torch.zeros(self.L.blob_bytes, dtype=torch.uint8, device="cuda")
        self.L.blob = self.blob.data_ptr()
        cabi.check(cabi.lib().cq_layer_prepare(C.byref(self.L), *[ptr(t) for t in self.t], None), "prepare")
        torch.cuda.synchronize()
        self.scratch = torch.zeros(cabi.lib().cq_scratch_bytes(), dtype=torch.uint8, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def matvec(self, x, y=None, accumulate=False):
        xd = dev(x) if isinstance(x, np.ndarray) else x
        M = xd.shape[0]
        if y is None:
            y = torch.full((M, self.L.N), float("nan"), dtype=torch.float16, device="cuda")
        self.cabi.check(self.cabi.lib().cq_layer_matvec(C.byref(self.L), ptr(xd), self.L.K, ptr(y), self.L.N, M,
                                                        int(accumulate), ptr(self.scratch), ptr(self.status), None),
                        "matvec")
        torch.cuda.synchronize()
        assert int(self.status.item()) == 0, "a device-side wait timed out"
        return y


def rel_err(y, ref):
    return float(np.abs(y.astype(np.float64) - ref).max() / np.abs(ref).max())


# ------------------------------------------------------------------ re-pack
@pytest.mark.parametrize("name", golden_cases())
def test_prepare_matches_layout_model_and_roundtrips(cabi, name):
    g = load_golden(name)
    p = Prepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    model, d = SM.build_blob(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    got = p.blob.cpu().numpy()
    assert d["blob_bytes"] == p.L.blob_bytes
    for sec, nbytes in (("off_stream", d["n_sub"] * d["n_gran"] * d["gran_bytes"]),
                        ("off_cherry", d["n_sub"] * d["cher_bytes"]),
                        ("off_osh", 4 * (d["Kp"] // 8)), ("off_cidx", 2 * d["Cp"])):
        o = d[sec]
        assert np.array_equal(got[o:o + nbytes], model[o:o + nbytes]), sec
    # inverse re-pack: byte-identical reference buffers
    outs = [torch.zeros_like(t) for t in p.t]
    cabi.check(cabi.lib().cq_layer_unprepare(C.byref(p.L), *[ptr(t) for t in outs], None), "unprepare")
    torch.cuda.synchronize()
    for a, b in zip(outs, p.t):
        assert torch.equal(a, b)


# ------------------------------------------------------------------ matvec on the golden layers
@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("M", [1, 2, 5])
def test_matvec_golden(cabi, name, M):
    g = load_golden(name)
    p = Prepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    x = g["x"][:M]
    y = p.matvec(x).cpu().numpy()
    assert np.isfinite(y).all()
    assert rel_err(y, g["y"][:M].astype(np.float64)) <= TIGHT_TOL
    ref = O.kernel_forward(x, g["qweight"], g["cherry_weight"], g["cherry_indices"], g["scales"], g["bits"], g["G"])
    assert rel_err(y, ref) <= 1e-3
    # bit-identical on a second run (no floating-point atomics anywhere)
    y2 = p.matvec(x).cpu().numpy()
    assert np.array_equal(y.view(np.uint16), y2.view(np.uint16))


def test_matvec_accumulates_like_the_reference(cabi):
    g = load_golden("k256_n32_b4_g128_f16")
    p = Prepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], 4, g["K"], g["G"])
    x = g["x"][:3]
    base = np.random.default_rng(0).normal(size=(3, g["N"])).astype(np.float16)
    y = p.matvec(x, y=dev(base.copy()), accumulate=True).cpu().numpy()
    ref = g["y"][:3].astype(np.float64) + base.astype(np.float64)
    assert rel_err(y, ref) <= TIGHT_TOL


def make_case(K, N, bits, G, seed, frac=1 / 256):
    w, idx = O.make_layer(K, N, bits, G, frac, seed, np.float16)
    p = O.pack(w, idx, bits, G)
    dense = O.unpack(p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], bits, G, K)
    return w, idx, p, dense


SHAPES = [(4096, 4096), (4096, 11008), (11008, 4096)]


@pytest.mark.parametrize("bits", [4, 3])
@pytest.mark.parametrize("K,N", SHAPES)
def test_matvec_llama7b_shapes(cabi, K, N, bits):
    """The headline configuration: LLaMA-7B linear shapes, 3- and 4-bit, group 128, cherry ratio 1/256, batch 1/4/16."""
    w, idx, p, dense = make_case(K, N, bits, 128, seed=K + N + bits)
    prep = Prepared(cabi, p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], bits, K, 128)
    rng = np.random.default_rng(5)
    for M in (1, 4, 16):
        x = rng.normal(size=(M, K)).astype(np.float16)
        y = prep.matvec(x).cpu().numpy()
        ref = O.forward_dense_fp64(x, dense)
        assert rel_err(y, ref) <= TIGHT_TOL, (K, N, bits, M)
    # GPU pack of the same weight is byte-identical to the oracle's pack
    outs = gpu_pack(cabi, w, idx, bits, 128)
    for key in ("qweight", "scales", "cherry_weight", "cherry_indices"):
        assert np.array_equal(outs[key].view(np.uint8), p[key].view(np.uint8)), key
    # GPU dense unpack is byte-identical to the oracle's unpack
    d = gpu_unpack(cabi, p, bits, K, 128)
    assert np.array_equal(d.view(np.uint16), dense.view(np.uint16))


@pytest.mark.parametrize("K,N,bits,G,frac,M", [
    (256, 8, 4, 128, 1 / 16, 1),        # one sub-tile, half of it padding rows
    (136, 24, 3, 128, 1 / 17, 3),       # K' = 128 exactly after 8 cherries
    (264, 40, 4, 128, 1 / 33, 2),       # K' = 256
    (1024, 4744, 4, 128, 1 / 64, 1),    # N not a multiple of 16 * anything nice, many sub-tiles per CTA
    (8192, 1024, 3, 128, 1 / 256, 8),   # GQA k/v projection shape of the 70B configuration
    (2048, 512, 3, 64, 1 / 256, 16),    # 64-wide groups, two activation tiles
    (2048, 512, 4, 2048, 1 / 256, 9),   # one group per row
    (512, 64, 4, 128, 0.0, 4),          # no cherries at all
    (28672, 256, 3, 128, 1 / 256, 2),   # longest K of the configurations (112 cherries)
])
def test_matvec_edge_shapes(cabi, K, N, bits, G, frac, M):
    w, idx, p, dense = make_case(K, N, bits, G, seed=K * 7 + N, frac=frac)
    prep = Prepared(cabi, p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], bits, K, G)
    x = np.random.default_rng(1).normal(size=(M, K)).astype(np.float16)
    y = prep.matvec(x).cpu().numpy()
    assert rel_err(y, O.forward_dense_fp64(x, dense)) <= TIGHT_TOL


def test_matvec_more_rows_than_one_launch_takes(cabi):
    """M > 16 (and M * K beyond the shared-memory plan) is split into several launches."""
    w, idx, p, dense = make_case(11008, 256, 4, 128, seed=3)
    prep = Prepared(cabi, p["qweight"], p["scales"], p["cherry_weight"], p["cherry_indices"], 4, 11008, 128)
    x = np.random.default_rng(2).normal(size=(37, 11008)).astype(np.float16)
    y = prep.matvec(x).cpu().numpy()
    assert rel_err(y, O.forward_dense_fp64(x, dense)) <= TIGHT_TOL


def test_linearity_and_zero_at_full_size(cabi):
    """Size-independent properties on the north-star layer (4096 -> 11008, 4-bit)."""
    K, N = 4096, 11008
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randint(0, 256, (4080 // 2, N), dtype=torch.uint8, device="cuda", generator=g)
    s = (torch.rand(32, N, device="cuda", generator=g) * 0.01 + 0.001).half()
    cw = (torch.randn(16, N, device="cuda", generator=g) * 0.2).half()
    idx = torch.sort(torch.randperm(K, device="cuda", generator=g)[:16]).values.to(torch.int16)
    prep = Prepared(cabi, q.cpu().numpy(), s.cpu().numpy(), cw.cpu().numpy(), idx.cpu().numpy(), 4, K, 128)
    x1 = torch.randn(1, K, device="cuda", generator=g).half()
    zero = prep.matvec(torch.zeros_like(x1))
    assert torch.count_nonzero(zero) == 0
    y1 = prep.matvec(x1).float()
    y2 = prep.matvec((x1 * 2).half()).float()
    assert float((y2 - 2 * y1).abs().max() / y2.abs().max()) <= 2e-3
    # a unit vector picks out one dequantised column: compare with the GPU dense unpack
    dense = torch.zeros(N, K, dtype=torch.float16, device="cuda")
    cabi.check(cabi.lib().cq_unpack_dense(ptr(q), ptr(s), ptr(cw), ptr(idx), 4, K, N, 16, 128, ptr(dense), None), "unpack")
    for col in (0, int(idx[0]), 4095, 1234):
        e = torch.zeros(1, K, dtype=torch.float16, device="cuda")
        e[0, col] = 1.0
        y = prep.matvec(e)[0].float()
        assert float((y - dense[:, col].float()).abs().max()) <= 1e-3 * float(dense[:, col].float().abs().max())


# ------------------------------------------------------------------ pack / unpack / dequantize
def gpu_pack(cabi, w, idx, bits, G):
    N, K = w.shape
    Cn = len(idx)
    wd, idd = dev(w), dev(idx.astype(np.int32))
    q = torch.zeros(((K - Cn) // 8 * bits, N), dtype=torch.uint8, device="cuda")
    s = torch.zeros(((K - Cn + G - 1) // G, N), dtype=torch.float16, device="cuda")
    cw = torch.zeros((Cn, N), dtype=torch.float16, device="cuda")
    ci = torch.zeros((Cn,), dtype=torch.int16, device="cuda")
    cabi.check(cabi.lib().cq_pack(ptr(wd), int(w.dtype == np.float32), ptr(idd), bits, K, N, Cn, G,
                                  ptr(q), ptr(s), ptr(cw), ptr(ci), None, None), "pack")
    torch.cuda.synchronize()
    return dict(qweight=q.cpu().numpy(), scales=s.cpu().numpy(), cherry_weight=cw.cpu().numpy(),
                cherry_indices=ci.cpu().numpy())


def gpu_unpack(cabi, p, bits, K, G):
    N = p["qweight"].shape[1]
    dense = torch.zeros((N, K), dtype=torch.float16, device="cuda")
    t = [dev(p[k]) for k in ("qweight", "scales", "cherry_weight", "cherry_indices")]
    cabi.check(cabi.lib().cq_unpack_dense(*[ptr(a) for a in t], bits, K, N, len(p["cherry_indices"]), G,
                                          ptr(dense), None), "unpack")
    torch.cuda.synchronize()
    return dense.cpu().numpy()


@pytest.mark.parametrize("name", golden_cases())
def test_gpu_pack_is_bit_exact(cabi, name):
    g = load_golden(name)
    outs = gpu_pack(cabi, g["weight"], g["cherry_unsorted"], g["bits"], g["G"])
    for key in ("qweight", "scales", "cherry_weight", "cherry_indices"):
        assert np.array_equal(outs[key].view(np.uint8), g[key].view(np.uint8)), key


@pytest.mark.parametrize("name", golden_cases())
def test_gpu_unpack_is_bit_exact(cabi, name):
    g = load_golden(name)
    d = gpu_unpack(cabi, g, g["bits"], g["K"], g["G"])
    assert np.array_equal(d.view(np.uint16), g["dense"].view(np.uint16))


@pytest.mark.parametrize("name", golden_cases())
def test_dequantize_normal(cabi, name):
    g = load_golden(name)
    q, sf = dev(g["qweight"]), dev(g["scales"].astype(np.float32))
    Kc = g["K"] - g["C"]
    out = torch.zeros((Kc, g["N"]), dtype=torch.float32, device="cuda")
    fn = cabi.lib().cq_dequantize3_normal if g["bits"] == 3 else cabi.lib().cq_dequantize4_normal
    cabi.check(fn(ptr(q), ptr(sf), ptr(out), q.shape[0], g["N"], g["K"], g["C"], g["G"], None), "dequantize")
    torch.cuda.synchronize()
    ref = O.dequantize_normal(g["qweight"], g["scales"].astype(np.float32), g["bits"], g["G"])
    assert np.array_equal(out.cpu().numpy(), ref)


# ------------------------------------------------------------------ the drop-in module
@pytest.mark.parametrize("name", golden_cases())
def test_quant_cuda_module_matches_reference_call(qc, name):
    """The call llama/qlinear.py:176-181 makes: zero-filled `out`, op accumulates into it."""
    g = load_golden(name)
    x = dev(g["x"])
    t = [dev(g[k]) for k in ("qweight", "cherry_weight", "cherry_indices", "scales")]
    out = torch.zeros(x.shape[0], g["N"], dtype=torch.float16, device="cuda")
    if g["bits"] == 4 and g["G"] >= 128:
        qc.vecquant4matmul_cherryq(x, *t, out, g["G"])
    elif g["bits"] == 3:
        qc.vecquant3matmul_cherryq(x, *t, out, g["G"], True)
    else:
        pytest.skip("the reference has no 4-bit kernel for groups below 128")
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), g["y"].astype(np.float64)) <= TIGHT_TOL
    # second call accumulates on top (mul += ...)
    if g["bits"] == 4:
        qc.vecquant4matmul_cherryq(x, *t, out, g["G"])
    else:
        qc.vecquant3matmul_cherryq(x, *t, out, g["G"], True)
    assert rel_err(out.cpu().numpy(), 2 * g["y"].astype(np.float64)) <= TIGHT_TOL
    qc.poll()


@pytest.mark.parametrize("name", [n for n in golden_cases() if "_b3_" in n])
def test_quant_cuda_fp32_variant(qc, name):
    """vecquant3matmul_cherryq(..., fp16=False): float tensors, int32 indices (benchmark_speed.py:32)."""
    g = load_golden(name)
    x = dev(g["x"].astype(np.float32))
    out = torch.zeros(x.shape[0], g["N"], dtype=torch.float32, device="cuda")
    qc.vecquant3matmul_cherryq(x, dev(g["qweight"]), dev(g["cherry_weight"].astype(np.float32)),
                               dev(g["cherry_indices"].astype(np.int32)), dev(g["scales"].astype(np.float32)),
                               out, g["G"], False)
    ref = O.kernel_forward(g["x"], g["qweight"], g["cherry_weight"], g["cherry_indices"], g["scales"], 3, g["G"])
    assert rel_err(out.cpu().numpy(), ref) <= 1e-5


def test_quant_cuda_error_behaviour(qc):
    g = load_golden("k256_n32_b4_g128_f16")
    x = dev(g["x"])
    t = [dev(g[k]) for k in ("qweight", "cherry_weight", "cherry_indices", "scales")]
    out = torch.zeros(x.shape[0], g["N"], dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 128"):       # csrc/quant_cuda_kernel.cu:684
        qc.vecquant4matmul_cherryq(x, *t, out, 64)
    with pytest.raises(RuntimeError):                                 # wrong dtype
        qc.vecquant4matmul_cherryq(x.float(), *t, out, 128)
    with pytest.raises(RuntimeError):                                 # CPU tensor
        qc.vecquant4matmul_cherryq(x.cpu(), *t, out, 128)
    with pytest.raises(RuntimeError):                                 # 3-bit with an unsupported group size
        qc.vecquant3matmul_cherryq(x, *t, out, 96, True)


# ------------------------------------------------------------------ module level
@pytest.mark.parametrize("name", ["k256_n32_b4_g128_f16", "k256_n40_b3_g64_f16", "k2048_n16_b3_g128_f16"])
def test_quantlinear_module(qc, name):
    import cherryq_b200
    from cherryq_b200.cherry_linear import QuantLinear as TrainLinear
    from cherryq_b200.qlinear import QuantLinear
    g = load_golden(name)
    frac = g["C"] / g["K"]
    tl = TrainLinear(g["K"], g["N"], bias=False, w_bits=g["bits"], group_size=g["G"], cherryq=True, cherry_fraction=frac)
    assert tl.num_cherries == g["C"]
    tl.weight.data = torch.from_numpy(g["weight"].astype(np.float32))
    tl = tl.half().cuda().eval()
    tl.register_cherry_indices(torch.from_numpy(g["cherry_unsorted"]))
    ql = QuantLinear(g["bits"], g["G"], tl.quantizer, frac, g["K"], g["N"], bias=False).cuda()
    ql.pack(tl)
    for key in ("qweight", "scales", "cherry_weight", "cherry_indices"):
        assert np.array_equal(getattr(ql, key).cpu().numpy().view(np.uint8), g[key].view(np.uint8)), key
    assert np.array_equal(ql.unpack().cpu().numpy().view(np.uint16), g["dense"].view(np.uint16))
    x = dev(g["x"]).reshape(1, 5, g["K"])
    y = ql(x)
    assert y.shape == (1, 5, g["N"])
    assert rel_err(y.reshape(5, -1).cpu().numpy(), g["y"].astype(np.float64)) <= TIGHT_TOL
    # fake-quant (training-side) forward: the second oracle
    yf = tl(x.reshape(5, -1)).detach().float().cpu().numpy()
    ref = g["x"].astype(np.float64) @ g["fake"].astype(np.float64).T
    assert rel_err(yf, ref) <= 5e-3
    # keep only the stream copy, then rebuild the reference buffers bit-exactly
    ql.release_reference_buffers()
    y2 = ql(x)
    assert torch.equal(y, y2)
    ql.restore_reference_buffers()
    for key in ("qweight", "scales", "cherry_weight", "cherry_indices"):
        assert np.array_equal(getattr(ql, key).cpu().numpy().view(np.uint8), g[key].view(np.uint8)), key
    # dequantize-once mode (llama/qlinear.py:183-195)
    with QuantLinear.dmode(layerwise_dequantize=False):
        y3 = ql(x)
    assert rel_err(y3.reshape(5, -1).float().cpu().numpy(), g["y"].astype(np.float64)) <= 5e-3


def test_a_wait_that_nothing_satisfies_gives_up_and_reports(cabi):
    """Failure detection without a fault: the bounded wait runs out (about one second), the kernel
    returns, the status word carries the time-out bit, and the context keeps working."""
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.check(cabi.lib().cq_selftest_bounded_wait(ptr(status), None), "selftest")
    torch.cuda.synchronize()
    assert int(status.item()) & 1
    g = load_golden("k256_n32_b4_g128_f16")
    p = Prepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], 4, g["K"], g["G"])
    y = p.matvec(g["x"][:1]).cpu().numpy()
    assert rel_err(y, g["y"][:1].astype(np.float64)) <= TIGHT_TOL
