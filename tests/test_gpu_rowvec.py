"""GPU parity of the one-row decode kernel (cq_rlayer_*), all through the C ABI (ctypes, raw device
pointers): re-pack against the numpy layout model and back, matvec against the fp64 dequantised
matmul of the oracle, on the golden fixtures, the LLaMA 7B / 13B / 70B shapes, edge shapes and
heavy-tailed activations."""
import ctypes as C
import math

import numpy as np
import pytest

import rowtile_model as RM
from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-2     # north-star bound: max |y - y_ref| / max |y_ref| against the fp64 dequantised matmul
TIGHT_TOL = 2e-3   # what exact integer sums + fp32 scaling + one fp16 store actually deliver


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


def rel_err(y, ref):
    return float(np.abs(np.asarray(y, dtype=np.float64) - ref).max() / np.abs(ref).max())


class RowPrepared:
    """A layer in the row-tile layout, prepared through the C ABI from reference-format buffers (device tensors)."""

    def __init__(self, cabi, q, s, cw, ci, bits, K, G):
        self.cabi, self.t = cabi, [q, s, cw, ci]
        self.L = cabi.rlayer_init(bits, K, q.shape[1], ci.shape[0], G)
        self.check = cabi.lib().cq_rlayer_check(C.byref(self.L))
        self.blob = torch.zeros(self.L.blob_bytes, dtype=torch.uint8, device="cuda")
        self.L.blob = self.blob.data_ptr()
        cabi.check(cabi.lib().cq_rlayer_prepare(C.byref(self.L), *[ptr(t) for t in self.t], None), "prepare")
        torch.cuda.synchronize()
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def matvec(self, x, y=None, accumulate=False):
        if y is None:
            y = torch.full((1, self.L.N), float("nan"), dtype=torch.float16, device="cuda")
        self.cabi.check(self.cabi.lib().cq_rlayer_matvec(C.byref(self.L), ptr(x), ptr(y), int(accumulate),
                                                         ptr(self.status), None), "matvec")
        torch.cuda.synchronize()
        assert int(self.status.item()) == 0, "a device-side wait timed out"
        return y

    def unprepare(self):
        outs = [torch.zeros_like(t) for t in self.t]
        self.cabi.check(self.cabi.lib().cq_rlayer_unprepare(C.byref(self.L), *[ptr(t) for t in outs], None), "unprepare")
        torch.cuda.synchronize()
        return outs


def golden_prepared(cabi, g):
    return RowPrepared(cabi, dev(g["qweight"]), dev(g["scales"]), dev(g["cherry_weight"]), dev(g["cherry_indices"]),
                       g["bits"], g["K"], g["G"])


# ------------------------------------------------------------------ re-pack
@pytest.mark.parametrize("name", golden_cases())
def test_prepare_matches_layout_model_and_roundtrips(cabi, name):
    g = load_golden(name)
    p = golden_prepared(cabi, g)
    model, d = RM.build_blob(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    got = p.blob.cpu().numpy()
    assert d["blob_bytes"] == p.L.blob_bytes
    for sec, nbytes in (("off_tiles", d["NT"] * d["tile_bytes"]), ("off_perm", d["NG"] * 256), ("off_cidx", d["Cp"] * 2)):
        o = d[sec]
        assert np.array_equal(got[o:o + nbytes], model[o:o + nbytes]), sec
    for a, b in zip(p.unprepare(), p.t):
        assert torch.equal(a, b)


# ------------------------------------------------------------------ matvec on the golden layers
@pytest.mark.parametrize("name", golden_cases())
def test_matvec_golden(cabi, name):
    g = load_golden(name)
    p = golden_prepared(cabi, g)
    assert p.check == 0
    for row in range(3):
        x = dev(g["x"][row:row + 1])
        y = p.matvec(x).cpu().numpy()
        assert np.isfinite(y).all()
        assert rel_err(y, g["y"][row:row + 1].astype(np.float64)) <= TIGHT_TOL
        ref = O.kernel_forward(g["x"][row:row + 1], g["qweight"], g["cherry_weight"], g["cherry_indices"], g["scales"],
                               g["bits"], g["G"])
        assert rel_err(y, ref) <= 1e-3
        # bit-identical on a second run (fixed summation order, no atomics)
        y2 = p.matvec(x).cpu().numpy()
        assert np.array_equal(y.view(np.uint16), y2.view(np.uint16))


def test_matvec_accumulates_like_the_reference(cabi):
    g = load_golden("k256_n32_b4_g128_f16")
    p = golden_prepared(cabi, g)
    base = np.random.default_rng(0).normal(size=(1, g["N"])).astype(np.float16)
    y = p.matvec(dev(g["x"][:1]), y=dev(base.copy()), accumulate=True).cpu().numpy()
    assert rel_err(y, g["y"][:1].astype(np.float64) + base.astype(np.float64)) <= TIGHT_TOL


def test_unaligned_activation_pointer(cabi):
    """x that is only 2-byte aligned takes the kernel's scalar staging path."""
    g = load_golden("k2048_n16_b4_g128_f16")
    p = golden_prepared(cabi, g)
    buf = torch.zeros(g["K"] + 8, dtype=torch.float16, device="cuda")
    buf[1:1 + g["K"]] = dev(g["x"][0])
    y = p.matvec(buf[1:1 + g["K"]]).cpu().numpy()
    assert rel_err(y, g["y"][:1].astype(np.float64)) <= TIGHT_TOL


# ------------------------------------------------------------------ model shapes
def gpu_layer(K, N, bits, G, seed, frac=1 / 256):
    """Synthetic layer with the configurations' distributions, packed by the GPU pack kernel (byte-identical to
    the oracle's pack, tests/test_gpu_parity.py) and unpacked by the GPU dense unpack (byte-identical to the
    oracle's unpack, same file): the fp64 reference of the big shapes is x . dense^T computed by torch in fp64."""
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    g = torch.Generator(device="cuda").manual_seed(seed)
    c = math.ceil(K * frac) // 8 * 8
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    idx = torch.randperm(K, device="cuda", generator=g)[:c].to(torch.int32)
    if c:
        w[:, idx.long()] = torch.randn(N, c, device="cuda", generator=g) * 0.2
    q, s, cw, ci = qc.pack(w.half().contiguous(), idx.contiguous(), bits, G)
    dense = qc.unpack_dense(q, s, cw, ci, bits, K, G)
    return q, s, cw, ci, dense


def ref64(x, dense):
    return (x.double() @ dense.double().T).cpu().numpy()


MODEL_SHAPES = [
    (4096, 4096, 4), (4096, 11008, 4), (11008, 4096, 4), (4096, 4096, 3), (4096, 11008, 3), (11008, 4096, 3),   # 7B
    (5120, 5120, 3), (5120, 13824, 3), (13824, 5120, 3),                                                       # 13B, C = 16 / 48
    (8192, 8192, 3), (8192, 1024, 3), (8192, 28672, 3), (28672, 8192, 3),                                      # 70B, C = 32 / 112
]


@pytest.mark.parametrize("K,N,bits", MODEL_SHAPES)
def test_matvec_model_shapes(cabi, K, N, bits):
    q, s, cw, ci, dense = gpu_layer(K, N, bits, 128, seed=K + N + bits)
    p = RowPrepared(cabi, q, s, cw, ci, bits, K, 128)
    assert p.check == 0
    g = torch.Generator(device="cuda").manual_seed(5)
    for _ in range(2):
        x = torch.randn(1, K, device="cuda", generator=g).half()
        assert rel_err(p.matvec(x).cpu().numpy(), ref64(x, dense)) <= TIGHT_TOL, (K, N, bits)
    for a, b in zip(p.unprepare(), p.t):
        assert torch.equal(a, b)


def test_layers_outside_the_envelope_are_refused_and_the_op_falls_back(cabi):
    """256 cherry columns (cherry ratio 1/16 of 4096) are more than a warp's slice of the activations holds:
    the C ABI says so and the drop-in op serves the call with the stream kernel."""
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    K, N = 4096, 1024
    q, s, cw, ci, dense = gpu_layer(K, N, 3, 128, seed=9, frac=1 / 16)
    assert ci.shape[0] == 256
    L = cabi.rlayer_init(3, K, N, ci.shape[0], 128)
    assert cabi.lib().cq_rlayer_check(C.byref(L)) == 9          # CQ_ERR_UNSUPPORTED
    assert cabi.lib().cq_rlayer_matvec(C.byref(L), ptr(q), ptr(q), 0, None, None) in (1, 9)   # no blob / unsupported
    for M in (1, 5):
        x = torch.randn(M, K, device="cuda").half()
        out = torch.zeros(M, N, dtype=torch.float16, device="cuda")
        qc.vecquant3matmul_cherryq(x, q, cw, ci, s, out, 128, True)
        torch.cuda.synchronize()
        assert rel_err(out.cpu().numpy(), ref64(x, dense)) <= TIGHT_TOL


@pytest.mark.parametrize("K,N,bits,G,frac", [
    (256, 8, 4, 128, 1 / 16),         # one tile, half of it padding rows
    (136, 24, 3, 128, 1 / 17),        # K' = 128 exactly after 8 cherries
    (264, 40, 4, 128, 1 / 33),        # K' = 256, N not a multiple of 16
    (1024, 4744, 4, 128, 1 / 64),     # more tiles than SMs, ragged last tile
    (2048, 512, 3, 64, 1 / 256),      # 64-wide groups
    (2048, 512, 4, 2048, 1 / 256),    # one group per row
    (2048, 512, 4, -1, 1 / 256),      # group_size -1 = whole row
    (512, 64, 4, 128, 0.0),           # no cherries at all
    (4096, 256, 4, 128, 112 / 4096),  # 112 cherry columns: seven cherry blocks
    (8192 + 32, 64, 3, 128, 1 / 256), # 64 groups exactly: the widest layer one CTA per tile takes
    (8192 + 160, 64, 4, 128, 1 / 256),# 65 groups: two CTAs per tile, 33 + 32 groups
    (12288, 64, 3, 128, 1 / 256),     # 96 groups: two CTAs per tile
    (16384 + 200, 48, 4, 128, 1 / 256),   # 130 groups: three CTAs per tile (44 + 44 + 42), ragged last group
    (28672, 72, 3, 64, 1 / 256),      # 224 groups of two scale sets: four CTAs per tile
    (32760, 16, 4, 128, 1 / 512),     # the widest row whose cherry columns fit the format's int16 indices (256 groups)
])
def test_matvec_edge_shapes(cabi, K, N, bits, G, frac):
    q, s, cw, ci, dense = gpu_layer(K, N, bits, G if G != -1 else K, seed=K * 7 + N, frac=frac)
    p = RowPrepared(cabi, q, s, cw, ci, bits, K, G)
    assert p.check == 0
    x = torch.randn(1, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).half()
    assert rel_err(p.matvec(x).cpu().numpy(), ref64(x, dense)) <= TIGHT_TOL
    for a, b in zip(p.unprepare(), p.t):
        assert torch.equal(a, b)


def test_linearity_zero_and_unit_vectors_at_full_size(cabi):
    """Size-independent properties on the north-star layer (4096 -> 11008, 4-bit)."""
    K, N = 4096, 11008
    q, s, cw, ci, dense = gpu_layer(K, N, 4, 128, seed=0)
    p = RowPrepared(cabi, q, s, cw, ci, 4, K, 128)
    x1 = torch.randn(1, K, device="cuda").half()
    assert torch.count_nonzero(p.matvec(torch.zeros_like(x1))) == 0
    y1 = p.matvec(x1).float()
    y2 = p.matvec((x1 * 2).half()).float()
    assert float((y2 - 2 * y1).abs().max() / y2.abs().max()) <= 2e-3
    for col in (0, int(ci[0]), 4095, 1234):
        e = torch.zeros(1, K, dtype=torch.float16, device="cuda")
        e[0, col] = 1.0
        y = p.matvec(e)[0].float()
        assert float((y - dense[:, col].float()).abs().max()) <= 1e-3 * float(dense[:, col].float().abs().max())


# ------------------------------------------------------------------ heavy-tailed activations
def elementwise_error(y, ref, floor_frac=1e-2):
    """max over elements of |y - ref| / max(|ref|, floor) with floor = floor_frac * rms(ref)."""
    floor = floor_frac * float(np.sqrt(np.mean(ref ** 2)))
    return float((np.abs(np.asarray(y, dtype=np.float64) - ref) / np.maximum(np.abs(ref), floor)).max())


@pytest.mark.parametrize("bits", [4, 3])
@pytest.mark.parametrize("scale", [100.0, 1000.0])
def test_outlier_channels(cabi, bits, scale):
    """LLaMA activations have a few channels 100-1000 times larger than the rest.  The kernel quantises every
    128-column group of x to 15 bits relative to the group's largest magnitude, so an outlier costs its 127
    group mates precision: with a 100 sigma outlier the step is 0.006 sigma, the 127 mates carry an rms
    error of 0.0018 sigma each, i.e. about 3e-4 of a typical |y| per output.  The max-norm bound must hold
    with room; element-wise, relative to max(|ref|, floor), the error is asserted for two floors (10 % and
    1 % of rms(ref)): outputs that happen to be near zero see the absolute error of their neighbours, as they
    do with the reference's fp16 atomic accumulation."""
    K, N = 4096, 11008
    q, s, cw, ci, dense = gpu_layer(K, N, bits, 128, seed=77 + bits)
    p = RowPrepared(cabi, q, s, cw, ci, bits, K, 128)
    g = torch.Generator(device="cuda").manual_seed(3)
    cherry = int(ci[3])
    normal = [c for c in range(K) if c not in set(ci.cpu().numpy().tolist())]
    cases = {
        "inside a group": [normal[700]],
        "on a group boundary": [normal[127], normal[128]],
        "on a cherry column": [cherry],
        "four channels": [normal[5], normal[1500], normal[2047], normal[4000]],
    }
    for where, cols in cases.items():
        x = torch.randn(1, K, device="cuda", generator=g)
        x[0, cols] *= scale
        x = x.half()
        ref = ref64(x, dense)
        y = p.matvec(x).cpu().numpy()
        assert rel_err(y, ref) <= TIGHT_TOL, (where, scale, bits)
        e10, e1 = elementwise_error(y, ref, 0.1), elementwise_error(y, ref, 0.01)
        assert e10 <= 2e-2 and e1 <= 2e-1, (where, scale, bits, e10, e1)


# ------------------------------------------------------------------ several layers in one launch
@pytest.mark.parametrize("K,Ns,bits,G", [
    (4096, (4096, 4096, 4096), 4, 128),          # 7B q / k / v
    (4096, (11008, 11008), 4, 128),              # 7B gate / up
    (8192, (8192, 1024, 1024), 3, 128),          # 70B q / k / v (grouped-query heads: small k, v)
    (5120, (13824, 13824), 3, 128),              # 13B gate / up
    (11008, (4096, 512), 4, 128),                # two wide layers (two CTAs per tile each)
    (1024, (48, 16, 8, 200), 3, 64),             # four small ragged layers, fewer tiles than SMs
    (2048, (4096, 24), 4, 128),                  # very uneven
])
def test_shared_input_launch_is_bit_identical_to_separate_launches(cabi, K, Ns, bits, G):
    lib = cabi.lib()
    frac = 1 / 256 if K >= 2048 else 1 / 64
    preps = []
    for i, N in enumerate(Ns):
        q, s, cw, ci, _ = gpu_layer(K, N, bits, G, seed=K + N + bits + 17 * i, frac=frac)
        preps.append(RowPrepared(cabi, q, s, cw, ci, bits, K, G))
    x = torch.randn(1, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(K)).half()
    want = [p.matvec(x) for p in preps]
    outs = [torch.full((1, N), float("nan"), dtype=torch.float16, device="cuda") for N in Ns]
    n = len(Ns)
    layers = (C.POINTER(cabi.cq_rlayer) * n)(*[C.pointer(p.L) for p in preps])
    ys = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.check(lib.cq_rlayers_matvec(layers, n, ptr(x), K, ys, max(Ns), 1, 0, ptr(status), None), "rlayers_matvec")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for o, w in zip(outs, want):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16))
    # accumulate adds to what the outputs hold
    cabi.check(lib.cq_rlayers_matvec(layers, n, ptr(x), K, ys, max(Ns), 1, 1, ptr(status), None), "rlayers_matvec")
    torch.cuda.synchronize()
    for o, p, w in zip(outs, preps, want):
        again = p.matvec(x, y=w.clone(), accumulate=True)
        assert torch.equal(o.view(torch.int16), again.view(torch.int16))


def test_shared_input_launch_refuses_layers_that_do_not_agree(cabi):
    lib = cabi.lib()
    a = RowPrepared(cabi, *gpu_layer(1024, 64, 4, 128, seed=1)[:4], 4, 1024, 128)
    b = RowPrepared(cabi, *gpu_layer(2048, 64, 4, 128, seed=2)[:4], 4, 2048, 128)
    c = RowPrepared(cabi, *gpu_layer(1024, 64, 3, 128, seed=3)[:4], 3, 1024, 128)
    x = torch.zeros(1, 2048, dtype=torch.float16, device="cuda")
    outs = [torch.zeros(1, 64, dtype=torch.float16, device="cuda") for _ in range(2)]
    ys = (C.c_void_p * 2)(*[o.data_ptr() for o in outs])
    for pair in ((a, b), (a, c)):
        layers = (C.POINTER(cabi.cq_rlayer) * 2)(*[C.pointer(p.L) for p in pair])
        assert lib.cq_rlayers_matvec(layers, 2, ptr(x), 2048, ys, 64, 1, 0, None, None) == 4     # CQ_ERR_BAD_SHAPE
    layers = (C.POINTER(cabi.cq_rlayer) * 2)(C.pointer(a.L), C.pointer(a.L))
    assert lib.cq_rlayers_matvec(layers, 5, ptr(x), 2048, ys, 64, 1, 0, None, None) == 1         # more than four layers
    assert lib.cq_rlayers_matvec(layers, 0, ptr(x), 2048, ys, 64, 1, 0, None, None) == 1
    assert lib.cq_rlayers_matvec(layers, 2, ptr(x), 1000, ys, 64, 1, 0, None, None) == 1         # ldx < K
    assert lib.cq_rlayers_matvec(layers, 2, ptr(x), 2048, ys, 32, 1, 0, None, None) == 1         # ldy < N
    assert lib.cq_rlayers_matvec(layers, 2, ptr(x), 2048, ys, 64, 0, 0, None, None) == 1         # no rows


def test_quantlinear_shared_input_forward_matches_separate_forwards():
    import cherryq_b200
    from cherryq_b200.qlinear import QuantLinear, forward_shared_input
    qc = cherryq_b200.load_quant_cuda()
    K = 2048
    lins = []
    for i, N in enumerate((512, 128, 128)):
        q, s, cw, ci, _ = gpu_layer(K, N, 4, 128, seed=40 + i)
        lin = QuantLinear(4, 128, None, 1 / 256, K, N, bias=(i == 1)).cuda()
        lin.qweight, lin.scales, lin.cherry_weight, lin.cherry_indices = q, s, cw, ci
        if lin.bias is not None:
            lin.bias = torch.randn(N, device="cuda").half()
        lins.append(lin)
    for rows in (1, 3, 4, 7, 8, 12):
        x = torch.randn(rows, K, device="cuda").half()
        together = forward_shared_input(lins, x)
        for lin, y in zip(lins, together):
            assert torch.equal(y, lin(x))


def test_host_buffer_entry_point(cabi):
    """cq_rlayer_matvec_host: activations from host memory, the output back in host memory when the call returns."""
    lib = cabi.lib()
    K, N = 4096, 4096
    q, s, cw, ci, dense = gpu_layer(K, N, 4, 128, seed=77)
    p = RowPrepared(cabi, q, s, cw, ci, 4, K, 128)
    xh = torch.randn(1, K).half().pin_memory()
    yh = torch.zeros(1, N, dtype=torch.float16).pin_memory()
    xd = torch.empty(1, K, dtype=torch.float16, device="cuda")
    yd = torch.empty(1, N, dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    for _ in range(2):
        yh.zero_()
        cabi.check(lib.cq_rlayer_matvec_host(C.byref(p.L), C.c_void_p(xh.data_ptr()), C.c_void_p(yh.data_ptr()), ptr(xd), ptr(yd),
                                             ptr(status), C.c_void_p(stream.cuda_stream)), "matvec_host")
        want = p.matvec(xh.cuda())            # no synchronisation between the call above and this read of yh is needed
        assert torch.equal(yh, want.cpu())
    assert int(status.item()) == 0
    # pageable host memory works too (the copies are then staged by the driver)
    xp, yp = xh.clone(), torch.zeros(1, N, dtype=torch.float16)
    cabi.check(lib.cq_rlayer_matvec_host(C.byref(p.L), C.c_void_p(xp.data_ptr()), C.c_void_p(yp.data_ptr()), ptr(xd), ptr(yd),
                                         ptr(status), None), "matvec_host")
    assert torch.equal(yp, want.cpu())


# ------------------------------------------------------------------ several activation rows in one launch
def rows_call(cabi, preps, x, ldx=None, pad=0, accumulate=False, base=None):
    """cq_rlayers_matvec on M rows; the outputs are column slices of one (M, sum N + pad) buffer."""
    lib = cabi.lib()
    M, K = x.shape[0], preps[0].L.K
    widths = [p.L.N for p in preps]
    ldy = sum(widths) + pad
    buf = torch.full((M, ldy), float("nan"), dtype=torch.float16, device="cuda") if base is None else base.clone()
    outs = list(buf[:, :sum(widths)].split(widths, dim=1))
    n = len(preps)
    layers = (C.POINTER(cabi.cq_rlayer) * n)(*[C.pointer(p.L) for p in preps])
    ys = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.check(lib.cq_rlayers_matvec(layers, n, ptr(x), ldx or x.stride(0), ys, ldy, M, int(accumulate), ptr(status), None),
               "rlayers_matvec")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return buf, outs


@pytest.mark.parametrize("K,N,bits,G", [(4096, 4096, 4, 128), (4096, 11008, 3, 128), (11008, 4096, 4, 128),
                                        (13824, 5120, 3, 128), (8192, 1024, 3, 128), (1024, 200, 3, 64),
                                        (640, 40, 4, 640), (28672, 1024, 3, 128)])
@pytest.mark.parametrize("M", [2, 3, 4, 5, 8, 11])
def test_rows_of_a_batch_are_bit_identical_to_single_row_calls(cabi, K, N, bits, G, M):
    frac = 1 / 256 if K >= 2048 else 1 / 64
    q, s, cw, ci, dense = gpu_layer(K, N, bits, G, seed=K + N + bits + M, frac=frac)
    p = RowPrepared(cabi, q, s, cw, ci, bits, K, G)
    g = torch.Generator(device="cuda").manual_seed(M)
    x = (torch.randn(M, K, device="cuda", generator=g) * torch.logspace(-2, 1, M, device="cuda")[:, None]).half()
    buf, (y,) = rows_call(cabi, [p], x)
    for m in range(M):
        want = p.matvec(x[m:m + 1].contiguous())
        assert torch.equal(y[m:m + 1].contiguous().view(torch.int16), want.view(torch.int16)), m
    assert rel_err(y.float().cpu().numpy(), ref64(x, dense)) <= TIGHT_TOL


def test_batch_with_strides_padding_accumulate_and_shared_input(cabi):
    K, Ns, bits = 2048, (512, 128, 136), 4
    preps = []
    for i, N in enumerate(Ns):
        q, s, cw, ci, _ = gpu_layer(K, N, bits, 128, seed=900 + i)
        preps.append(RowPrepared(cabi, q, s, cw, ci, bits, K, 128))
    M = 6
    wide = torch.randn(M, K + 24, device="cuda").half()
    x = wide[:, 8:8 + K]                                     # row stride K + 24, rows 16-byte aligned
    buf, outs = rows_call(cabi, preps, x, pad=5)
    assert bool(torch.isnan(buf[:, sum(Ns):]).all())          # the padding columns are not written
    for p, o in zip(preps, outs):
        for m in range(M):
            want = p.matvec(x[m:m + 1].contiguous())
            assert torch.equal(o[m:m + 1].contiguous().view(torch.int16), want.view(torch.int16))
    odd = wide[:, 3:3 + K]                                   # rows only 2-byte aligned: scalar staging path
    _, outs2 = rows_call(cabi, preps, odd)
    for p, o in zip(preps, outs2):
        want = torch.cat([p.matvec(odd[m:m + 1].contiguous()) for m in range(M)])
        assert torch.equal(o.contiguous().view(torch.int16), want.view(torch.int16))
    base = torch.randn(M, sum(Ns), device="cuda").half()
    acc, outs3 = rows_call(cabi, preps, x, accumulate=True, base=base)
    col = 0
    for p, o in zip(preps, outs3):
        for m in range(M):
            want = p.matvec(x[m:m + 1].contiguous(), y=base[m:m + 1, col:col + p.L.N].contiguous(), accumulate=True)
            assert torch.equal(o[m:m + 1].contiguous().view(torch.int16), want.view(torch.int16))
        col += p.L.N


@pytest.mark.parametrize("bits", [4, 3])
@pytest.mark.parametrize("M", [2, 4, 7, 8])
def test_drop_in_ops_route_decode_batches_to_the_row_kernel(bits, M):
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    K, N = 4096, 1024
    q, s, cw, ci, dense = gpu_layer(K, N, bits, 128, seed=bits * 10 + M)
    x = torch.randn(M, K, device="cuda").half()
    base = torch.randn(M, N, device="cuda").half()
    out = base.clone()
    if bits == 4:
        qc.vecquant4matmul_cherryq(x, q, cw, ci, s, out, 128)
    else:
        qc.vecquant3matmul_cherryq(x, q, cw, ci, s, out, 128, True)
    torch.cuda.synchronize()
    ref = base.double().cpu().numpy() + ref64(x, dense)
    assert rel_err(out.float().cpu().numpy(), ref) <= TIGHT_TOL


@pytest.mark.parametrize("K,N,bits,M", [(11008, 4096, 4, 1), (11008, 4096, 3, 4), (4096, 512, 4, 3), (28672, 1024, 3, 1),
                                        (2048, 264, 4, 6)])
def test_swiglu_folded_into_the_down_projection(cabi, K, N, bits, M):
    """cq_rlayer_matvec_swiglu against the element-wise kernel followed by the plain call: bit-identical."""
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    q, s, cw, ci, dense = gpu_layer(K, N, bits, 128, seed=K + N + M)
    p = RowPrepared(cabi, q, s, cw, ci, bits, K, 128)
    g = torch.Generator(device="cuda").manual_seed(M)
    gate = (torch.randn(M, K, device="cuda", generator=g) * 2).half()
    up = torch.randn(M, K, device="cuda", generator=g).half()
    act = qc.silu_mul(gate, up)
    _, (want,) = rows_call(cabi, [p], act)
    y = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    cabi.check(cabi.lib().cq_rlayer_matvec_swiglu(C.byref(p.L), ptr(gate), ptr(up), K, ptr(y), N, M, ptr(status), None), "swiglu")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(y.view(torch.int16), want.contiguous().view(torch.int16))
    ref = ref64(torch.nn.functional.silu(gate.float()).half() * up, dense)
    assert rel_err(y.float().cpu().numpy(), ref) <= TIGHT_TOL
    # unaligned rows take the scalar staging path
    wide_g = torch.zeros(M, K + 8, dtype=torch.float16, device="cuda")
    wide_u = torch.zeros(M, K + 8, dtype=torch.float16, device="cuda")
    wide_g[:, 1:1 + K], wide_u[:, 1:1 + K] = gate, up
    y2 = torch.zeros_like(y)
    cabi.check(cabi.lib().cq_rlayer_matvec_swiglu(C.byref(p.L), ptr(wide_g[:, 1:]), ptr(wide_u[:, 1:]), K + 8, ptr(y2), N, M,
                                                  ptr(status), None), "swiglu")
    torch.cuda.synchronize()
    assert torch.equal(y2, y)
