"""GPU parity tests of the prefill GEMM (tcgen05 tensor cores, weights dequantised into tensor
memory) through the C ABI and through the drop-in `quant_cuda` ops, against the reference's dense
mode: x . unpack()^T with the fp16 weights of `unpack()` (golden fixtures / numpy oracle)."""
import ctypes as C

import numpy as np
import pytest

from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O
from test_gpu_parity import Prepared, dev, make_case, ptr, rel_err
from test_gpu_tile import TilePrepared

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

# fp16 inputs, exact fp16 weights of unpack(), fp32 accumulation in the tensor core, one fp16 store:
# the error against the fp64 product is the store's rounding (2^-11 relative per element)
GEMM_TOL = 1e-3


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


def gemm(cabi, p, x, y=None, accumulate=False):
    lib = cabi.lib()
    xd = dev(x) if isinstance(x, np.ndarray) else x
    M = xd.shape[0]
    ws = torch.empty(lib.cq_tlayer_gemm_workspace_bytes(C.byref(p.L), M), dtype=torch.uint8, device="cuda")
    if y is None:
        y = torch.full((M, p.L.N), float("nan"), dtype=torch.float16, device="cuda")
    cabi.check(lib.cq_tlayer_gemm(C.byref(p.L), ptr(xd), p.L.K, ptr(y), p.L.N, M, int(accumulate), ptr(ws),
                                  ptr(p.status), None), "gemm")
    torch.cuda.synchronize()
    assert int(p.status.item()) == 0, f"a device-side wait timed out (status {int(p.status.item())})"
    return y


@pytest.mark.parametrize("name", golden_cases())
@pytest.mark.parametrize("M", [32, 45, 130])
def test_gemm_on_golden_layers(cabi, name, M):
    g = load_golden(name)
    p = TilePrepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    x = np.random.default_rng(M).normal(size=(M, int(g["K"]))).astype(np.float16)
    y = gemm(cabi, p, x).cpu().numpy()
    assert np.isfinite(y).all()
    ref = x.astype(np.float64) @ g["dense"].astype(np.float64).T          # dense = the reference's unpack()
    assert rel_err(y, ref) <= GEMM_TOL
    y2 = gemm(cabi, p, x).cpu().numpy()
    assert np.array_equal(y.view(np.uint16), y2.view(np.uint16))


@pytest.mark.parametrize("K,N,bits,M", [(4096, 11008, 4, 256), (4096, 11008, 3, 200), (11008, 4096, 4, 128),
                                         (4096, 4096, 3, 33), (4096, 4096, 4, 520)])
def test_gemm_llama7b_shapes(cabi, K, N, bits, M):
    w, idx, pk, dense = make_case(K, N, bits, 128, seed=K + N + bits)
    p = TilePrepared(cabi, pk["qweight"], pk["scales"], pk["cherry_weight"], pk["cherry_indices"], bits, K, 128)
    x = torch.randn(M, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).half()
    y = gemm(cabi, p, x)
    ref = x.float() @ dev(dense).float().T                                 # fp32 matmul of the dequantised weights
    err = float((y.float() - ref).abs().max() / ref.abs().max())
    assert err <= 2e-3, err


@pytest.mark.parametrize("K,N,bits,G,frac,M", [
    (256, 24, 4, 128, 1 / 16, 40),       # N not a multiple of 16, one row tile mostly empty
    (640, 136, 3, 64, 1 / 32, 64),       # 64-wide groups, two row tiles, second one 8 rows
    (384, 16, 4, -1, 1 / 24, 32),        # one group per row
    (1024, 264, 3, 128, 0.0, 100),       # no cherries
    (512, 128, 4, 256, 0.25, 129),       # 128 cherry columns = 8 cherry items
])
def test_gemm_edge_shapes(cabi, K, N, bits, G, frac, M):
    w, idx = O.make_layer(K, N, bits, K if G == -1 else G, frac, 3, np.float16)
    pk = O.pack(w, idx, bits, K if G == -1 else G)
    dense = O.unpack(pk["qweight"], pk["scales"], pk["cherry_weight"], pk["cherry_indices"], bits, K if G == -1 else G, K)
    p = TilePrepared(cabi, pk["qweight"], pk["scales"], pk["cherry_weight"], pk["cherry_indices"], bits, K, G)
    x = np.random.default_rng(7).normal(size=(M, K)).astype(np.float16)
    y = gemm(cabi, p, x).cpu().numpy()
    ref = x.astype(np.float64) @ dense.astype(np.float64).T
    assert rel_err(y, ref) <= GEMM_TOL


def test_gemm_accumulates_like_the_reference(cabi):
    g = load_golden("k256_n32_b4_g128_f16")
    p = TilePrepared(cabi, g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], 4, g["K"], g["G"])
    rng = np.random.default_rng(0)
    x = rng.normal(size=(48, int(g["K"]))).astype(np.float16)
    base = rng.normal(size=(48, int(g["N"]))).astype(np.float16)
    y = gemm(cabi, p, x, y=dev(base.copy()), accumulate=True).cpu().numpy()
    ref = x.astype(np.float64) @ g["dense"].astype(np.float64).T + base.astype(np.float64)
    assert rel_err(y, ref) <= GEMM_TOL


def test_gemm_equals_the_matvec_path(cabi):
    """The same layer and activations through the decode kernel (16 rows at a time) and the GEMM."""
    w, idx, pk, dense = make_case(2048, 512, 4, 128, seed=9)
    p = TilePrepared(cabi, pk["qweight"], pk["scales"], pk["cherry_weight"], pk["cherry_indices"], 4, 2048, 128)
    x = np.random.default_rng(2).normal(size=(64, 2048)).astype(np.float16)
    a = gemm(cabi, p, x).float()
    b = Prepared(cabi, pk["qweight"], pk["scales"], pk["cherry_weight"], pk["cherry_indices"], 4, 2048, 128).matvec(x).float()
    assert float((a - b).abs().max() / b.abs().max()) <= 2e-3


@pytest.mark.parametrize("bits", [4, 3])
def test_quant_cuda_ops_route_large_batches_to_the_gemm(qc, bits):
    K, N, G, M = 1024, 384, 128, 96
    w, idx, pk, dense = make_case(K, N, bits, G, seed=bits)
    t = [dev(pk[k]) for k in ("qweight", "cherry_weight", "cherry_indices", "scales")]
    x = torch.randn(M, K, device="cuda").half()
    base = torch.randn(M, N, device="cuda").half()
    out = base.clone()
    if bits == 4:
        qc.vecquant4matmul_cherryq(x, t[0], t[1], t[2], t[3], out, G)
    else:
        qc.vecquant3matmul_cherryq(x, t[0], t[1], t[2], t[3], out, G, True)
    torch.cuda.synchronize()
    qc.poll()
    ref = x.float() @ dev(dense).float().T + base.float()
    assert float((out.float() - ref).abs().max() / ref.abs().max()) <= 2e-3
    # the decode path on a slice of the same rows agrees
    out2 = base[:8].clone()
    if bits == 4:
        qc.vecquant4matmul_cherryq(x[:8].contiguous(), t[0], t[1], t[2], t[3], out2, G)
    else:
        qc.vecquant3matmul_cherryq(x[:8].contiguous(), t[0], t[1], t[2], t[3], out2, G, True)
    torch.cuda.synchronize()
    assert float((out2.float() - out[:8].float()).abs().max() / ref.abs().max()) <= 2e-3
