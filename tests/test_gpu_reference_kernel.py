"""This library's matvec against the REFERENCE PROJECT'S OWN CUDA KERNEL, compiled unmodified by
oracle/build_ref.py into oracle/_ref/ (second oracle; batch 1 only - the reference's batched kernels
re-use shared memory without a barrier - and output widths that are multiples of 128, the only
widths for which its blocks initialise their whole activation slice).  Skipped when the reference
extension has not been built."""
import numpy as np
import pytest

from oracle import build_ref
from oracle import cherryq_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ref = build_ref.load()
    if ref is None:
        pytest.skip("the reference extension is not built (python oracle/build_ref.py)")
    import cherryq_b200
    return ref, cherryq_b200.load_quant_cuda()


@pytest.mark.parametrize("K,N,bits", [(1024, 256, 4), (1024, 256, 3), (4096, 4096, 4), (4096, 4096, 3)])
def test_same_result_as_the_reference_kernel_at_batch_1(mods, K, N, bits):
    ref, qc = mods
    G = 128
    w, idx = O.make_layer(K, N, bits, G, 1 / 256 if K >= 4096 else 1 / 64, K + bits, np.float16)
    p = O.pack(w, idx, bits, G)
    t = [torch.from_numpy(np.ascontiguousarray(p[k])).cuda() for k in ("qweight", "cherry_weight", "cherry_indices", "scales")]
    x = torch.randn(1, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(bits)).half()
    a = torch.zeros(1, N, dtype=torch.float16, device="cuda")
    b = torch.zeros(1, N, dtype=torch.float16, device="cuda")
    if bits == 4:
        ref.vecquant4matmul_cherryq(x, t[0], t[1], t[2], t[3], a, G)
        qc.vecquant4matmul_cherryq(x, t[0], t[1], t[2], t[3], b, G)
    else:
        ref.vecquant3matmul_cherryq(x, t[0], t[1], t[2], t[3], a, G, True)
        qc.vecquant3matmul_cherryq(x, t[0], t[1], t[2], t[3], b, G, True)
    torch.cuda.synchronize()
    qc.poll()
    # the reference adds K/128 + 1 fp16 partial sums per output with fp16 atomics (2^-11 each);
    # this library rounds once.  Both are compared with the fp64 oracle as well.
    exact = torch.from_numpy(O.kernel_forward(x.cpu().numpy(), p["qweight"], p["cherry_weight"], p["cherry_indices"],
                                              p["scales"], bits, G)).cuda()
    scale = float(exact.abs().max())
    err_ref = float((a.double() - exact).abs().max()) / scale
    err_ours = float((b.double() - exact).abs().max()) / scale
    assert err_ours <= 1e-3
    assert err_ref <= 1e-2
    assert float((a.float() - b.float()).abs().max()) / scale <= 1e-2
    assert err_ours <= err_ref + 1e-4          # one rounding instead of dozens of fp16 atomics
