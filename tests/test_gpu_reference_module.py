"""The reference project's own `llama/qlinear.py`, unmodified, running on this library's `quant_cuda`
module: its import of `quant_cuda` resolves to the drop-in, `pack()` is the reference's host code,
`forward()` calls the reference-named ops with the reference's argument order.  Needs a checkout of
the reference project ($CHERRYQ_REFERENCE_ROOT or a `reference` directory beside this repository);
skipped where there is none."""
import os
import sys

import numpy as np
import pytest

from oracle import build_ref

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_qlinear():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    root = build_ref.reference_root()
    path = os.path.join(root, "llama", "qlinear.py")
    if not os.path.isfile(path):
        pytest.skip("no checkout of the reference project here")
    import cherryq_b200
    qc = cherryq_b200.load_quant_cuda()
    saved = {k: sys.modules.get(k) for k in ("quant_cuda", "llama", "llama.qlinear", "llama.cherry_linear", "llama.quantizer")}
    for k in saved:
        sys.modules.pop(k, None)
    sys.modules["quant_cuda"] = qc                      # what `import quant_cuda` in the reference file finds
    sys.path.insert(0, root)
    try:
        import llama.cherry_linear as ref_train
        import llama.qlinear as ref_packed
        assert os.path.samefile(ref_packed.__file__, path) and ref_packed.quant_cuda is qc
        yield ref_train, ref_packed
    finally:
        sys.path.remove(root)
        for k, v in saved.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v


@pytest.mark.parametrize("bits,group", [(4, 128), (3, 128), (3, 64)])
@pytest.mark.parametrize("rows", [1, 3, 24])
def test_reference_quantlinear_forward_runs_on_the_drop_in(ref_qlinear, bits, group, rows):
    ref_train, ref_packed = ref_qlinear
    K, N, fraction = 1024, 256, 1 / 64
    torch.manual_seed(bits * 100 + group + rows)
    train = ref_train.QuantLinear(K, N, w_bits=bits, group_size=group, cherryq=True, cherry_fraction=fraction,
                                      bias=False).half()
    train.register_cherry_indices(torch.randperm(K)[:train.num_cherries].to(torch.int32))
    ref = ref_packed.QuantLinear(bits, group, train.quantizer, fraction, K, N, bias=False)
    ref.pack(train)                                      # the reference's own host-side pack
    ref = ref.cuda()
    x = torch.randn(rows, K, device="cuda").half()
    y = ref(x)                                           # reference forward -> quant_cuda.vecquant{3,4}matmul_cherryq
    dense = ref.unpack().float()                         # reference unpack, (N, K)
    want = x.float() @ dense.T
    err = float((y.float() - want).abs().max() / want.abs().max())
    assert y.shape == (rows, N) and y.dtype == torch.float16
    assert err <= 1e-2, err
