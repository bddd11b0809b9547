"""The numpy oracle against the fixtures frozen from the reference's own code."""
import numpy as np
import pytest

from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O


@pytest.mark.parametrize("name", golden_cases())
def test_pack_matches_reference(name):
    g = load_golden(name)
    p = O.pack(g["weight"], g["cherry_unsorted"], g["bits"], g["G"])
    for key in ("qweight", "scales", "cherry_weight", "cherry_indices"):
        assert p[key].dtype == g[key].dtype
        assert np.array_equal(p[key].view(np.uint8), g[key].view(np.uint8)), key


@pytest.mark.parametrize("name", golden_cases())
def test_unpack_matches_reference(name):
    g = load_golden(name)
    w = O.unpack(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["G"], g["K"])
    assert np.array_equal(w.view(np.uint16), g["dense"].view(np.uint16))


@pytest.mark.parametrize("name", golden_cases())
def test_fake_quant_matches_reference(name):
    g = load_golden(name)
    w = O.fake_quant_weight(g["weight"], g["cherry_unsorted"], g["bits"], g["G"])
    assert w.dtype == g["fake"].dtype
    assert np.array_equal(w, g["fake"])


@pytest.mark.parametrize("name", golden_cases())
def test_forward_matches_reference(name):
    g = load_golden(name)
    y = O.forward_dense_fp64(g["x"], g["dense"])
    assert np.abs(y - g["y"]).max() <= 1e-4 * np.abs(g["y"]).max()
    yk = O.kernel_forward(g["x"], g["qweight"], g["cherry_weight"], g["cherry_indices"], g["scales"], g["bits"], g["G"])
    # the kernel's (u - off) * s in fp32/fp64 differs from unpack()'s fp16-rounded product
    assert np.abs(yk - g["y"]).max() <= 2e-3 * np.abs(g["y"]).max()


@pytest.mark.parametrize("bits", [3, 4])
def test_code_pack_roundtrip_and_bit_order(bits):
    rng = np.random.default_rng(bits)
    u = rng.integers(0, 2 ** bits, size=(64, 8)).astype(np.uint8)
    q = O.pack_codes(u, bits)
    assert q.shape == (64 // 8 * bits, 8)
    assert np.array_equal(O.unpack_codes(q, bits), u)
    # the layout the reference kernels decode (csrc/quant_cuda_kernel.cu:813-829, :650-667)
    if bits == 4:
        assert np.array_equal(q[0], u[0] | (u[1] << 4))
    else:
        w = sum(u[i].astype(np.uint32) << (3 * i) for i in range(8))
        assert np.array_equal(q[0], (w & 0xFF).astype(np.uint8))
        assert np.array_equal(q[1], ((w >> 8) & 0xFF).astype(np.uint8))
        assert np.array_equal(q[2], ((w >> 16) & 0xFF).astype(np.uint8))


def test_compact_to_original_is_the_normal_column_list():
    rng = np.random.default_rng(0)
    for k, c in [(64, 8), (256, 16), (512, 0), (128, 120)]:
        idx = np.sort(rng.permutation(k)[:c]).astype(np.int16)
        cols = O.normal_columns(k, idx)
        got = [O.compact_to_original(i, idx) for i in range(k - c)]
        assert got == list(cols)


def test_dequantize_normal_matches_dense_normal_columns():
    g = load_golden("k384_n16_b4_g256_f16")
    out = O.dequantize_normal(g["qweight"], g["scales"].astype(np.float32), 4, g["G"])
    cols = O.normal_columns(g["K"], g["cherry_indices"])
    ref = g["dense"][:, cols].T.astype(np.float32)
    assert np.abs(out - ref).max() <= 1e-3 * np.abs(ref).max()


def test_num_cherries():
    for k, want in [(4096, 16), (11008, 40), (5120, 16), (13824, 48), (8192, 32), (28672, 112), (256, 0)]:
        assert O.num_cherries(k, 1 / 256) == want


@pytest.mark.parametrize("name", golden_cases())
def test_torch_port_unpack_matches_reference(name):
    import torch
    from oracle import torch_port as TP
    g = load_golden(name)
    dense = TP.unpack(torch.from_numpy(g["qweight"]), torch.from_numpy(g["scales"]), torch.from_numpy(g["cherry_weight"]),
                      torch.from_numpy(g["cherry_indices"]), g["bits"], g["G"], g["K"])
    assert np.array_equal(dense.numpy().view(np.uint16), g["dense"].view(np.uint16))
