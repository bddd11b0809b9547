"""The stream layout + the warp-level walk of it reproduce the oracle (CPU only)."""
import numpy as np
import pytest

import stream_model as SM
from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O


@pytest.mark.parametrize("name", [n for n in golden_cases() if "k2048" not in n])
def test_walk_of_stream_equals_oracle(name):
    g = load_golden(name)
    blob, d = SM.build_blob(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    y = SM.consume_blob(blob, d, g["x"])
    ref = O.kernel_forward(g["x"], g["qweight"], g["cherry_weight"], g["cherry_indices"], g["scales"], g["bits"], g["G"])
    # activations enter as 15-bit integers per granule (step = max|x| / 16256): each product is off
    # by at most 3.1e-5 of the granule's largest activation
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()


def test_dims_of_target_layer():
    d = SM.dims(4, 4096, 11008, 16, 128)
    assert (d["Kc"], d["n_gran"], d["n_sub"], d["gran_bytes"], d["cher_bytes"]) == (4080, 32, 688, 1056, 512)
    d = SM.dims(3, 8192, 28672, 32, 128)
    assert (d["gran_bytes"], d["n_gran"], d["cher_bytes"]) == (800, 64, 1024)
    assert SM.dims(3, 256, 40, 16, 64)["gran_bytes"] == 832


@pytest.mark.parametrize("name", ["k256_n32_b4_g128_f16", "k256_n40_b3_g64_f16", "k384_n16_b4_g256_f16", "k640_n8_b3_g64_f32"])
def test_walk_of_tile_layout_equals_oracle(name):
    g = load_golden(name)
    blob, d = SM.build_tile_blob(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    y = SM.consume_tile_blob(blob, d, g["x"])
    ref = O.kernel_forward(g["x"], g["qweight"], g["cherry_weight"], g["cherry_indices"], g["scales"], g["bits"], g["G"])
    assert np.abs(y - ref).max() <= 1e-6 * np.abs(ref).max()
