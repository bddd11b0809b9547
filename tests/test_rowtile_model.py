"""CPU checks of the row-tile layout model against the oracle and the library's host-side planner."""
import numpy as np
import pytest

import rowtile_model as RM
from conftest import golden_cases, load_golden
from oracle import cherryq_oracle as O


@pytest.mark.parametrize("name", golden_cases())
def test_model_round_trip(name):
    """Codes written by the layout model and read back with the kernel's masks are the oracle's codes."""
    g = load_golden(name)
    blob, d = RM.build_blob(g["qweight"], g["scales"], g["cherry_weight"], g["cherry_indices"], g["bits"], g["K"], g["G"])
    assert np.array_equal(RM.decode_codes(blob, d), O.unpack_codes(g["qweight"], g["bits"]).astype(np.uint32))


@pytest.mark.parametrize("bits,K,N,Cn,G", [(4, 4096, 11008, 16, 128), (3, 11008, 4096, 40, 128), (3, 640, 40, 0, 64),
                                           (3, 8192, 28672, 32, 128), (4, 256, 8, 16, 128), (3, 28672, 8192, 112, 128),
                                           (4, 16384, 64, 64, 128)])
def test_model_dims_match_library(bits, K, N, Cn, G):
    from cherryq_b200 import _cabi
    L = _cabi.rlayer_init(bits, K, N, Cn, G)
    d = RM.dims(bits, K, N, Cn, G)
    for key in ("Kc", "NG", "sets", "Cp", "NT", "tile_bytes", "ksplit", "off_tiles", "off_perm", "off_cidx", "off_work", "blob_bytes"):
        assert getattr(L, key) == d[key], key
