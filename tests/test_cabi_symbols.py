"""The C-ABI library loads without a GPU and exports every symbol include/cherryq.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cherryq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import cherryq_b200
    from cherryq_b200 import _cabi
    if not os.path.exists(cherryq_b200.lib_path()):
        import __graft_entry__
        __graft_entry__.build()
    lib = ctypes.CDLL(cherryq_b200.lib_path())
    names = declared_symbols()
    assert len(names) >= 20
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(_cabi.SYMBOLS) == sorted(n for n in names if n in _cabi.SYMBOLS)
    assert set(_cabi.SYMBOLS) <= set(names)


def test_host_only_entry_points():
    from cherryq_b200 import _cabi
    lib = _cabi.lib()
    assert lib.cq_abi_version() == 3
    assert _cabi.strerror(0) == "ok"
    assert "multiple of 128" in _cabi.strerror(3)
    L = _cabi.layer_init(4, 4096, 11008, 16, 128)
    assert (L.Kc, L.n_gran, L.n_sub, L.gran_bytes) == (4080, 32, 688, 1056)
    T = _cabi.tlayer_init(3, 8192, 28672, 32, 128)
    assert (T.n_tile, T.n_cher, T.gran_bytes) == (224, 2, 6400)
    R = _cabi.rlayer_init(4, 4096, 11008, 16, 128)
    assert (R.NG, R.NT, R.Cp, R.tile_bytes) == (32, 688, 16, 32 * 1024 + 32 * 32 + 512)
    R3 = _cabi.rlayer_init(3, 640, 40, 0, 64)
    assert (R3.NG, R3.sets, R3.NT, R3.tile_bytes) == (5, 2, 3, 5 * 768 + 5 * 2 * 32)
    assert lib.cq_scratch_bytes() >= 2 * 1024 * 1024
    for bad in [(5, 4096, 64, 16, 128), (4, 4100, 64, 16, 128), (4, 4096, 64, 16, 96)]:
        with pytest.raises(RuntimeError):
            _cabi.layer_init(*bad)


def test_package_fails_loudly_without_native_library(monkeypatch, tmp_path):
    import cherryq_b200
    monkeypatch.setenv("CHERRYQ_LIB", str(tmp_path / "nope.so"))
    from cherryq_b200 import _cabi
    monkeypatch.setattr(_cabi, "_lib", None)
    with pytest.raises(cherryq_b200.NativeLibraryMissing):
        _cabi.lib()
