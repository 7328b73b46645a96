"""The kernel library loads without a GPU and exports every entry point that
include/xdlb200.h declares (no compute calls here)."""
import ctypes
import os
import re

import pkg

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "xdlb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    m = pkg.load()
    m.build_native()
    L = ctypes.CDLL(m.capi.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), "libxdlb200.so does not export %s" % n
    # and the Python binding table covers the header
    assert set(names) == set(m.capi.SYMBOLS), set(names) ^ set(m.capi.SYMBOLS)


def test_argument_errors_are_reported_without_a_gpu():
    m = pkg.load()
    L = m.lib()
    assert L.xb_gemm(None, None) == -1
    assert b"null" in L.xb_last_error()
    assert L.xb_table_row_pitch(18, m.capi.XB_F16) == 48
    assert L.xb_table_row_pitch(16, m.capi.XB_F32) == 64


def test_host_index_builder_matches_lookup_rule():
    import numpy as np
    m = pkg.load()
    keys = np.array([5, 1 << 40, -7, 5, 99], np.int64)          # a repeated key keeps its first row
    slots = 16
    sk = np.zeros(slots, np.int64)
    sr = np.zeros(slots, np.int32)
    rc = m.lib().xb_table_build_index_host(keys.ctypes.data, len(keys), slots, sk.ctypes.data, sr.ctypes.data)
    assert rc == 0
    found = {int(k): int(r) for k, r in zip(sk, sr) if r >= 0}
    assert found == {5: 0, 1 << 40: 1, -7: 2, 99: 4}
    assert m.lib().xb_table_build_index_host(keys.ctypes.data, len(keys), 8, sk.ctypes.data, sr.ctypes.data) == -1
