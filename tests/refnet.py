"""ctypes access to oracle/_ref/libblaze_cpu.so: the reference's own Workspace / Net / CPU operators, compiled
unmodified by oracle/build_ref_dense.sh. TEST INFRASTRUCTURE: imported by tests/ and by the reference arm of
bench.py only."""
import ctypes as C
import os
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(ROOT, "oracle", "_ref", "libblaze_cpu.so")
NP_DTYPE = {1: np.float32, 2: np.int32, 10: np.int64, 12: np.float16}

_lib = None


def lib():
    """The library, or None when it has not been built (no reference checkout was mounted)."""
    global _lib
    if _lib is None and os.path.exists(LIB_PATH):
        L = C.CDLL(LIB_PATH)
        L.refnet_blas.restype = C.c_char_p
        L.refnet_last_error.restype = C.c_char_p
        L.refnet_create.restype = C.c_void_p
        L.refnet_create.argtypes = [C.c_char_p, C.c_char_p]
        L.refnet_destroy.argtypes = [C.c_void_p]
        L.refnet_feed.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int64), C.c_int, C.c_void_p, C.c_size_t]
        L.refnet_run.argtypes = [C.c_void_p]
        L.refnet_output.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_int), C.c_void_p,
                                    C.c_size_t, C.POINTER(C.c_size_t)]
        _lib = L
    return _lib


def blas_name():
    return lib().refnet_blas().decode()


class RefNet:
    """One reference Net created from NetDef text (device_type 0), optionally with a QED file for its Embedding ops."""

    def __init__(self, netdef_text, qed_file=None):
        L = lib()
        with tempfile.NamedTemporaryFile("w", suffix=".conf", delete=False) as f:
            f.write(netdef_text)
            path = f.name
        try:
            self.h = L.refnet_create(path.encode(), qed_file.encode() if qed_file else None)
        finally:
            os.unlink(path)
        if not self.h:
            raise RuntimeError("reference net: " + L.refnet_last_error().decode())

    def feed(self, name, array):
        a = np.ascontiguousarray(array)
        shape = (C.c_int64 * max(a.ndim, 1))(*a.shape)
        rc = lib().refnet_feed(self.h, name.encode(), shape, a.ndim, a.ctypes.data, a.nbytes)
        if rc:
            raise RuntimeError("reference net feed %s: %s" % (name, lib().refnet_last_error().decode()))

    def run(self):
        if lib().refnet_run(self.h):
            raise RuntimeError("reference net run: " + lib().refnet_last_error().decode())

    def output(self, name):
        shape, nd, nbytes = (C.c_int64 * 8)(), C.c_int(), C.c_size_t()
        dt = lib().refnet_output(self.h, name.encode(), shape, C.byref(nd), None, 0, C.byref(nbytes))
        if dt < 0:
            raise RuntimeError("reference net output %s: %s" % (name, lib().refnet_last_error().decode()))
        out = np.empty([shape[i] for i in range(nd.value)], NP_DTYPE[dt])
        lib().refnet_output(self.h, name.encode(), shape, C.byref(nd), out.ctypes.data, out.nbytes, C.byref(nbytes))
        return out

    def close(self):
        if self.h:
            lib().refnet_destroy(self.h)
            self.h = None
