"""Direct access to the kernel libraries' C entry points (ctypes), for tests that call one
kernel's launcher with chosen arguments and for measurements.  The product path does not
come through here: the engine library opens the same files itself (ops/kernels.cpp).

A library is built on first use (ops/build.py) and loaded from the package's own
build folder, never from an installed location.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

from . import build

P, I, F = c_void_p, c_int, c_float


_SIGNATURES = {
    "rowwise": {
        "rowwise_embedding": [P, P, P, I, I, I, I, P],
        "rowwise_gather_rows": [P, P, P, I, I, I, P],
        "rowwise_rmsnorm": [P, P, I, P, I, I, F, I, P],
        "rowwise_swiglu": [P, P, I, I, I, P],
        "rowwise_rope_kv_write": [P, P, P, P, I, I, I, I, P, P, P, I, I, I, I, I, P],
        "rowwise_advance": [P, P, P, P, P, P, I, P],
    },
    "gemm_simt": {
        "gemm_simt": [P, I, P, I, P, I, P, I, P, I, I, I, I, I, I, P],
    },
    "gemm_tc": {
        "gemm_tc": [P, P, P, I, P, I, P, I, I, I, I, I, I, P, c_longlong, P, I, P, I, I, I, I, P],
        "gemm_tc_act": [P, P, P, I, P, I, P, I, I, I, I, I, I, P, c_longlong, P, I, P, I, I, I, I, I, P],
        "gemm_tc_plan": [I, I, I, I, I, I, I, P],
    },
    "attention_simt": {
        "attention_simt": [P, I, P, P, P, P, I, I, P, P, I, I, I, I, I, F, I, P, I, P],
    },
    "attention_mma": {
        "attention_mma": [P, I, P, P, P, I, P, I, I, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P, I, P, P],
        "attention_mma_supports": [I, I],
        "attention_mma_clusters_at_once": [I, I],
    },
    "attention_tc": {
        "attention_tc": [P, I, I, P, P, P, I, P, I, P, P, P, P, I, I, I, I, I, I, F, P, P],
        "attention_tc_supports": [I, I, I, I, I],
    },
    "sampling": {
        "sampling_sample": [P, I, I, I, P, P, P, c_ulonglong, P, P, P],
    },
}


from ..native import KernelError  # noqa: E402


class Family:
    def __init__(self, name):
        build.ensure_built([name])
        self.name = name
        self.path = build.library_path(name)
        try:
            self.cdll = ctypes.CDLL(self.path)
        except OSError as e:
            raise KernelError("cannot load %s: %s" % (self.path, e)) from e
        self._last_error = getattr(self.cdll, name + "_last_error")
        self._last_error.restype = ctypes.c_char_p
        self._last_error.argtypes = []
        for fn, argtypes in _SIGNATURES.get(name, {}).items():
            f = getattr(self.cdll, fn)
            f.argtypes = argtypes
            f.restype = c_int

    def call(self, fn, *args):
        rc = getattr(self.cdll, fn)(*args)
        if rc != 0:
            raise KernelError("%s: %s" % (fn, self._last_error().decode("utf-8", "replace")))

    def declare(self, fn, argtypes, restype=c_int):
        f = getattr(self.cdll, fn)
        f.argtypes = argtypes
        f.restype = restype
        return f


_families = {}


def family(name) -> Family:
    fam = _families.get(name)
    if fam is None:
        fam = _families[name] = Family(name)
    return fam


def loaded_libraries():
    return {n: f.path for n, f in _families.items()}
