"""Weights as the library handles them (weights/*.cpp, include/friday/weights.h): the
safetensors container, sharded checkpoints, the one error that lists everything wrong
between a model and a folder, and the random-weights mode that writes model folders."""
import json
from ctypes import byref, c_void_p

from .. import native
from ..native import WeightsError  # noqa: F401

_SIZES = {"F64": 8, "I64": 8, "F32": 4, "I32": 4, "BF16": 2, "F16": 2, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1}


def write_model_dir(path, config, seed, dtype="BF16", shards=1):
    """config.json and model.safetensors (or `shards` shard files and an index) with seeded random weights:
    matrices, tables and biases N(0, 0.02), norm weights 1 + N(0, 0.02)."""
    native.call("friday_write_random_model", native.text(str(path)), native.text(json.dumps(config)), int(seed),
                native.text(dtype), int(shards))
    return str(path)


def check_weights(model_dir):
    """Raises one WeightsError listing missing and unexpected tensors and wrong shapes; needs no GPU."""
    native.call("friday_check_weights", native.text(str(model_dir)))


def storage_plan(model_dir, dtype="bfloat16"):
    """For every tensor of the folder, the dtype an engine of `dtype` keeps it in, and the stacked tensor it lands in
    (bfloat16 unless the file stores it in 32 bits; members of a stacked tensor share its dtype).  Needs no GPU."""
    return native.call_json("friday_storage_plan", native.text(str(model_dir)), native.text(dtype))


def random_tensor(seed, name, count, one=False):
    """The random-weights mode's float32 numbers for tensor `name` (before rounding to the stored dtype)."""
    import numpy as np
    out = np.empty((count,), dtype=np.float32)
    native.call("friday_random_tensor", int(seed), native.text(name), 1 if one else 0, int(count),
                c_void_p(out.ctypes.data))
    return out


class SafetensorsFile:
    """The library's reader of one safetensors file: names, dtypes, shapes, raw bytes."""

    def __init__(self, path):
        self.path = str(path)
        self._h = c_void_p()
        native.call("friday_safetensors_open", native.text(self.path), byref(self._h))
        listing = native.call_json("friday_safetensors_list", self._h)
        self.metadata = listing["metadata"] or {}
        self.entries = {t["name"]: (t["dtype"], tuple(t["shape"])) for t in listing["tensors"]}

    def names(self):
        return list(self.entries)

    def dtype_shape(self, name):
        return self.entries[name]

    def raw(self, name):
        """The tensor's bytes (little-endian, row-major)."""
        dtype, shape = self.entries[name]
        n = _SIZES[dtype]
        for s in shape:
            n *= s
        buf = bytearray(n)
        if n:
            import ctypes
            native.call("friday_safetensors_read", self._h, native.text(name),
                        ctypes.addressof((ctypes.c_char * n).from_buffer(buf)), n)
        return bytes(buf)

    def close(self):
        if self._h:
            native.lib().friday_safetensors_free(self._h)
            self._h = None

    def __del__(self):
        if getattr(self, "_h", None) and native._lib is not None:
            self.close()


def write_safetensors(path, tensors, metadata=None):
    """tensors: list of (name, dtype name, shape, bytes), written in the order given."""
    import ctypes
    header = [{"name": n, "dtype": d, "shape": list(s)} for n, d, s, _ in tensors]
    blobs = [bytes(b) for _, _, _, b in tensors]
    arr = (ctypes.c_void_p * max(len(blobs), 1))()
    keep = []
    for i, b in enumerate(blobs):
        cb = ctypes.create_string_buffer(b, max(len(b), 1))
        keep.append(cb)
        arr[i] = ctypes.addressof(cb)
    native.call("friday_safetensors_write", native.text(str(path)), native.text(json.dumps(header)), arr,
                native.text(json.dumps(metadata)) if metadata else None)
