"""Reading and writing the safetensors container: an 8-byte little-endian header length,
a JSON header (name -> dtype, shape, byte range), then the raw bytes.

The reference reads GGUF (gguf_file.h:53-91) through a table name -> offset, size, shape,
dtype (model_layout.h:17-23); this is the same idea for the format that model folders
with a config.json use.  The file is memory-mapped (privately: torch wants writable
memory, the file itself is never written); a tensor's bytes are touched only when it is
asked for.
"""
import json
import mmap
import struct

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise SafetensorsError("%s: too short to be a safetensors file" % path)
        (n,) = struct.unpack("<Q", head)
        size = self._f.seek(0, 2)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError("%s: header length %d does not fit the file (%d bytes)" % (path, n, size))
        self._f.seek(8)
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError("%s: header is not JSON: %s" % (path, e)) from e
        self.metadata = header.pop("__metadata__", {})
        self.entries = {}
        self._base = 8 + n
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError("%s: tensor '%s' has dtype %s, which is not supported"
                                       % (path, name, info["dtype"]))
            lo, hi = info["data_offsets"]
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            count = 1
            for s in shape:
                count *= s
            if hi - lo != count * torch.empty((), dtype=dtype).element_size() or self._base + hi > size:
                raise SafetensorsError("%s: tensor '%s' has a byte range that does not match its shape" % (path, name))
            self.entries[name] = (dtype, shape, lo, hi)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self):
        return list(self.entries)

    def dtype_shape(self, name):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name):
        """A CPU tensor that views the mapped file (copy it before the file is closed)."""
        dtype, shape, lo, hi = self.entries[name]
        if hi == lo:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._mm)[self._base + lo:self._base + hi]
        return torch.frombuffer(buf, dtype=dtype).reshape(shape)

    def close(self):
        # Tensors handed out may still view the map; let the garbage collector end it.
        self._mm = None
        self._f.close()


def write_safetensors(path, tensors, metadata=None):
    """tensors: name -> CPU tensor (written in the order given)."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError("tensor '%s' has dtype %s, which safetensors cannot hold" % (name, t.dtype))
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
