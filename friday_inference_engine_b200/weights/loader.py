"""Fills a model's parameters by tensor name.

The model declares what it needs (name -> shape, kind); a source offers tensors by name
(a safetensors file, or seeded random numbers).  Before a byte is copied the two lists
are compared and every difference is reported in ONE error: tensors that the model
needs and the source lacks, tensors that the source has and the model does not know,
and tensors whose shape is wrong.  The reference reports these cases one at a time and
some of them as a bare std::out_of_range (model_layout.cpp:66, transformer.cpp:527,
1000-1005); here the message is the list.

Storage rule: floating tensors are kept in the activation dtype (bfloat16 or float32);
in bfloat16 mode a tensor that the file stores in 32 bits stays in 32 bits; integer
tables become int32.
"""
import torch


class WeightsError(ValueError):
    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


def storage_dtype(file_dtype, kind, compute_dtype):
    if kind == "int":
        return torch.int32
    if not file_dtype.is_floating_point:
        raise WeightsError("an integer tensor (%s) where a floating one is needed" % file_dtype)
    if compute_dtype == torch.float32:
        return torch.float32
    if file_dtype in (torch.float32, torch.float64):
        return torch.float32
    return compute_dtype


def check_names(expected, source, ignorable=(), where="weights"):
    """Raises one WeightsError that lists every mismatch between `expected`
    (name -> Param) and what `source` offers."""
    have = list(source.names())
    have_set = set(have)
    missing = [n for n in expected if n not in have_set]
    unexpected = [n for n in have if n not in expected and n not in ignorable]
    wrong = []
    for n, param in expected.items():
        if n in have_set:
            _, shape = source.dtype_shape(n)
            if tuple(shape) != tuple(param.shape):
                wrong.append((n, tuple(shape), tuple(param.shape)))
    if not (missing or unexpected or wrong):
        return
    lines = ["%s do not fit the model:" % where]
    if missing:
        lines.append("  missing (%d): %s" % (len(missing), ", ".join(missing)))
    if unexpected:
        lines.append("  unexpected (%d): %s" % (len(unexpected), ", ".join(unexpected)))
    if wrong:
        lines.append("  wrong shape (%d): %s" % (len(wrong), "; ".join(
            "%s is %s, the model needs %s" % (n, list(g), list(w)) for n, g, w in wrong)))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def load_weights(model, source, where=None):
    """Sets every parameter of `model` (an object with named_params(), finalize(), env and
    ignorable_tensors()) from `source`."""
    env = model.env
    expected = {}
    owners = {}
    for name, part, local, param in model.named_params():
        if name in expected:
            # a layer that the run order names twice still has its tensors once
            continue
        expected[name] = param
        owners[name] = (part, local)
    check_names(expected, source, model.ignorable_tensors(), where or getattr(source, "path", "weights"))
    for name, param in expected.items():
        file_dtype, _ = source.dtype_shape(name)
        dtype = storage_dtype(file_dtype, param.kind, env.dtype)
        t = source.tensor(name)
        t = t.to(device=env.device, dtype=dtype, non_blocking=False).contiguous()
        part, local = owners[name]
        part.set_tensor(local, t)
    model.finalize()
    return model
