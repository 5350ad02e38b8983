"""The binding: loads libfriday_engine.so (built on first use) and declares its C interface
(include/friday/capi.h).  Everything between a model folder and its logits happens inside
that library; the classes of this package only marshal arguments.

Errors that the library reports come back as this module's exceptions, one class per kind
(ConfigError, WeightsError, StepError, CacheError, CacheFull, GenerationError,
KernelError, BuildError); a WeightsError carries the lists `missing`, `unexpected` and
`wrong_shape`.
"""
import ctypes
import json
import threading
from ctypes import (CFUNCTYPE, POINTER, Structure, byref, c_char_p, c_float, c_int, c_int64, c_size_t, c_uint64,
                    c_void_p)

from .ops import build


class FridayError(RuntimeError):
    pass


class ConfigError(FridayError, ValueError):
    """A config.json that cannot be used; the message names the key."""


class WeightsError(FridayError, ValueError):
    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


class StepError(FridayError, ValueError):
    """A step that cannot be run: unknown token id, a sequence too long, a bad request."""


class CacheError(FridayError):
    pass


class CacheFull(CacheError):
    """No free slot or page is left."""


class GenerationError(FridayError, ValueError):
    pass


class KernelError(FridayError):
    """A kernel refused its arguments or the CUDA runtime reported an error."""


class BuildError(FridayError):
    pass


_KINDS = {100: FridayError, 101: ConfigError, 102: WeightsError, 103: StepError, 104: CacheError, 105: CacheFull,
          106: GenerationError, 107: KernelError, 108: BuildError}


class Tensor(Structure):
    """FridayTensor (capi.h)."""
    _fields_ = [("data", c_void_p), ("dtype", c_int), ("ndim", c_int), ("shape", c_int64 * 4), ("ld", c_int64)]


class KV(Structure):
    _fields_ = [("k_pool", c_void_p), ("v_pool", c_void_p), ("pool_pages", c_int), ("block_table", c_void_p),
                ("table_width", c_int), ("page_size", c_int), ("window", c_int), ("n_kv_heads", c_int),
                ("head_dim", c_int), ("dtype", c_int), ("write", c_int)]


class Geometry(Structure):
    _fields_ = [("rows", c_int), ("n_seqs", c_int), ("max_q_len", c_int), ("max_kv_len", c_int), ("decode", c_int),
                ("row_seq", c_void_p), ("row_pos", c_void_p), ("seq_start", c_void_p), ("seq_qlen", c_void_p),
                ("seq_pos0", c_void_p)]


STEP_HOOK = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int),
                      POINTER(c_int))
SAMPLE_HOOK = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int))
ALLOC_HOOK = CFUNCTYPE(c_int, c_void_p, POINTER(c_int))
FREE_HOOK = CFUNCTYPE(c_int, c_void_p, c_int)
ON_STEP = CFUNCTYPE(None, c_void_p, c_int, POINTER(c_int), POINTER(c_int))
BUILDER = CFUNCTYPE(c_int, c_char_p)


class LoopHooks(Structure):
    _fields_ = [("user", c_void_p), ("step", STEP_HOOK), ("sample", SAMPLE_HOOK), ("alloc_slot", ALLOC_HOOK),
                ("free_slot", FREE_HOOK)]


P, I, F, S = c_void_p, c_int, c_float, c_char_p
PP, PS, PI = POINTER(c_void_p), POINTER(c_char_p), POINTER(c_int)
T = POINTER(Tensor)

_SIGNATURES = {
    "friday_set_builder": [BUILDER],
    "friday_load_plugin": [S],
    "friday_read_config": [S, PS],
    "friday_registered": [S, PS],
    "friday_describe_model": [S, PS],
    "friday_write_random_model": [S, S, c_uint64, S, I],
    "friday_check_weights": [S],
    "friday_storage_plan": [S, S, PS],
    "friday_random_tensor": [c_uint64, S, I, c_int64, P],
    "friday_safetensors_open": [S, PP],
    "friday_safetensors_list": [P, PS],
    "friday_safetensors_read": [P, S, P, c_size_t],
    "friday_safetensors_write": [S, S, PP, S],
    "friday_cache_new": [S, c_int64, I, I, PP],
    "friday_cache_alloc_slot": [P, PI],
    "friday_cache_free_slot": [P, I],
    "friday_cache_reserve": [P, I, PI, PI],
    "friday_cache_commit": [P, I, PI, PI],
    "friday_cache_info": [P, PS],
    "friday_generate_loop": [I, PI, PI, POINTER(LoopHooks), I, I, I, S, PS],
    "friday_engine_new": [S, PP],
    "friday_engine_info": [P, PS],
    "friday_engine_alloc_slot": [P, PI],
    "friday_engine_free_slot": [P, I],
    "friday_engine_slot_length": [P, I, PI],
    "friday_engine_step": [P, I, PI, PI, PI, PI, PI, P, I, POINTER(c_int64)],
    "friday_engine_step_token": [P, I, I, P],
    "friday_engine_prefill": [P, PI, I, I, P],
    "friday_engine_generate": [P, I, PI, PI, S, ON_STEP, P, PS],
    "friday_engine_set_trace": [P, P, I],
    "friday_engine_check": [P],
    "friday_engine_profile": [P, PS],
    "friday_engine_stats": [P, PS],
    "friday_decoder_new": [P, I, PI, PI, F, c_uint64, PI, PI, PP],
    "friday_decoder_step": [P, PI],
    "friday_decoder_sampled": [P, PI],
    "friday_decoder_logits": [P, P, I],
    "friday_decoder_retire": [P, I],
    "friday_decoder_info": [P, PS],
    "friday_decoder_close": [P, P],
    "friday_ops_new": [I, P, PP],
    "friday_ops_embedding": [P, P, c_int64, T, T],
    "friday_ops_gather_rows": [P, P, c_int64, T, T],
    "friday_ops_rmsnorm": [P, T, T, F, T],
    "friday_ops_swiglu": [P, T, T],
    "friday_ops_rope_kv_write": [P, T, P, P, P, I, I, I, I, POINTER(KV)],
    "friday_ops_advance": [P, P, P, P, P, P, P, I],
    "friday_ops_scale_rows": [P, T, F],
    "friday_ops_finish_logits": [P, T, T, F, F],
    "friday_ops_linear": [P, T, T, F, T, T, T, T, T, T],
    "friday_ops_linear_tc": [P, T, T, T, T, T, I, I, I, I],
    "friday_ops_linear_simt": [P, T, T, T, T, T],
    "friday_ops_linear_norm": [P, T, T, F, T, T, F, T, T, T, T, T, PI],
    "friday_ops_qkv_rope_write": [P, T, T, F, T, T, P, P, P, I, I, I, I, POINTER(KV), T],
    "friday_ops_linear_swiglu": [P, T, T, F, T, T],
    "friday_ops_attention": [P, T, c_int64, T, POINTER(KV), POINTER(Geometry), I, I, I, I, F],
    "friday_ops_sample": [P, T, P, P, P, c_uint64, P, P],
    "friday_ops_plan": [P, c_int64, c_int64, c_int64, PI, PI, PI],
    "friday_ops_decode_splits": [P, I, I, I, I, I, PI],
    "friday_ops_attention_splits": [P, c_int64, I, I, PI],
    "friday_ops_tensor_core_ok": [P, T, T, T, PI],
    "friday_ops_info": [P, PS],
    "friday_ops_check_status": [P],
}
_VOID = {"friday_engine_free": [P], "friday_cache_free": [P], "friday_decoder_free": [P], "friday_ops_free": [P],
         "friday_safetensors_free": [P]}

_lib = None
_lock = threading.Lock()
_builder_ref = None


def _build_family(name):
    """The library's builder hook: makes sure a kernel family's library was built from the present sources."""
    try:
        build.ensure_built([name.decode("utf-8")])
        return 0
    except Exception as e:  # noqa: BLE001 - reported to stderr; the library raises a KernelError of its own
        import sys
        print("[friday] %s" % e, file=sys.stderr, flush=True)
        return 1


def lib():
    """The loaded engine library (built first if its sources changed)."""
    global _lib, _builder_ref
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = build.ensure_engine_built()
        except build.BuildError as e:
            raise BuildError(str(e)) from None
        try:
            cdll = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)      # plug-ins resolve the library's symbols
        except OSError as e:
            raise BuildError("cannot load %s: %s" % (path, e)) from e
        for name, argtypes in _SIGNATURES.items():
            f = getattr(cdll, name)
            f.argtypes = argtypes
            f.restype = c_int
        for name, argtypes in _VOID.items():
            f = getattr(cdll, name)
            f.argtypes = argtypes
            f.restype = None
        for name in ("friday_last_error", "friday_last_error_detail", "friday_loaded_libraries"):
            getattr(cdll, name).restype = c_char_p
            getattr(cdll, name).argtypes = []
        _builder_ref = BUILDER(_build_family)
        cdll.friday_set_builder(_builder_ref)
        _lib = cdll
    return _lib


def check(rc):
    """Raises this module's exception for a non-zero return code."""
    if rc == 0:
        return
    cdll = lib()
    text = cdll.friday_last_error().decode("utf-8", "replace")
    cls = _KINDS.get(rc, FridayError)
    if cls is WeightsError:
        detail = cdll.friday_last_error_detail().decode("utf-8", "replace")
        d = json.loads(detail) if detail else {}
        raise WeightsError(text, d.get("missing", ()), d.get("unexpected", ()),
                           [(n, tuple(g), tuple(w)) for n, g, w in d.get("wrong_shape", ())])
    raise cls(text)


def call(name, *args):
    check(getattr(lib(), name)(*args))


def call_json(name, *args):
    """For functions whose last argument hands a JSON string back."""
    out = c_char_p()
    check(getattr(lib(), name)(*args, byref(out)))
    return json.loads(out.value.decode("utf-8"))


def text(s):
    return s.encode("utf-8") if isinstance(s, str) else s


def ints(values):
    values = list(values)
    return (c_int * max(len(values), 1))(*values)


def ragged(lists):
    """(offsets, values) as C int arrays for a list of lists."""
    offsets, values = [0], []
    for x in lists:
        values.extend(int(v) for v in x)
        offsets.append(len(values))
    return ints(offsets), ints(values)


def loaded_libraries():
    """Paths of the kernel libraries that the engine library has opened, and its own."""
    out = [p for p in lib().friday_loaded_libraries().decode().split("\n") if p]
    return [build.engine_library_path()] + out
