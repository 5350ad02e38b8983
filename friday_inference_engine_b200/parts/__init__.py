"""Parts and how to add one (parts/parts.cpp, include/friday/parts.h).

A part is a C++ class of one of five categories (norm, position, mixer, feed_forward,
block) registered under a name; the architecture's specification chooses parts by name,
layer by layer.  A new part, or a new architecture, lives in a shared library of its own
that registers itself when it is loaded: load_plugin(path).  build_plugin compiles such a
library from a .cu or .cpp file against the package's headers.
"""
import os
import subprocess

from .. import native
from ..ops import build

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")


def registered_parts(category):
    return native.call_json("friday_registered", native.text(category))


def load_plugin(path):
    native.call("friday_load_plugin", native.text(path))


def build_plugin(source, out_path):
    """Compiles `source` (.cu or .cpp) into the shared library `out_path` with the package's include paths; the
    library resolves the engine's symbols from the already loaded libfriday_engine.so."""
    native.lib()
    cmd = [build._nvcc()] + build.ARCH_FLAGS + ["-O2", "-std=c++17", "--shared", "-Xcompiler", "-fPIC", "-I", build.INCLUDE,
                                                "-I", build.PACKAGE, "-o", out_path, source]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise native.BuildError("nvcc failed for %s:\n%s\n%s" % (source, " ".join(cmd), proc.stdout))
    return os.path.abspath(out_path)
