"""Builds the library: the engine (C++ under src/, headers under include/friday/) and the
CUDA kernels under csrc/ for sm_100a, one shared library per kernel file.

libfriday_engine.so holds everything between a model folder and its logits:
configuration, weights, parts, cache, step function, decoder, generation loop.  It opens
the kernel libraries itself, each when it is first needed; a kernel family (rowwise,
gemm_simt, gemm_tc, attention_simt, attention_mma, attention_tc, sampling) is one .cu
file with a C interface and becomes one .so beside it
(friday_inference_engine_b200/_build/).  A library is compiled when it is first needed
and was not made from the present sources, so a run compiles what its model and dtype
use and nothing else.  If the package folder cannot be written, the libraries go to a
per-user folder under the system's temporary directory.

    python -m friday_inference_engine_b200.ops.build        # everything, for C++ users

There is no fallback: a library that cannot be built or loaded raises.
"""
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--expt-relaxed-constexpr"]
FAMILIES = ("rowwise", "gemm_simt", "attention_simt", "sampling", "gemm_tc", "attention_mma", "attention_tc")
PACKAGE = os.path.dirname(_HERE)
SOURCE_DIRS = ("config", "weights", "parts", "cache", "engine", "sampling", "ops")
INCLUDE = os.path.join(PACKAGE, "include")
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-Wall", "-Wno-unused-function"]
# libraries other than the runtime that a family links
EXTRA_LIBS = {}


class BuildError(RuntimeError):
    pass


def _nvcc():
    for cand in (os.environ.get("FRIDAY_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $FRIDAY_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other path")


def _writable_dir(path):
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, ".w%d" % os.getpid())
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


_build_dir = None


def build_dir():
    global _build_dir
    if _build_dir is None:
        pref = os.environ.get("FRIDAY_BUILD_DIR") or os.path.join(os.path.dirname(_HERE), "_build")
        if _writable_dir(pref):
            _build_dir = pref
        else:
            tag = hashlib.sha1(CSRC.encode()).hexdigest()[:10]
            alt = os.path.join(tempfile.gettempdir(), "friday_b200_build_%d_%s" % (os.getuid(), tag))
            if not _writable_dir(alt):
                raise BuildError("neither %s nor %s can be written: nowhere to build the kernels" % (pref, alt))
            _build_dir = alt
    return _build_dir


def _sources(family):
    src = os.path.join(CSRC, family + ".cu")
    if not os.path.exists(src):
        raise BuildError("no kernel source %s" % src)
    deps = [src] + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cuh", ".h"))]
    return src, deps


def library_path(family):
    return os.path.join(build_dir(), "libfriday_%s.so" % family)


def _fingerprint(family, extra_flags=()):
    """Hash of everything the library is made from: sources, headers, flags."""
    _, deps = _sources(family)
    h = hashlib.sha1()
    for d in deps:
        with open(d, "rb") as f:
            h.update(os.path.basename(d).encode() + b"\0" + f.read() + b"\0")
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + list(extra_flags) + EXTRA_LIBS.get(family, [])).encode())
    return h.hexdigest()


def is_fresh(family):
    """True if the built library was made from the sources as they are now (by content,
    not by time stamp: copies and checkouts do not keep time stamps in order)."""
    lib = library_path(family)
    try:
        with open(lib + ".sha1") as f:
            return os.path.exists(lib) and f.read().strip() == _fingerprint(family)
    except OSError:
        return False


def compile_family(family, verbose=False, extra_flags=()):
    """Runs nvcc for one family; returns the library's path."""
    src, _ = _sources(family)
    lib = library_path(family)
    tmp = "%s.%d.tmp" % (lib, os.getpid())
    cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + list(extra_flags) + ["-I", CSRC, "-o", tmp, src]
    cmd += EXTRA_LIBS.get(family, [])
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError("nvcc failed for %s:\n%s\n%s" % (family, " ".join(cmd), proc.stdout))
    os.replace(tmp, lib)
    with open(lib + ".sha1", "w") as f:
        f.write(_fingerprint(family, extra_flags))
    if verbose and proc.stdout.strip():
        print(proc.stdout, file=sys.stderr)
    return lib


def ensure_built(families, progress=True):
    """Compiles, in parallel, those of `families` that are missing or stale.

    While nvcc runs, a line is printed to stderr every few seconds so that a caller
    watching a first run sees that it is alive.
    """
    todo = [f for f in dict.fromkeys(families) if not is_fresh(f)]
    if not todo:
        return
    errors = []
    t0 = time.time()

    def work(fam):
        try:
            compile_family(fam)
        except Exception as e:  # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(f,), daemon=True) for f in todo]
    if progress:
        print("[friday] compiling CUDA kernels for sm_100a: %s" % ", ".join(todo), file=sys.stderr, flush=True)
    for t in threads:
        t.start()
    while any(t.is_alive() for t in threads):
        for t in threads:
            t.join(timeout=5.0 / len(threads))
        if progress and any(t.is_alive() for t in threads):
            print("[friday] ... still compiling (%.0f s)" % (time.time() - t0), file=sys.stderr, flush=True)
    if errors:
        raise errors[0]
    if progress:
        print("[friday] kernels built in %.0f s" % (time.time() - t0), file=sys.stderr, flush=True)


# ---------------------------------------------------------------------------------------
# the engine: C++ translation units compiled in parallel, linked with the CUDA runtime
# ---------------------------------------------------------------------------------------

def _cuda_home():
    nvcc = _nvcc()
    return os.path.dirname(os.path.dirname(os.path.realpath(nvcc)))


def _cxx():
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++")):
        if cand and (os.path.exists(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler was found (looked at $CXX, g++, c++): the engine cannot be built")


def _engine_inputs():
    units, headers = [], []
    for d in SOURCE_DIRS:
        folder = os.path.join(PACKAGE, d)
        units += sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".cpp"))
        headers += sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith(".h"))
    headers += sorted(os.path.join(INCLUDE, "friday", f) for f in os.listdir(os.path.join(INCLUDE, "friday")))
    headers += [os.path.join(CSRC, "gemm_tc_fusion.h"), os.path.join(CSRC, "philox.h")]
    return units, headers


def engine_library_path():
    return os.path.join(build_dir(), "libfriday_engine.so")


def _engine_fingerprint():
    units, headers = _engine_inputs()
    h = hashlib.sha1()
    for d in units + headers:
        with open(d, "rb") as f:
            h.update(os.path.relpath(d, PACKAGE).encode() + b"\0" + f.read() + b"\0")
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()


def engine_is_fresh():
    lib = engine_library_path()
    try:
        with open(lib + ".sha1") as f:
            return os.path.exists(lib) and f.read().strip() == _engine_fingerprint()
    except OSError:
        return False


def ensure_engine_built(progress=True):
    """Compiles the C++ files of config/, weights/, parts/, cache/, engine/, sampling/ and ops/ (in parallel) and links libfriday_engine.so, unless it was made from the present sources."""
    if engine_is_fresh():
        return engine_library_path()
    units, _ = _engine_inputs()
    cuda = _cuda_home()
    cxx = _cxx()
    objdir = os.path.join(build_dir(), "obj.%d" % os.getpid())
    os.makedirs(objdir, exist_ok=True)
    t0 = time.time()
    if progress:
        print("[friday] compiling the engine (%d C++ files)" % len(units), file=sys.stderr, flush=True)
    errors, objs = [], []

    def work(unit, obj):
        cmd = [cxx] + HOST_FLAGS + ["-I", INCLUDE, "-I", PACKAGE, "-I", os.path.join(cuda, "include"), "-c", unit, "-o", obj]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            errors.append(BuildError("the C++ compiler failed for %s:\n%s\n%s" % (unit, " ".join(cmd), proc.stdout)))

    threads = []
    for unit in units:
        obj = os.path.join(objdir, os.path.basename(unit)[:-4] + ".o")
        objs.append(obj)
        threads.append(threading.Thread(target=work, args=(unit, obj), daemon=True))
    for t in threads:
        t.start()
    while any(t.is_alive() for t in threads):
        for t in threads:
            t.join(timeout=5.0 / len(threads))
        if progress and any(t.is_alive() for t in threads):
            print("[friday] ... still compiling (%.0f s)" % (time.time() - t0), file=sys.stderr, flush=True)
    try:
        if errors:
            raise errors[0]
        lib = engine_library_path()
        tmp = "%s.%d.tmp" % (lib, os.getpid())
        cmd = [cxx, "-shared", "-o", tmp] + objs + ["-L", os.path.join(cuda, "lib64"), "-lcudart_static", "-ldl", "-lrt",
                                                     "-lpthread"]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            raise BuildError("linking the engine failed:\n%s\n%s" % (" ".join(cmd), proc.stdout))
        os.replace(tmp, lib)
        with open(lib + ".sha1", "w") as f:
            f.write(_engine_fingerprint())
    finally:
        shutil.rmtree(objdir, ignore_errors=True)
    if progress:
        print("[friday] engine built in %.0f s" % (time.time() - t0), file=sys.stderr, flush=True)
    return engine_library_path()


def build_all(progress=True):
    fams = [f for f in FAMILIES if os.path.exists(os.path.join(CSRC, f + ".cu"))]
    engine = ensure_engine_built(progress=progress)
    ensure_built(fams, progress=progress)
    return [engine] + [library_path(f) for f in fams]


if __name__ == "__main__":
    for path in build_all():
        print(path)
