"""Builds the CUDA libraries of this package with nvcc for sm_100a and loads them.

Each library is a small group of `.cu` files compiled with one set of defines
(the activation type, a head size).  A library is built the first time something
asks for it and kept beside the sources in `_build/`, under a name that carries a
hash of its sources and flags, so a changed source is rebuilt and an unchanged one
is only loaded.  If the package folder cannot be written, a per-user folder under
the system's temporary directory is used instead.  While nvcc runs, a line is
printed to stderr every few seconds.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Sequence, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# Tokens per cache page: the one definition.  The kernels get it as -DTL_PAGE, the cache and
# the generation loop import it from here.
PAGE_TOKENS = 64
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              f"-DTL_PAGE={PAGE_TOKENS}"]

# library name -> (sources, defines)
LIBRARIES: Dict[str, Tuple[Sequence[str], Sequence[str]]] = {
    "core_f32": (("elementwise.cu", "gemm_generic.cu", "attention_generic.cu"), ("-DTL_DTYPE=0",)),
    "core_bf16": (("elementwise.cu", "gemm_generic.cu", "attention_generic.cu"), ("-DTL_DTYPE=1",)),
    "sampling": (("sampling.cu",), ()),
    "random_init": (("random_init.cu",), ()),
}

# Set before any library is loaded: build the diagnostic variant whose kernels note when they
# start and end (-DTL_TRACE; another hash, so another file).
TRACE = False

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def register_library(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> None:
    LIBRARIES[name] = (tuple(sources), tuple(defines))


def find_nvcc() -> str:
    for cand in (os.environ.get("TL_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $TL_NVCC, PATH and /usr/local/cuda/bin): the CUDA "
                     "kernels of this package cannot be built and there is no other path")


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _closure(sources: Sequence[str]) -> List[str]:
    """The sources and every file of this folder that they include, directly or not."""
    seen: List[str] = []
    todo = list(sources)
    while todo:
        f = todo.pop()
        if f in seen or not os.path.isfile(os.path.join(_HERE, f)):
            continue
        seen.append(f)
        with open(os.path.join(_HERE, f), "r", encoding="utf-8") as fh:
            todo.extend(_INCLUDE.findall(fh.read()))
    return sorted(seen)


def _digest(sources: Sequence[str], defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in _closure(sources):
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(f.encode() + b"\0" + fh.read())
    h.update(" ".join(list(ARCH_FLAGS) + BASE_FLAGS + list(defines)).encode())
    return h.hexdigest()[:12]


def build_dir() -> str:
    d = os.environ.get("TL_BUILD_DIR") or os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"torchless_rs_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _defines(name: str) -> Tuple[Sequence[str], Sequence[str]]:
    sources, defines = LIBRARIES[name]
    return sources, tuple(defines) + (("-DTL_TRACE",) if TRACE else ())


def _file_tag(name: str) -> str:
    return name + ("_trace" if TRACE else "")


def library_path(name: str) -> str:
    sources, defines = _defines(name)
    return os.path.join(build_dir(), f"libtl_{_file_tag(name)}_{_digest(sources, defines)}.so")


def _run_with_progress(cmd: List[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            cwd=_HERE)
    out: List[str] = []
    reader = threading.Thread(target=lambda: out.append(proc.stdout.read()), daemon=True)
    reader.start()
    last = t0
    while proc.poll() is None:
        time.sleep(0.2)
        if time.time() - last >= 5.0:
            last = time.time()
            print(f"[torchless_rs_b200] compiling {what} ... {int(last - t0)} s", file=sys.stderr,
                  flush=True)
    reader.join()
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed for {what}:\n{' '.join(cmd)}\n{''.join(out)}")


def _remove_stale(name: str, keep: str) -> None:
    """Builds of the same library from older sources (another digest in the name) go away."""
    prefix, bdir = f"libtl_{name}_", os.path.dirname(keep)
    for f in os.listdir(bdir):
        rest = f[len(prefix):-3] if f.startswith(prefix) and f.endswith(".so") else ""
        if len(rest) == 12 and all(c in "0123456789abcdef" for c in rest) and \
                os.path.join(bdir, f) != keep:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass


def build_library(name: str, verbose: bool = True, extra_flags: Sequence[str] = ()) -> str:
    """Compiles the library if its file is not there yet; returns the path."""
    if name not in LIBRARIES:
        raise BuildError(f"no CUDA library named '{name}'")
    path = library_path(name)
    if os.path.isfile(path):
        return path
    nvcc = find_nvcc()
    sources, defines = _defines(name)
    bdir = os.path.dirname(path)
    tag = os.path.basename(path)[:-3]
    if verbose:
        print(f"[torchless_rs_b200] building {os.path.basename(path)} for sm_100a "
              f"({len(sources)} source files)", file=sys.stderr, flush=True)
    objs = [os.path.join(bdir, f"{tag}_{os.path.splitext(s)[0]}.{os.getpid()}.o") for s in sources]

    def one(pair):
        src, obj = pair
        cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *defines, *extra_flags, "-I", _HERE, "-c",
               os.path.join(_HERE, src), "-o", obj]
        _run_with_progress(cmd, f"{src} [{name}]")
    try:
        with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 2)) as ex:
            list(ex.map(one, zip(sources, objs)))
        tmp = f"{path}.{os.getpid()}.tmp"
        _run_with_progress([nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs, "-lcudart"],
                           f"link {name}")
        os.replace(tmp, path)  # atomic: a concurrent builder ends with the same file
        _remove_stale(_file_tag(name), path)
    finally:
        for o in objs:
            if os.path.exists(o):
                os.remove(o)
    return path


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library; built first if needed.  Fails loudly: there is no
    fallback without these kernels."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"could not load {path}: {e}") from e
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [build_library(n, verbose) for n in list(LIBRARIES)]
