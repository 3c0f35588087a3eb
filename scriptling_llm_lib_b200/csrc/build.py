"""Compiles the CUDA sources for sm_100a with nvcc and loads them through their C symbols.

Each library is one shared object built from one .cu file (plus the headers it includes), placed
in `csrc/_build/` inside the package. A library is compiled the first time something asks for it,
so a 32-bit run never waits for the bfloat16 tensor-core kernels and the other way round; the
source hash is stored beside the object and a changed source is rebuilt. While nvcc runs, a line
is printed every few seconds. There is no fallback: if the object can neither be found nor built,
loading fails with the compiler's message.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr"]

# library name -> (source file, headers and includes that it depends on)
LIBRARIES: dict[str, tuple[str, tuple[str, ...]]] = {
    "f32": ("lib_f32.cu", ("common.cuh", "generic_kernels.cuh", "generic_launchers.inc")),
    "bf16": ("lib_bf16.cu", ("common.cuh", "generic_kernels.cuh", "generic_launchers.inc")),
    "sampling": ("lib_sampling.cu", ("common.cuh", "philox.cuh")),
    "random": ("lib_random.cu", ("common.cuh", "philox.cuh")),
    "probe": ("lib_probe.cu", ("common.cuh",)),
    "decode_bf16": ("decode_bf16.cu", ("common.cuh", "attn_decode_noalloc.h")),
    "gemm_tcgen05": ("gemm_tcgen05.cu", ("common.cuh", "tcgen05.cuh")),
    "attn_prefill_tcgen05": ("attn_prefill_tcgen05.cu", ("common.cuh", "tcgen05.cuh")),
}

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def register_library(name: str, source: str, depends: tuple[str, ...] = ()) -> None:
    LIBRARIES[name] = (source, tuple(depends))


def find_nvcc() -> str:
    for cand in (os.environ.get("SLLM_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $SLLM_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be built and there is no other code path")


def _source_hash(name: str) -> str:
    src, deps = LIBRARIES[name]
    h = hashlib.sha256()
    for fn in (src,) + deps:
        h.update(fn.encode())
        h.update((CSRC / fn).read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()[:20]


def _fallback_dir() -> Path:
    """A per-user folder for built objects when the package folder cannot be written: under
    $XDG_CACHE_HOME or ~/.cache, else under the system's temp folder."""
    base = os.environ.get("XDG_CACHE_HOME") or (os.path.join(os.path.expanduser("~"), ".cache")
                                                if os.path.expanduser("~") not in ("", "~", "/") else "")
    if base:
        try:
            os.makedirs(base, mode=0o700, exist_ok=True)
            if os.access(base, os.W_OK | os.X_OK):
                return Path(base) / "sllm_b200_build"
        except OSError:
            pass
    return Path(tempfile.gettempdir()) / f"sllm_b200_build_{os.getuid()}"


def _private_dir(d: Path, create: bool) -> bool:
    """True when `d` is a real folder (no symlink) owned by this user that nobody else can write:
    objects are loaded into the process from it, so a folder anyone could have prepared is refused."""
    if create:
        try:
            os.mkdir(d, 0o700)
        except FileExistsError:
            pass
        except OSError:
            return False
    try:
        st = os.lstat(d)
    except OSError:
        return False
    import stat
    return stat.S_ISDIR(st.st_mode) and st.st_uid == os.getuid() and not (st.st_mode & 0o022)


def _tree_writable() -> bool:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    """csrc/_build when it can be written; else a private per-user folder (mode 0700, checked)."""
    if _tree_writable():
        return CSRC / "_build"
    d = _fallback_dir()
    if not _private_dir(d, create=True):
        raise KernelBuildError(f"{CSRC / '_build'} cannot be written and the fallback folder {d} is not a private "
                               f"folder of this user (it must be a real directory owned by uid {os.getuid()} that no "
                               "one else can write); remove it or set XDG_CACHE_HOME")
    return d


def library_path(name: str) -> Path | None:
    """An up-to-date object for `name`, if one is there already: in csrc/_build, and only when
    that folder cannot be written also in the private fallback folder."""
    tag = _source_hash(name)
    dirs = [CSRC / "_build"]
    if not _tree_writable():
        fb = _fallback_dir()
        if _private_dir(fb, create=False):
            dirs.append(fb)
    for d in dirs:
        so, stamp = d / f"sllm_{name}.so", d / f"sllm_{name}.hash"
        if so.is_file() and stamp.is_file() and stamp.read_text().strip() == tag:
            return so
    return None


def compile_library(name: str, verbose: bool = True) -> Path:
    if name not in LIBRARIES:
        raise KernelBuildError(f"no kernel library named {name!r}; known: {', '.join(sorted(LIBRARIES))}")
    have = library_path(name)
    if have is not None:
        return have
    nvcc = find_nvcc()
    out_dir = build_dir()
    src = CSRC / LIBRARIES[name][0]
    so = out_dir / f"sllm_{name}.so"
    tmp_so = out_dir / f".sllm_{name}.{os.getpid()}.so"
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp_so), str(src)]
    t0 = time.time()
    if verbose:
        print(f"[sllm_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            out, _ = proc.communicate(timeout=5.0)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[sllm_b200]   still compiling {src.name} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp_so.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{out}")
    os.replace(tmp_so, so)
    (out_dir / f"sllm_{name}.hash").write_text(_source_hash(name))
    if verbose:
        print(f"[sllm_b200] built {so.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return so


def load_library(name: str) -> ctypes.CDLL:
    """The loaded shared object of `name`; compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            from ..cache.needs import PAGE
            built_with = lib.sllm_page_tokens() if hasattr(lib, "sllm_page_tokens") else PAGE
            if built_with != PAGE:
                raise KernelBuildError(f"{path} was built for cache pages of {built_with} tokens; the cache uses {PAGE} "
                                       "(SLLM_PAGE in csrc/common.cuh and PAGE in cache/needs.py must agree)")
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> list[Path]:
    return [compile_library(n, verbose) for n in sorted(LIBRARIES)]
