"""Ahead-of-time, in-tree build of the native code (sm_100a only).

Two artefacts, both written next to this file so that they travel with the
source tree:

* ``_lib/libgefen_host.so`` – host-only C++ (exact-DP codebook solver), C ABI,
  loaded with ``ctypes``.
* ``_C.so`` – every CUDA kernel (``csrc/*.cu``, compiled by ``nvcc`` straight to
  ``sm_100a`` with ``-lineinfo``; the kernel files include no torch headers so a
  file compiles in seconds) plus ``csrc/bindings.cpp`` (the ``TORCH_LIBRARY``
  operator registrations, compiled by ``g++``).  Loaded with
  ``torch.ops.load_library``; operators appear under ``torch.ops.gefenx``.

The reference JIT-builds four extensions at first use with no arch flags of its
own (reference ``src/gefen/kernels/_build_notice.py:378-474``); here nothing is
compiled at run time unless the artefact is missing or older than its sources
and a compiler is present.  ``GEFENX_FORCE_REBUILD=1`` forces a rebuild,
``GEFENX_VERBOSE_BUILD=1`` echoes the compiler commands.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List, Optional

_PKG = Path(__file__).resolve().parent
_CSRC = _PKG / "csrc"
_OBJ = _PKG / "_build"
_HOST_SO = _PKG / "_lib" / "libgefen_host.so"
_CUDA_SO = _PKG / "_C.so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
_lock = threading.Lock()
_host_handle: Optional[ctypes.CDLL] = None
_cuda_loaded = False
_cuda_error: Optional[str] = None


def _verbose() -> bool:
    return os.environ.get("GEFENX_VERBOSE_BUILD", "0") not in ("", "0")


def _run(cmd: List[str]) -> None:
    if _verbose():
        print("[gefen_x_b200.build]", " ".join(cmd), flush=True)
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError(
            "native build step failed ({}):\n{}\n{}".format(
                proc.returncode, " ".join(cmd), proc.stdout[-6000:]
            )
        )
    if _verbose() and proc.stdout.strip():
        print(proc.stdout, flush=True)


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _stale(artifact: Path, sources) -> bool:
    stamp = artifact.with_suffix(artifact.suffix + ".sha")
    if os.environ.get("GEFENX_FORCE_REBUILD", "0") not in ("", "0"):
        return True
    if not artifact.exists():
        return True
    if not stamp.exists():
        return False  # shipped binary without a stamp: trust it
    return stamp.read_text().strip() != _digest(sources)


def _nvcc() -> Optional[str]:
    cand = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    exe = Path(cand) / "bin" / "nvcc"
    if exe.exists():
        return str(exe)
    return shutil.which("nvcc")


# --------------------------------------------------------------------------
# host library
# --------------------------------------------------------------------------
def host_sources():
    return sorted((_CSRC / "host").glob("*.cpp"))


def build_host(force: bool = False) -> Path:
    srcs = host_sources()
    if not force and not _stale(_HOST_SO, srcs):
        return _HOST_SO
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found for the host library")
    _HOST_SO.parent.mkdir(parents=True, exist_ok=True)
    tmp = _HOST_SO.with_suffix(".tmp.so")
    _run([cxx, "-O3", "-march=x86-64-v2", "-fopenmp", "-shared", "-fPIC", "-std=c++17",
          *map(str, srcs), "-o", str(tmp)])
    os.replace(tmp, _HOST_SO)
    _HOST_SO.with_suffix(".so.sha").write_text(_digest(srcs))
    return _HOST_SO


def host_lib() -> Optional[ctypes.CDLL]:
    """The host C library, building it on first use; ``None`` if impossible."""
    global _host_handle
    with _lock:
        if _host_handle is not None:
            return _host_handle
        try:
            path = build_host()
            lib = ctypes.CDLL(str(path))
            lib.gefen_exact_dp.restype = ctypes.c_int
            lib.gefen_exact_dp.argtypes = [
                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p,
            ]
            lib.gefen_exact_dp_monotone.restype = ctypes.c_int
            lib.gefen_exact_dp_monotone.argtypes = list(lib.gefen_exact_dp.argtypes)
            _host_handle = lib
        except Exception:  # pragma: no cover - toolchain missing
            _host_handle = None
        return _host_handle


# --------------------------------------------------------------------------
# CUDA library
# --------------------------------------------------------------------------
def cuda_sources():
    return sorted(_CSRC.glob("*.cu"))


def _all_cuda_inputs():
    return cuda_sources() + sorted(_CSRC.glob("*.cuh")) + sorted(_CSRC.glob("*.h")) + [
        _CSRC / "bindings.cpp"
    ]


def build_cuda(force: bool = False, jobs: Optional[int] = None) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``_C.so``."""
    inputs = _all_cuda_inputs()
    if not force and not _stale(_CUDA_SO, inputs):
        return _CUDA_SO
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    import torch
    from torch.utils import cpp_extension as ce

    _OBJ.mkdir(parents=True, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{_CSRC}"]
    cuda_home = str(Path(nvcc).resolve().parent.parent)
    headers = sorted(_CSRC.glob("*.cuh")) + sorted(_CSRC.glob("*.h"))
    hdr_digest = _digest(headers) if headers else ""

    def obj_for(src: Path) -> Path:
        return _OBJ / (src.stem + ".o")

    def needs(src: Path) -> bool:
        o = obj_for(src)
        stamp = o.with_suffix(".o.sha")
        want = _digest([src]) + hdr_digest
        if force or not o.exists() or not stamp.exists() or stamp.read_text() != want:
            return True
        return False

    def mark(src: Path) -> None:
        obj_for(src).with_suffix(".o.sha").write_text(_digest([src]) + hdr_digest)

    def compile_cu(src: Path) -> None:
        if not needs(src):
            return
        _run([nvcc, *NVCC_ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", f"-I{_CSRC}", f"-I{cuda_home}/include",
              "-c", str(src), "-o", str(obj_for(src))])
        mark(src)

    def compile_cpp(src: Path) -> None:
        if not needs(src):
            return
        cxx = shutil.which("g++") or "c++"
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        _run([cxx, "-O2", "-fPIC", "-std=c++17", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", str(src), "-o", str(obj_for(src))])
        mark(src)

    cus = cuda_sources()
    cpp = _CSRC / "bindings.cpp"
    with ThreadPoolExecutor(max_workers=jobs or min(8, (os.cpu_count() or 2))) as ex:
        futs = [ex.submit(compile_cu, s) for s in cus] + [ex.submit(compile_cpp, cpp)]
        for f in futs:
            f.result()

    libdirs = ce.library_paths("cuda")
    link = [shutil.which("g++") or "c++", "-shared", "-o", str(_CUDA_SO.with_suffix(".tmp.so")),
            *[str(obj_for(s)) for s in cus], str(obj_for(cpp))]
    for d in libdirs:
        link += [f"-L{d}", f"-Wl,-rpath,{d}"]
    link += [f"-L{cuda_home}/lib64", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda",
             "-ltorch_cuda", "-lcudart"]
    _run(link)
    os.replace(_CUDA_SO.with_suffix(".tmp.so"), _CUDA_SO)
    _CUDA_SO.with_suffix(".so.sha").write_text(_digest(inputs))
    return _CUDA_SO


def cuda_lib_path() -> Path:
    return _CUDA_SO


def load_cuda(required: bool = False) -> bool:
    """Load ``_C.so`` into ``torch.ops.gefenx``.

    Returns whether the operators are available.  With ``required=True`` a
    failure raises instead (used on CUDA devices, where a silent fallback to
    the torch path would hide a missing build).
    """
    global _cuda_loaded, _cuda_error
    with _lock:
        if _cuda_loaded:
            return True
        if _cuda_error is not None and not required:
            return False
        try:
            import torch

            path = _CUDA_SO
            if _stale(path, _all_cuda_inputs()) and _nvcc() is not None:
                path = build_cuda()
            if not path.exists():
                raise RuntimeError("{} is missing and nvcc is not available".format(path))
            torch.ops.load_library(str(path))
            _cuda_loaded = True
            _cuda_error = None
            return True
        except Exception as exc:
            _cuda_error = "{}: {}".format(type(exc).__name__, exc)
            if required:
                raise RuntimeError(
                    "gefen_x_b200: the sm_100a extension could not be loaded ({}). "
                    "Run `python -m gefen_x_b200.build`.".format(_cuda_error)
                ) from exc
            return False


def cuda_load_error() -> Optional[str]:
    return _cuda_error


def build_all(force: bool = False) -> None:
    build_host(force)
    build_cuda(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", _HOST_SO, _CUDA_SO)
