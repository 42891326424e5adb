"""Build and load the native CUDA library (``libqw_kernels.so``).

The library is compiled in-tree with ``nvcc -gencode arch=compute_100a,code=sm_100a`` from
``csrc/*.cu`` and loaded through ctypes; argument types of every ``qwk_*`` launcher are derived
from the prototypes in ``csrc/kernels.h`` so that pointers and 64-bit integers are passed
correctly.  On a machine with a GPU a missing library is an error (the ops never fall back to
PyTorch silently); on a CPU-only machine ``load()`` returns ``None`` unless the library exists.
"""
from __future__ import annotations

import ctypes
import glob
import os
import re
import shutil
import subprocess
from typing import Dict, List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libqw_kernels.so")
CHECKED_LIB_PATH = os.path.join(HERE, "libqw_kernels_checked.so")      # the same sources with -DQW_DEVICE_CHECKS
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

_lib: Optional[ctypes.CDLL] = None


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def sources() -> List[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def want_checked() -> bool:
    """QW_DEVICE_CHECKS=1 selects the bounds-checked build of the kernels."""
    return os.environ.get("QW_DEVICE_CHECKS", "0").strip().lower() in ("1", "true", "on", "yes")


def _stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, jobs: int = 8, checked: bool = False) -> str:
    """Compile every ``.cu`` to an object (in parallel) and link the shared library (``checked``: the bounds-checked
    variant, ``libqw_kernels_checked.so``)."""
    out_path = CHECKED_LIB_PATH if checked else LIB_PATH
    if not force and not _stale(out_path):
        return out_path
    nvcc = nvcc_path()
    objdir = os.path.join(HERE, "build_checked" if checked else "build")
    os.makedirs(objdir, exist_ok=True)
    common = ARCH_FLAGS + ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                           "--expt-relaxed-constexpr", "-I", CSRC] + (["-DQW_DEVICE_CHECKS"] if checked else [])
    if verbose:
        common += ["-Xptxas", "-v"]
    procs, objs = [], []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        hdrs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh"))
        if not force and os.path.exists(obj) and all(os.path.getmtime(obj) >= os.path.getmtime(d) for d in [src] + hdrs):
            continue
        procs.append((src, subprocess.Popen([nvcc] + common + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
        while len([p for _, p in procs if p.poll() is None]) >= jobs:
            procs[0][1].wait()
    log = []
    for src, p in procs:
        out, _ = p.communicate()
        log.append(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{out}")
    link = [nvcc] + ARCH_FLAGS + ["-shared", "-o", out_path] + objs
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout)
    if verbose:
        print("\n".join(log))
    return out_path


_CTYPE = {
    "int": ctypes.c_int, "float": ctypes.c_float, "double": ctypes.c_double, "long long": ctypes.c_longlong,
    "unsigned long long": ctypes.c_ulonglong, "cudaStream_t": ctypes.c_void_p, "unsigned int": ctypes.c_uint,
    "size_t": ctypes.c_size_t,
}


def _parse_prototypes(path: str) -> Dict[str, list]:
    txt = open(path).read()
    out = {}
    for m in re.finditer(r"int (qw\w+)\(([^)]*)\);", txt):
        args = []
        for a in m.group(2).split(","):
            a = a.strip()
            if "*" in a:
                args.append(ctypes.c_void_p)
            else:
                ty = " ".join(a.split()[:-1]).replace("const ", "").strip()
                args.append(_CTYPE[ty])
        out[m.group(1)] = args
    return out


def load(required: Optional[bool] = None) -> Optional[ctypes.CDLL]:
    """Load the library.  ``required`` defaults to "a CUDA device is present"."""
    global _lib
    if _lib is not None:
        return _lib
    if required is None:
        try:
            import torch
            required = torch.cuda.is_available()
        except Exception:
            required = False
    path = CHECKED_LIB_PATH if want_checked() else LIB_PATH
    if not os.path.exists(path):
        if required:
            raise RuntimeError(f"{path} is missing: run `python -m qwb200.build` (the CUDA ops have no fallback)")
        return None
    try:
        lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    except OSError:
        if required:
            raise
        return None
    for name, args in _parse_prototypes(os.path.join(CSRC, "kernels.h")).items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = ctypes.c_int
    if hasattr(lib, "qwrt_last_launches"):
        lib.qwrt_last_launches.restype = ctypes.c_longlong
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
