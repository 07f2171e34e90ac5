"""Build and load the sm_100a kernel library.

All device code of this package lives in ``csrc/*.cu`` and is compiled with
plain ``nvcc`` into ONE shared library next to this file
(``lib/libdmuon_b200.so``).  The library exports ``extern "C"`` launchers that
take raw device pointers and a CUDA stream handle; Python calls them through
``ctypes`` (no torch headers are involved, so a full rebuild takes seconds).

The reference builds its single CUDA extension through
``torch.utils.cpp_extension`` without an architecture flag (setup.py:21-30);
here the architecture is always ``sm_100a``.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from pathlib import Path

_HERE = Path(__file__).resolve().parent
CSRC = _HERE / "csrc"
LIBDIR = _HERE / "lib"
LIBPATH = LIBDIR / "libdmuon_b200.so"
STAMP = LIBDIR / "libdmuon_b200.stamp"

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-Xcompiler",
    "-fPIC",
]

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.glob("*")):
        if path.suffix in (".cu", ".cuh", ".h"):
            h.update(path.name.encode())
            h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    for root in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").exists():
            return str(Path(root) / "bin" / "nvcc")
    return None


def is_current() -> bool:
    return LIBPATH.exists() and STAMP.exists() and STAMP.read_text().strip() == _fingerprint()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library."""
    with _lock:
        if not force and is_current():
            return LIBPATH
        nvcc = _nvcc()
        if nvcc is None:
            raise RuntimeError("nvcc not found: cannot build the dmuon_b200 kernel library")
        LIBDIR.mkdir(exist_ok=True)
        objdir = LIBDIR / "obj"
        objdir.mkdir(exist_ok=True)
        objs = []
        procs = []
        for src in _sources():
            obj = objdir / (src.stem + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
            objs.append(str(obj))
        for src, proc in procs:
            out, _ = proc.communicate()
            if verbose and out:
                print(out.decode(errors="replace"))
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{out.decode(errors='replace')}")
        tmp = LIBPATH.with_suffix(".so.tmp")
        link = [nvcc, "-shared", "-o", str(tmp), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout.decode(errors='replace')}")
        os.replace(tmp, LIBPATH)
        STAMP.write_text(_fingerprint())
        return LIBPATH


def load() -> ctypes.CDLL:
    """Return the loaded kernel library, building it first if it is stale.

    Raises if the library can neither be found nor built: on a GPU machine a
    silent fallback to eager PyTorch would hide that the kernels are not in
    use.
    """
    global _lib
    if _lib is not None:
        return _lib
    if not is_current():
        if _nvcc() is not None:
            build()
        elif not LIBPATH.exists():
            raise RuntimeError(f"{LIBPATH} is missing and nvcc is not available to build it")
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(str(LIBPATH))
    return _lib


def is_loaded() -> bool:
    return _lib is not None


def _main() -> int:
    """``python -m dmuon_b200.ops.build [--force] [--verbose]``: compile the kernel library in place."""
    import argparse

    ap = argparse.ArgumentParser(description="Compile dmuon_b200's CUDA sources for sm_100a into the package.")
    ap.add_argument("--force", action="store_true", help="rebuild even if the library is up to date")
    ap.add_argument("--verbose", action="store_true", help="print ptxas resource usage (registers, spills, shared memory)")
    args = ap.parse_args()
    path = build(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
