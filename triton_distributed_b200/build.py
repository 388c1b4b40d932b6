"""In-tree build of the native library (``lib/libb200dist.so``) for sm_100a.

Every ``.cu`` / ``.cc`` under ``csrc/`` is compiled with nvcc into ``build/`` and linked into one
shared object next to the Python package, so that a checkout is self-contained (no JIT cache).
Compilation is incremental (source / header mtimes) and parallel.

Role in the reference: CMake + setup.py building ``libtriton_distributed.so`` and the Triton
backend (``CMakeLists.txt:15-26``, ``csrc/lib/CMakeLists.txt:47``, ``python/setup.py``).

Usage: ``python -m triton_distributed_b200.build [--force] [--verbose] [--debug]``

``--debug`` builds a second library, ``lib/libb200dist_debug.so``, with ``-DB200_DEBUG_CHECKS``: bounds-checked symmetric
address translation and pseudo-random delays in front of every notify / wait / barrier (see ``b200/primitives.cuh``).
``B200DIST_DEBUG_LIB=1`` makes the package load it instead of the regular library.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
BUILD = PKG.parent / "build" / "b200dist"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libb200dist.so"
DEBUG_LIB_PATH = LIB_DIR / "libb200dist_debug.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-cudart", "static",
    "-x", "cu",
    "-I", str(CSRC / "include"),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return exe


def sources() -> list[Path]:
    out = sorted(list(CSRC.glob("runtime/*.cc")) + list(CSRC.glob("runtime/*.cu")) + list(CSRC.glob("kernels/*.cu")))
    return out


def _headers_mtime() -> float:
    return max((h.stat().st_mtime for h in (CSRC / "include").rglob("*") if h.is_file()), default=0.0)


def _compile(src: Path, obj: Path, verbose: bool, ptxas_v: bool, debug: bool = False) -> tuple[Path, str]:
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-DB200_DEBUG_CHECKS"] if debug else []), "-c", str(src), "-o", str(obj)]
    if ptxas_v:
        cmd += ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return src, proc.stderr if (verbose or ptxas_v) else ""


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False, jobs: int | None = None,
          debug: bool = False) -> Path:
    """Compile what is out of date and link the shared library (the checking build with ``debug``). Returns its path."""
    BUILD.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    hdr_time = max(_headers_mtime(), Path(__file__).stat().st_mtime)
    lib_path = DEBUG_LIB_PATH if debug else LIB_PATH
    todo, objs = [], []
    for src in sources():
        obj = BUILD / (src.parent.name + "_" + src.stem + (".dbg.o" if debug else ".o"))
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            todo.append((src, obj))
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
            futs = [ex.submit(_compile, s, o, verbose, ptxas_v, debug) for s, o in todo]
            for f in concurrent.futures.as_completed(futs):
                src, log = f.result()
                if verbose or ptxas_v:
                    print(f"[build] {src.name}\n{log}", file=sys.stderr)
    if todo or not lib_path.exists():
        cmd = [_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(lib_path), *map(str, objs), "-lpthread", "-ldl", "-lrt"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return lib_path


def compile_extension(source: str | Path, out_dir: str | Path | None = None, extra_flags: list[str] | None = None) -> Path:
    """Compile ONE user ``.cu`` file written against ``b200/primitives.cuh`` (and ``tcgen05.cuh``) into a shared object
    for sm_100a and return its path (load it with ``ctypes.CDLL``). Recompiled only when the source or a header is
    newer than the output. This is how a kernel that uses ``wait`` / ``notify`` / ``symm_at`` / ``putmem_signal_block``
    is built outside the library, the counterpart of JIT-compiling a ``@triton.jit`` function in the reference."""
    src = Path(source).resolve()
    out_dir = Path(out_dir) if out_dir is not None else BUILD / "ext"
    out_dir.mkdir(parents=True, exist_ok=True)
    out = out_dir / (src.stem + ".so")
    if out.exists() and out.stat().st_mtime >= max(src.stat().st_mtime, _headers_mtime()):
        return out
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", str(src), "-o", str(out), *(extra_flags or [])]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--debug", action="store_true", help="build lib/libb200dist_debug.so with B200_DEBUG_CHECKS")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose, ptxas_v=args.ptxas_v, debug=args.debug))


if __name__ == "__main__":
    main()
