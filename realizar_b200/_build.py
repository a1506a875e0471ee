"""In-tree build of the native libraries.

Two shared objects are produced next to the package:

* ``_lib/librlz_cpu.so``  – g++: quantisers, fused CPU dots, GGUF parser, CPU decoder.
* ``_lib/librlz_cuda.so`` – nvcc, ``sm_100a`` only: every GPU kernel plus the C launchers.

Both expose plain ``extern "C"`` entry points and are loaded with ``ctypes`` (no torch ABI
dependency, so a cross-compiled library built on a machine without a GPU runs unchanged on
the GPU host).  Objects are rebuilt only when a source or header is newer than the output.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"
OBJ = PKG / "_lib" / "obj"

CPU_SOURCES = ["quant_cpu.cpp", "cpu_engine.cpp", "gguf_native.cpp", "gemv_emu.cpp", "apr_native.cpp"]
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
              "-Xptxas", "-v", "-DNDEBUG"]


def _newer(src_paths, out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(p.stat().st_mtime > t for p in src_paths)


def _headers():
    return list(CSRC.glob("*.h")) + list((CSRC / "kernels").glob("*.cuh")) + list((CSRC / "kernels").glob("*.h"))


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def build_cpu(verbose: bool = False, sanitize: str | None = None) -> Path:
    """``sanitize``: "address" (AddressSanitizer + UndefinedBehaviorSanitizer) or "thread" builds a second library,
    ``librlz_cpu_asan.so`` / ``librlz_cpu_tsan.so``, that a process loads instead of the regular one through ``RLZ_CPU_LIB``
    (with the sanitizer runtime preloaded: ``LD_PRELOAD=$(gcc -print-file-name=libasan.so)``)."""
    LIB.mkdir(exist_ok=True)
    out = LIB / {None: "librlz_cpu.so", "address": "librlz_cpu_asan.so", "thread": "librlz_cpu_tsan.so"}[sanitize]
    srcs = [CSRC / s for s in CPU_SOURCES if (CSRC / s).exists()]
    if _newer(srcs + _headers(), out):
        flags = ["-O3"] if sanitize is None else ["-O1", "-g", "-fno-omit-frame-pointer",
                                                   "-fsanitize=address,undefined" if sanitize == "address" else "-fsanitize=thread"]
        cmd = ["g++", *flags, "-std=c++17", "-shared", "-fPIC", "-pthread", "-fno-math-errno",
               "-o", str(out)] + [str(s) for s in srcs]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return out


def cuda_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


def build_cuda(verbose: bool = False, jobs: int | None = None) -> Path | None:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link ``librlz_cuda.so``.

    The ptxas resource report (registers / spills / shared memory per kernel) of each
    translation unit is kept in ``_lib/obj/<name>.ptxas.txt``.
    """
    nvcc = nvcc_path()
    if nvcc is None:
        return None
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    out = LIB / "librlz_cuda.so"
    hdrs = _headers()
    srcs = cuda_sources()

    def compile_one(src: Path):
        obj = OBJ / (src.stem + ".o")
        if not _newer([src] + hdrs, obj):
            return obj, False
        cmd = [nvcc, *NVCC_ARCH, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd))
        r = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".ptxas.txt")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-6000:]}")
        return obj, True

    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = [o for o, _ in results]
    if any(changed for _, changed in results) or not out.exists():
        cmd = [nvcc, *NVCC_ARCH, "-shared", "-Xcompiler", "-fPIC", "-o", str(out)] + [str(o) for o in objs] + ["-lcuda"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return out


def build_all(verbose: bool = False):
    cpu = build_cpu(verbose)
    cuda = build_cuda(verbose)
    return cpu, cuda


if __name__ == "__main__":
    c, g = build_all(verbose="-v" in sys.argv)
    print("cpu :", c)
    print("cuda:", g)
