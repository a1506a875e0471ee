"""ctypes handles for the in-tree native libraries (built on first use if missing)."""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_double, c_float, c_int, c_int64, c_uint64, c_void_p, POINTER
from pathlib import Path

from . import _build

_lock = threading.Lock()
_cpu = None
_cuda = None


def cpu_lib() -> ctypes.CDLL:
    """librlz_cpu.so: quantisers, fused CPU dots, GGUF/APR parsers, CPU decoder, scheduler core."""
    global _cpu
    with _lock:
        if _cpu is None:
            path = _build.LIB / "librlz_cpu.so"
            if os.environ.get("RLZ_CPU_LIB"):                # another flavour of the library (sanitizer builds)
                path = _build.Path(os.environ["RLZ_CPU_LIB"])
            elif not path.exists() or os.environ.get("RLZ_REBUILD"):
                path = _build.build_cpu()
            lib = ctypes.CDLL(str(path))
            lib.rlz_block_elems.argtypes = [c_int]
            lib.rlz_block_bytes.argtypes = [c_int]
            lib.rlz_row_bytes.argtypes = [c_int, c_int64]
            lib.rlz_row_bytes.restype = c_int64
            lib.rlz_quantize.argtypes = [c_int, c_void_p, c_void_p, c_int64, c_int64]
            lib.rlz_dequantize.argtypes = [c_int, c_void_p, c_void_p, c_int64]
            lib.rlz_matvec.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64]
            lib.rlz_matvec_multi.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64]
            lib.rlz_gguf_open_buffer.argtypes = [c_void_p, c_uint64, c_char_p, c_int]
            lib.rlz_gguf_open_buffer.restype = c_void_p
            lib.rlz_gguf_open_file.argtypes = [c_char_p, c_char_p, c_int]
            lib.rlz_gguf_open_file.restype = c_void_p
            lib.rlz_gguf_close.argtypes = [c_void_p]
            lib.rlz_gguf_json.argtypes = [c_void_p, POINTER(c_uint64)]
            lib.rlz_gguf_json.restype = c_void_p
            lib.rlz_gguf_base.argtypes = [c_void_p]
            lib.rlz_gguf_base.restype = c_void_p
            lib.rlz_gguf_size.argtypes = [c_void_p]
            lib.rlz_gguf_size.restype = c_uint64
            lib.rlz_gguf_advise.argtypes = [c_void_p, c_int]
            lib.rlz_gguf_lock.argtypes = [c_void_p]
            lib.rlz_cpu_model_create.argtypes = [c_void_p]
            lib.rlz_cpu_model_create.restype = c_void_p
            lib.rlz_cpu_model_free.argtypes = [c_void_p]
            lib.rlz_cpu_model_set_tensor.argtypes = [c_void_p, c_char_p, c_int, c_void_p, c_int64, c_int64]
            lib.rlz_cpu_model_validate.argtypes = [c_void_p]
            lib.rlz_cpu_forward.argtypes = [c_void_p, c_int, c_int, c_void_p]
            lib.rlz_cpu_forward_rows.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p]
            lib.rlz_cpu_prefill.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
            lib.rlz_cpu_layer_trace.argtypes = [c_void_p, c_void_p]
            lib.rlz_cpu_generate_greedy.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
            _cpu = lib
        return _cpu


def cuda_lib_path() -> Path:
    """The kernel library; ``RLZ_CUDA_LIB`` may point at an alternative build (kernel tuning runs)."""
    return Path(os.environ["RLZ_CUDA_LIB"]) if os.environ.get("RLZ_CUDA_LIB") else _build.LIB / "librlz_cuda.so"


def cuda_lib() -> ctypes.CDLL:
    """librlz_cuda.so: the sm_100a kernels.  Raises if the library cannot be built or loaded:
    GPU paths never fall back silently to another implementation."""
    global _cuda
    with _lock:
        if _cuda is None:
            path = cuda_lib_path()
            if not path.exists() or os.environ.get("RLZ_REBUILD"):
                built = _build.build_cuda()
                if built is None:
                    raise RuntimeError("librlz_cuda.so is missing and nvcc was not found to build it")
                path = built
            _cuda = ctypes.CDLL(str(path))
            from .ops import _signatures
            _signatures.declare(_cuda)
        return _cuda


__all__ = ["cpu_lib", "cuda_lib", "cuda_lib_path", "c_void_p", "c_int", "c_int64", "c_float", "c_double"]
