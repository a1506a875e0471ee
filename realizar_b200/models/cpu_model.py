"""Python handle on the C++ CPU decoder (``csrc/cpu_engine.cpp``): the single-process CPU
configuration of the engine and the quantised-path oracle (reference parity:
``OwnedQuantizedModel::forward_cached`` / ``generate_with_cache``,
src/gguf/inference/fails.rs:92-336)."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from .._native import cpu_lib
from .weights import ModelWeights


class CpuModel:
    def __init__(self, weights: ModelWeights, max_seq: int = 512):
        self.weights = weights
        self.cfg = weights.config
        self.max_seq = max_seq
        lib = cpu_lib()
        cfg_bytes = self.cfg.pack_for_cpu_engine(max_seq)
        self._h = lib.rlz_cpu_model_create(ctypes.c_char_p(cfg_bytes))
        self._keep = []
        for name, t in weights.tensors.items():
            data = np.ascontiguousarray(t.numpy_bytes())
            self._keep.append(data)
            shape = t.shape if len(t.shape) == 2 else (1, int(np.prod(t.shape)))
            rc = lib.rlz_cpu_model_set_tensor(self._h, name.encode(), int(t.qtype), data.ctypes.data_as(ctypes.c_void_p), shape[0], shape[1])
            if rc and not name.startswith("rope_freqs"):
                raise ValueError(f"CPU engine does not know tensor '{name}' (rc={rc})")
        if "output.weight" not in weights.tensors:
            t = weights["token_embd.weight"]
            data = self._keep[list(weights.tensors).index("token_embd.weight")]
            lib.rlz_cpu_model_set_tensor(self._h, b"output.weight", int(t.qtype), data.ctypes.data_as(ctypes.c_void_p), t.shape[0], t.shape[1])
        rc = lib.rlz_cpu_model_validate(self._h)
        if rc:
            raise ValueError(f"model is missing required tensors (rc={rc})")

    def close(self):
        if self._h:
            cpu_lib().rlz_cpu_model_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, token: int, pos: int) -> np.ndarray:
        logits = np.empty(self.cfg.vocab_size, dtype=np.float32)
        rc = cpu_lib().rlz_cpu_forward(self._h, int(token), int(pos), logits.ctypes.data_as(ctypes.c_void_p))
        if rc:
            raise ValueError(f"forward failed (rc={rc}): token={token} pos={pos} max_seq={self.max_seq}")
        return logits

    @staticmethod
    def forward_rows(models: Sequence["CpuModel"], tokens: Sequence[int], positions: Sequence[int]) -> np.ndarray:
        """One decode step for several sequences in lock-step (``models[i]`` is fed ``tokens[i]`` at ``positions[i]``; every model
        keeps its own KV cache, all were built from the same weights): every projection is one batched product, so the step reads
        the weights once for all sequences.  Returns logits ``[len(models), vocab]``; row by row they equal ``forward``."""
        n = len(models)
        handles = (ctypes.c_void_p * n)(*[m._h for m in models])
        tk = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        ps = np.ascontiguousarray(np.asarray(positions, dtype=np.int32))
        logits = np.empty((n, models[0].cfg.vocab_size), dtype=np.float32)
        rc = cpu_lib().rlz_cpu_forward_rows(handles, tk.ctypes.data_as(ctypes.c_void_p), ps.ctypes.data_as(ctypes.c_void_p), n,
                                            logits.ctypes.data_as(ctypes.c_void_p))
        if rc:
            raise ValueError(f"forward_rows failed (rc={rc})")
        return logits

    def layer_trace(self) -> np.ndarray:
        out = np.empty(self.cfg.num_layers, dtype=np.float32)
        cpu_lib().rlz_cpu_layer_trace(self._h, out.ctypes.data_as(ctypes.c_void_p))
        return out

    def prefill(self, tokens: Sequence[int], pos0: int = 0, chunk: int = 32) -> np.ndarray:
        """Run prompt tokens at positions ``pos0 ..`` in chunks of ``chunk`` tokens (every projection one batched product per
        chunk, the output matrix only for the last token); returns the logits after the last token.  ``chunk=1`` is the
        token-by-token path; both give the same logits bit for bit."""
        p = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        logits = np.empty(self.cfg.vocab_size, dtype=np.float32)
        rc = cpu_lib().rlz_cpu_prefill(self._h, p.ctypes.data_as(ctypes.c_void_p), len(p), int(pos0), int(chunk), logits.ctypes.data_as(ctypes.c_void_p))
        if rc:
            raise ValueError(f"prefill failed (rc={rc}): {len(p)} tokens at position {pos0}, max_seq={self.max_seq}")
        return logits

    def generate_greedy(self, prompt: Sequence[int], n_gen: int, eos: Optional[int] = None):
        """Returns (tokens, prefill_seconds, decode_seconds)."""
        p = np.asarray(prompt, dtype=np.int32)
        out = np.zeros(n_gen, dtype=np.int32)
        tm = np.zeros(2, dtype=np.float64)
        n = cpu_lib().rlz_cpu_generate_greedy(self._h, p.ctypes.data_as(ctypes.c_void_p), len(p), n_gen,
                                              -1 if eos is None else int(eos), out.ctypes.data_as(ctypes.c_void_p),
                                              tm.ctypes.data_as(ctypes.c_void_p))
        if n < 0:
            raise ValueError(f"generate failed (rc={n})")
        return out[:n].tolist(), float(tm[0]), float(tm[1])
