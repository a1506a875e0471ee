"""ctypes mirrors of the parameter blocks in ``csrc/kernels`` and the argument types of every
exported launcher of ``librlz_cuda.so``."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_int32, c_int64, c_longlong, c_void_p

GEMV_MAX_MATS = 4
GEMV_MAX_X = 4

ACT_NONE, ACT_GELU, ACT_SILU = 0, 1, 2
COMBINE_ADD, COMBINE_SILU_MUL, COMBINE_GELU_MUL = 0, 1, 2
NORM_NONE, NORM_RMS, NORM_LAYER = 0, 1, 2


class GemvSeg(Structure):
    _fields_ = [("W", c_void_p), ("stride", c_int64), ("qtype", c_int32), ("k", c_int32), ("x_id", c_int32), ("_pad", c_int32)]


class GemvMat(Structure):
    _fields_ = [("seg", GemvSeg * 2), ("bias", c_void_p), ("bias2", c_void_p), ("nseg", c_int32), ("combine", c_int32),
                ("n", c_int32), ("out_off", c_int32), ("act", c_int32), ("has_residual", c_int32), ("rows_per_cta", c_int32),
                ("cta_begin", c_int32), ("q_out", c_void_p), ("q_out_k", c_int32), ("q_out_col0", c_int32)]


class GemvX(Structure):
    _fields_ = [("x", c_void_p), ("nw", c_void_p), ("nb", c_void_p), ("ld", c_int64), ("k", c_int32), ("norm", c_int32),
                ("eps", c_float), ("_pad", c_int32), ("pre", c_void_p)]


AR_MAX_RANKS = 8


class GemvAr(Structure):
    _fields_ = [("inbox", c_void_p * AR_MAX_RANKS), ("epoch", c_void_p), ("status", c_void_p), ("spin_limit", c_int64),
                ("rank", c_int32), ("world", c_int32), ("enabled", c_int32), ("n", c_int32)]


class GemvParams(Structure):
    _fields_ = [("mat", GemvMat * GEMV_MAX_MATS), ("xs", GemvX * GEMV_MAX_X), ("y", c_void_p), ("residual", c_void_p),
                ("ldy", c_int64), ("ld_res", c_int64), ("nmat", c_int32), ("batch", c_int32), ("max_k", c_int32),
                ("max_rows", c_int32), ("any_generic", c_int32), ("_pad", c_int32), ("ar", GemvAr)]


class CandExchange(Structure):
    _fields_ = [("inbox", c_void_p * AR_MAX_RANKS), ("epoch", c_void_p), ("status", c_void_p), ("spin_limit", c_int64),
                ("rank", c_int32), ("world", c_int32), ("batch", c_int32), ("max_batch", c_int32)]


class AttnDecodeParams(Structure):
    _fields_ = [("qkv", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("positions", c_void_p),
                ("page_table", c_void_p), ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("partial", c_void_p),
                ("counters", c_void_p), ("ld_qkv", c_int64), ("ld_out", c_int64), ("n_heads", c_int32), ("n_kv_heads", c_int32),
                ("head_dim", c_int32), ("max_pages", c_int32), ("rope_dim", c_int32), ("rope_type", c_int32), ("splits", c_int32),
                ("batch", c_int32), ("q_off", c_int32), ("k_off", c_int32), ("v_off", c_int32), ("pt_stride", c_int32),
                ("rope_theta", c_float), ("eps", c_float), ("scale", c_float), ("no_append", c_int32), ("window", c_int32),
                ("rope_table_len", c_int32), ("rope_table", c_void_p), ("kv_q8", c_int32), ("num_pages", c_int32)]


class AttnPrefillParams(Structure):
    _fields_ = [("qkv", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("page_table", c_void_p),
                ("ld_qkv", c_int64), ("ld_out", c_int64), ("n_heads", c_int32), ("n_kv_heads", c_int32), ("head_dim", c_int32),
                ("q_off", c_int32), ("n_tokens", c_int32), ("pos0", c_int32), ("window", c_int32), ("kv_q8", c_int32), ("scale", c_float),
                ("out_bf16", c_int32), ("pos0_ptr", c_void_p)]


class SampleParams(Structure):
    _fields_ = [("logits", c_void_p), ("ld", c_int64), ("vocab", c_int32), ("batch", c_int32), ("temperature", c_void_p),
                ("top_k", c_void_p), ("top_p", c_void_p), ("min_p", c_void_p), ("uniform", c_void_p), ("out", c_void_p),
                ("out_logprob", c_void_p)]


class ShardSample(Structure):
    _fields_ = [("inbox", c_void_p * AR_MAX_RANKS), ("flags", c_void_p * AR_MAX_RANKS), ("epoch", c_void_p), ("status", c_void_p),
                ("spin_limit", c_int64), ("rank", c_int32), ("world", c_int32), ("batch_cap", c_int32), ("K", c_int32),
                ("index_offset", c_int32), ("_pad", c_int32)]


class GemmParams(Structure):
    _fields_ = [("W", c_void_p), ("w_stride", c_int64), ("qtype", c_int32), ("n", c_int32), ("k", c_int32), ("m", c_int32),
                ("X", c_void_p), ("ldx", c_int64), ("Y", c_void_p), ("ldy", c_int64), ("bias", c_void_p), ("residual", c_void_p),
                ("ld_res", c_int64), ("act", c_int32), ("splitk", c_int32), ("atomic_out", c_int32), ("_pad", c_int32),
                ("ar_inbox", c_void_p * 8), ("ar_epoch", c_void_p), ("ar_row_pairs", c_int64), ("ar_rank", c_int32), ("ar_world", c_int32),
                ("ar_rows", c_int32), ("ar_enabled", c_int32), ("ar_site", c_int32), ("ar_nsites", c_int32), ("ar_splits", c_int32), ("flags", c_int32),
                ("rs_flags", c_void_p * 8), ("rs_own_rows", c_int32), ("rs_ntiles", c_int32), ("rs_mtiles", c_int32), ("_pad2", c_int32)]


class RsReduce(Structure):
    _fields_ = [("inbox", c_void_p), ("flags", c_void_p), ("ag_flags", c_void_p * AR_MAX_RANKS), ("xb", c_void_p * AR_MAX_RANKS),
                ("xpeer", c_void_p * AR_MAX_RANKS), ("x", c_void_p), ("nw", c_void_p), ("nb", c_void_p), ("epoch", c_void_p),
                ("status", c_void_p), ("spin_limit", c_int64), ("ldx", c_int64), ("ldxb", c_int64), ("ld_in", c_int64),
                ("rank", c_int32), ("world", c_int32), ("splits_stride", c_int32), ("splits_used", c_int32), ("rows_cap", c_int32),
                ("own_rows", c_int32), ("own_cap", c_int32), ("tokens", c_int32), ("n", c_int32), ("nt", c_int32), ("n_tiles", c_int32),
                ("ntiles_cap", c_int32), ("mtiles_cap", c_int32), ("site", c_int32), ("nsites", c_int32), ("norm", c_int32),
                ("push_x", c_int32), ("wait_ag", c_int32), ("eps", c_float), ("_pad", c_int32)]


class StepOp(Structure):
    _fields_ = [("kind", c_int32), ("grid", c_int32), ("params", c_int64)]


class StepEmbed(Structure):
    _fields_ = [("table", c_void_p), ("tokens", c_void_p), ("pos_table", c_void_p), ("positions", c_void_p), ("out", c_void_p),
                ("row_bytes", c_int64), ("qtype", c_int32), ("hidden", c_int32), ("vocab", c_int32), ("_pad", c_int32)]


class StepArgmax(Structure):
    _fields_ = [("logits", c_void_p), ("out", c_void_p), ("out_val", c_void_p), ("vocab", c_int32), ("index_offset", c_int32)]


class StepProgram(Structure):
    _fields_ = [("blob", c_void_p), ("sync", c_void_p), ("status", c_void_p), ("spin_limit", c_int64), ("nops", c_int32),
                ("occ", c_int32), ("attn_gt", c_int32), ("skip", c_int32)]


def declare(lib: ctypes.CDLL) -> None:
    lib.rlz_launch_count.restype = c_longlong
    lib.rlz_set_pdl.argtypes = [c_int]
    lib.rlz_device_info.argtypes = [c_int, POINTER(c_int), POINTER(c_longlong)]
    lib.rlz_cuda_error_string.argtypes = [c_int]
    lib.rlz_cuda_error_string.restype = ctypes.c_char_p
    lib.rlz_gemv.argtypes = [POINTER(GemvParams), c_void_p]
    lib.rlz_gemv_stream.argtypes = [POINTER(GemvParams), c_void_p]
    lib.rlz_gemv_slab.argtypes = [POINTER(GemvParams), c_void_p]
    lib.rlz_gemv_slab_check.argtypes = [POINTER(GemvParams)]
    lib.rlz_gemv_slab_error.argtypes = [c_int]
    lib.rlz_gemv_slab_trace_enable.argtypes = [c_int]
    lib.rlz_gemv_slab_trace_read.argtypes = [c_void_p, c_int, c_int]
    lib.rlz_gemv_trace_enable.argtypes = [c_int]
    lib.rlz_gemv_trace_read.argtypes = [c_void_p, c_int, c_int]
    lib.rlz_gemv_prepare.argtypes = [POINTER(GemvParams), POINTER(c_int)]
    lib.rlz_gemv_smem_bytes.argtypes = [POINTER(GemvParams)]
    lib.rlz_gemv_smem_bytes.restype = c_longlong
    lib.rlz_decode_step.argtypes = [POINTER(StepProgram), c_longlong, c_void_p]
    lib.rlz_decode_step_attn_smem.argtypes = [c_int]
    lib.rlz_device_error.argtypes = [c_int]
    lib.rlz_gemm_kquant.argtypes = [POINTER(GemmParams), c_void_p]
    lib.rlz_gemm_error.argtypes = [c_int]
    lib.rlz_gemm_plan.argtypes = [POINTER(GemmParams), POINTER(c_int), POINTER(c_int), POINTER(c_int)]
    lib.rlz_rs_reduce.argtypes = [POINTER(RsReduce), c_void_p]
    lib.rlz_gemm_trace_enable.argtypes = [c_int]
    lib.rlz_gemm_trace_read.argtypes = [c_void_p, c_int]
    lib.rlz_symm_alloc.argtypes = [ctypes.c_ulonglong, POINTER(c_void_p), c_void_p]
    lib.rlz_symm_open.argtypes = [c_void_p, POINTER(c_void_p)]
    lib.rlz_symm_close.argtypes = [c_void_p]
    lib.rlz_symm_free.argtypes = [c_void_p]
    lib.rlz_epoch_bump.argtypes = [c_void_p, c_void_p]
    lib.rlz_cand_exchange.argtypes = [POINTER(CandExchange), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.rlz_attn_decode.argtypes = [POINTER(AttnDecodeParams), c_void_p]
    lib.rlz_attn_decode_error.argtypes = [c_int]
    lib.rlz_attn_decode_partial_floats.argtypes = [c_int, c_int, c_int, c_int]
    lib.rlz_attn_decode_partial_floats.restype = c_longlong
    lib.rlz_attn_decode_counter_ints.argtypes = [c_int, c_int]
    lib.rlz_attn_decode_counter_ints.restype = c_longlong
    lib.rlz_embed.argtypes = [c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p]
    lib.rlz_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_int, c_float, c_void_p]
    lib.rlz_head_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_float, c_void_p]
    lib.rlz_rope.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_int, c_float, c_void_p, c_int, c_void_p]
    lib.rlz_elementwise.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong,
                                    c_longlong, c_int, c_int, c_void_p]
    lib.rlz_kv_append.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.rlz_kv_append_q8.argtypes = lib.rlz_kv_append.argtypes
    lib.rlz_to_bf16.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_void_p]
    lib.rlz_norm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_float, c_void_p]
    lib.rlz_swiglu_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_longlong, c_int, c_void_p]
    lib.rlz_attn_prefill.argtypes = [POINTER(AttnPrefillParams), c_void_p]
    lib.rlz_attn_prefill_impl.argtypes = [POINTER(AttnPrefillParams), c_void_p, c_int]
    lib.rlz_attn_prefill_supported.argtypes = [c_int]
    lib.rlz_attn_prefill_error.argtypes = [c_int]
    lib.rlz_ll_reduce.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p]
    lib.rlz_advance.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.rlz_page_rows.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.rlz_argmax.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
    lib.rlz_sample.argtypes = [POINTER(SampleParams), c_void_p]
    lib.rlz_sample_push.argtypes = [POINTER(SampleParams), POINTER(ShardSample), c_void_p]
    lib.rlz_sample_merge.argtypes = [POINTER(SampleParams), POINTER(ShardSample), c_void_p]
    lib.rlz_history_push.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p]
    lib.rlz_logit_controls.argtypes = [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                                       c_void_p, c_void_p]
    lib.rlz_logprob_rows.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]
    lib.rlz_penalties.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    for name in ("rlz_gemm_kquant", "rlz_attn_prefill", "rlz_flash_decode_static", "rlz_symm_alloc"):
        pass  # declared by their own modules when present
