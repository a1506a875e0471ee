"""Block quantisation: layouts, round trips, decoder cross-checks and the CPU fused dots."""
import ctypes

import numpy as np
import pytest
import torch

from realizar_b200 import quant
from realizar_b200._native import cpu_lib
from realizar_b200.quant import BLOCK_SPECS, QType
from realizar_b200.quant.device_layout import dev_row_bytes, to_device_layout
from realizar_b200.quant.torch_quant import quantize_torch

ALL = [QType.Q4_0, QType.Q4_1, QType.Q5_0, QType.Q5_1, QType.Q8_0, QType.Q2_K, QType.Q4_K, QType.Q5_K, QType.Q6_K]
# relative L2 error bounds of a round trip on N(0, 0.02) data
BOUND = {QType.Q4_0: 0.12, QType.Q4_1: 0.11, QType.Q5_0: 0.06, QType.Q5_1: 0.055, QType.Q8_0: 0.01, QType.Q2_K: 0.35,
         QType.Q4_K: 0.10, QType.Q5_K: 0.05, QType.Q6_K: 0.025}


def _w(n=32, k=512, seed=0):
    return (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)


def test_block_sizes_match_spec():
    assert (BLOCK_SPECS[QType.Q4_K].nbytes, BLOCK_SPECS[QType.Q5_K].nbytes, BLOCK_SPECS[QType.Q6_K].nbytes) == (144, 176, 210)
    assert (BLOCK_SPECS[QType.Q4_0].nbytes, BLOCK_SPECS[QType.Q8_0].nbytes) == (18, 34)
    for t, s in BLOCK_SPECS.items():
        if t in quant.WEIGHT_TYPES:
            assert cpu_lib().rlz_block_bytes(int(t)) == s.nbytes and cpu_lib().rlz_block_elems(int(t)) == s.elems


@pytest.mark.parametrize("qt", ALL)
def test_round_trip_error(qt):
    w = _w()
    q = quant.quantize(w, qt)
    assert q.size == quant.tensor_bytes(qt, w.shape)
    y = quant.dequantize(q, qt, w.shape)
    assert np.linalg.norm(y - w) / np.linalg.norm(w) < BOUND[qt]


def test_numpy_decoders_agree_with_native():
    w = _w(8, 1024, 3)
    for qt, fn in ((QType.Q4_K, quant.dequantize_q4_k_numpy), (QType.Q6_K, quant.dequantize_q6_k_numpy)):
        q = quant.quantize(w, qt)
        assert np.array_equal(fn(q, w.size), quant.dequantize(q, qt, w.shape).ravel())


def test_q4_0_layout_low_then_high_nibbles():
    x = np.zeros((1, 32), np.float32); x[0, 0] = -8.0; x[0, 16] = 7.0; x[0, 1] = 1.0
    q = quant.quantize(x, QType.Q4_0)
    d = q[:2].view(np.float16)[0]
    assert d == 1.0 and (q[2] & 0xF) == 0 and (q[2] >> 4) == 15 and (q[3] & 0xF) == 9


def test_q5_k_uses_canonical_high_bit_order():
    # element 0 of sub-block j takes bit j of qh[0]
    x = np.zeros((1, 256), np.float32)
    x[0, 3 * 32] = 31.0            # sub-block 3 -> bit 3
    q = quant.quantize(x, QType.Q5_K)
    assert q[16] & (1 << 3)
    assert np.abs(quant.dequantize(q, QType.Q5_K, x.shape) - x).max() < 0.51


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_K, QType.Q6_K, QType.Q8_0, QType.Q4_0, QType.Q5_0])
def test_torch_quantisers_emit_valid_blocks(qt):
    w = torch.from_numpy(_w(16, 512, 7))
    q = quantize_torch(w, qt).numpy()
    assert q.size == quant.tensor_bytes(qt, w.shape)
    y = quant.dequantize(q, qt, w.shape)
    assert np.linalg.norm(y - w.numpy()) / np.linalg.norm(w.numpy()) < BOUND[qt] * 1.6


@pytest.mark.parametrize("qt", ALL + [QType.F16, QType.BF16, QType.F32])
def test_fused_matvec_matches_dequantised(qt):
    w = _w(40, 512, 5)
    q = quant.quantize(w, qt)
    wd = quant.dequantize(q, qt, w.shape)
    x = np.random.default_rng(1).standard_normal((2, 512)).astype(np.float32)
    y = quant.matvec(q, qt, 40, 512, x)
    ref = x @ wd.T
    assert np.abs(y - ref).max() / np.abs(ref).max() < 0.02


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_K, QType.Q6_K, QType.Q8_0, QType.Q4_0])
@pytest.mark.parametrize("k", [256, 2560])
def test_gpu_unit_functions_on_host(qt, k):
    """The bit manipulation of the GPU fast path (csrc/gemv_units.h) run on the CPU."""
    lib = cpu_lib()
    lib.rlz_emu_gemv.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
    n, B = 9, 2
    w = _w(n, k, 11)
    q = quant.quantize(w, qt)
    wd = quant.dequantize(q, qt, w.shape)
    dev = to_device_layout(torch.from_numpy(q), qt, n, k).numpy().copy()
    assert dev.shape[1] == dev_row_bytes(qt, k) and dev.shape[1] % 16 == 0
    x = np.random.default_rng(2).standard_normal((B, k)).astype(np.float32)
    y = np.zeros((B, n), np.float32)
    assert lib.rlz_emu_gemv(int(qt), dev.ctypes.data, dev.shape[1], x.ctypes.data, y.ctypes.data, n, k, B) == 0
    ref = x @ wd.T
    assert np.abs(y - ref).max() / np.abs(ref).max() < 0.02


@pytest.mark.parametrize("qt", [QType.Q4_K, QType.Q5_K, QType.Q6_K])
@pytest.mark.parametrize("k", [256, 2560])
def test_gpu_block_functions_on_host(qt, k):
    """Whole-block dot products of the streamed GEMV (csrc/gemv_blocks.h) run on the CPU."""
    lib = cpu_lib()
    lib.rlz_emu_gemv_blocks.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int]
    n, B = 7, 2
    w = _w(n, k, 13)
    q = quant.quantize(w, qt)
    wd = quant.dequantize(q, qt, w.shape)
    dev = to_device_layout(torch.from_numpy(q), qt, n, k).numpy().copy()
    x = np.random.default_rng(3).standard_normal((B, k)).astype(np.float32)
    y = np.zeros((B, n), np.float32)
    assert lib.rlz_emu_gemv_blocks(int(qt), dev.ctypes.data, dev.shape[1], x.ctypes.data, y.ctypes.data, n, k, B) == 0
    ref = x @ wd.T
    assert np.abs(y - ref).max() / np.abs(ref).max() < 0.02


def test_rejects_bad_shapes():
    with pytest.raises(ValueError):
        quant.quantize(np.zeros((2, 100), np.float32), QType.Q4_K)
    with pytest.raises(ValueError):
        quant.dequantize(np.zeros(10, np.uint8), QType.Q4_K, (1, 256))
    assert quant.qtype_from_size(144 * 4, 2, 512) == QType.Q4_K


@pytest.mark.parametrize("qt", [QType.Q4_0, QType.Q4_1, QType.Q5_0, QType.Q5_1, QType.Q8_0, QType.Q4_K, QType.Q5_K, QType.Q6_K])
def test_simd_fused_dots_match_dequantised_reference(qt):
    """The fused dequant-dot of every block type (AVX2, and AVX-512 VNNI where the host has it) against a float64 product
    with the dequantised weights; the only difference allowed is the int8 quantisation of the activations."""
    import ctypes
    from realizar_b200._native import cpu_lib
    lib = cpu_lib()
    lib.rlz_cpu_dot_path.argtypes = [ctypes.c_int]
    rng = np.random.default_rng(int(qt) + 100)
    n, k = 37, 256 * 3
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    q = quant.quantize(w, qt)
    wd = quant.dequantize(q, qt, (n, k)).astype(np.float64)
    for batch in (1, 3):
        x = rng.standard_normal((batch, k)).astype(np.float32)
        y = quant.matvec(q, qt, n, k, x if batch > 1 else x[0])
        ref = x.astype(np.float64) @ wd.T
        err = np.abs(np.asarray(y).reshape(batch, n) - ref).max() / np.abs(ref).max()
        assert err < 0.02, (qt, batch, err)
    assert lib.rlz_cpu_dot_path(int(qt)) in (0, 1, 2)
    if lib.rlz_cpu_has_avx2():
        assert lib.rlz_cpu_dot_path(int(qt)) >= 1          # no block type of the public surface is left on the scalar path


def test_multi_matrix_product_equals_separate_products():
    """Several matrices with one input in one parallel region (Q / K / V, gate / up in the CPU decoder): bit-identical to one call
    per matrix; matrices whose block types need different activation formats are refused (-2) so the caller falls back."""
    import ctypes
    from realizar_b200._native import cpu_lib
    lib, rng = cpu_lib(), np.random.default_rng(0)
    for types, k, want in (((QType.Q5_0, QType.Q5_0, QType.Q8_0), 896, 0), ((QType.Q4_K, QType.Q6_K), 512, 0), ((QType.Q4_K, QType.Q8_0), 512, -2)):
        ns, B = [64, 20, 33][:len(types)], 3
        x = rng.standard_normal((B, k)).astype(np.float32)
        qs, ys, refs = [], [], []
        for qt, n in zip(types, ns):
            q = np.ascontiguousarray(np.frombuffer(quant.quantize((rng.standard_normal((n, k)) * 0.1).astype(np.float32), qt), np.uint8))
            qs.append(q); ys.append(np.zeros((B, n), np.float32))
            r = np.zeros((B, n), np.float32)
            assert lib.rlz_matvec(int(qt), q.ctypes.data, x.ctypes.data, r.ctypes.data, n, k, B) == 0
            refs.append(r)
        m = len(types)
        rc = lib.rlz_matvec_multi(m, (ctypes.c_int * m)(*[int(t) for t in types]), (ctypes.c_void_p * m)(*[q.ctypes.data for q in qs]),
                                  (ctypes.c_int64 * m)(*ns), k, x.ctypes.data, (ctypes.c_void_p * m)(*[y.ctypes.data for y in ys]), B)
        assert rc == want
        if rc == 0:
            assert all(np.array_equal(a, b) for a, b in zip(ys, refs))
