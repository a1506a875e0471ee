"""GGUF reader / writer, header limits and corrupt-input handling."""
import struct

import numpy as np
import pytest

from realizar_b200.formats.gguf import GGUFBuilder, GGUFError, GGUFModel, T_F32, T_I32, T_STR, T_U8
from realizar_b200.models.config import ModelConfig, named_config
from realizar_b200.models.weights import ModelWeights, synthetic_weights, weights_to_gguf
from realizar_b200.quant import QType


def _tiny():
    b = GGUFBuilder("llama")
    b.add_u32("llama.block_count", 2).add_f32("llama.rope.freq_base", 10000.0).add_bool("flag", True)
    b.add_string("general.name", "tést \"quoted\"\n").add_array("arr", T_I32, [1, -2, 3]).add_string_array("tokenizer.ggml.tokens", ["a", "b\\", "Ġc"])
    b.add_tensor("w", np.arange(512, dtype=np.float32).reshape(2, 256) / 100, QType.Q4_K)
    b.add_tensor("v", np.ones((3, 32), np.float32), QType.F32)
    return b.build()


def test_round_trip_metadata_and_tensors(tmp_path):
    blob = _tiny()
    g = GGUFModel.from_bytes(blob)
    assert g.version == 3 and g.architecture == "llama"
    assert g.metadata["llama.block_count"] == 2 and g.metadata["flag"] is True
    assert g.metadata["general.name"] == "tést \"quoted\"\n" and g.metadata["arr"] == [1, -2, 3]
    assert g.vocabulary() == ["a", "b\\", "Ġc"]
    assert g.tensors["w"].shape == (2, 256) and g.tensors["w"].ne == (256, 2) and g.tensors["w"].nbytes == 288
    assert g.tensors["w"].offset % 32 == 0 and g.data_start % 32 == 0
    assert np.allclose(g.tensor_f32("v"), 1.0)
    p = tmp_path / "m.gguf"
    p.write_bytes(blob)
    g2 = GGUFModel.from_path(p)
    g2.advise("sequential")
    assert np.array_equal(g2.tensor_data("w"), g.tensor_data("w"))


def test_config_from_synthetic_model():
    cfg = named_config("tiny-phi2")
    w = synthetic_weights(cfg, seed=0)
    g = GGUFModel.from_bytes(weights_to_gguf(w, vocabulary=[f"t{i}" for i in range(cfg.vocab_size)]))
    c2 = ModelConfig.from_gguf(g)
    assert (c2.hidden_dim, c2.num_heads, c2.head_dim, c2.rope_dim, c2.parallel_residual, c2.fused_qkv) == (320, 4, 80, 32, True, True)
    assert c2.uses_layernorm and not c2.gated_ffn and c2.rope_type == 2 and c2.vocab_size == 512
    w2 = ModelWeights.from_gguf(g)
    assert set(w2.tensors) == set(w.tensors)


@pytest.mark.parametrize("mutate,msg", [
    (lambda b: b"XXXX" + b[4:], "magic"),
    (lambda b: b[:4] + struct.pack("<I", 9) + b[8:], "version"),
    (lambda b: b[:8] + struct.pack("<Q", 100001) + b[16:], "tensor_count"),
    (lambda b: b[:16] + struct.pack("<Q", 10001) + b[24:], "metadata_count"),
    (lambda b: b[:20], "small"),
    (lambda b: b[:200], "end of file|exceeds file size"),
])
def test_corrupt_headers_are_rejected(mutate, msg):
    with pytest.raises(GGUFError, match=msg):
        GGUFModel.from_bytes(mutate(_tiny()))


def test_truncated_tensor_data_and_bad_values():
    blob = _tiny()
    with pytest.raises(GGUFError, match="exceeds file size"):
        GGUFModel.from_bytes(blob[:-64])
    # unknown value type
    head = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 77)
    with pytest.raises(GGUFError, match="value type"):
        GGUFModel.from_bytes(head + b"\0" * 64)
    # array longer than the limit
    head = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<IIQ", 9, T_U8, 10_000_001)
    with pytest.raises(GGUFError, match="array length"):
        GGUFModel.from_bytes(head + b"\0" * 64)
    # string length larger than the file
    head = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1 << 40)
    with pytest.raises(GGUFError):
        GGUFModel.from_bytes(head + b"\0" * 64)


def test_random_byte_flips_never_crash():
    blob = bytearray(_tiny())
    rng = np.random.default_rng(0)
    for _ in range(300):
        b = bytearray(blob)
        for pos in rng.integers(0, min(len(b), 400), size=3):
            b[pos] = int(rng.integers(0, 256))
        try:
            g = GGUFModel.from_bytes(bytes(b))
            for name in g.tensors:
                g.tensor_data(name)
        except GGUFError:
            pass
