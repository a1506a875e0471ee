"""APR v2, SafeTensors, format detection, the unified loader and converters."""
import json
import struct

import numpy as np
import pytest

from realizar_b200.formats import apr, detect
from realizar_b200.formats.apr import AprBuilder, AprError, AprModel, to_gguf_name
from realizar_b200.formats.convert import convert, requantize, weights_to_apr
from realizar_b200.formats.safetensors import SafeTensorsError, SafeTensorsFile, write_safetensors
from realizar_b200.models.config import named_config
from realizar_b200.models.cpu_model import CpuModel
from realizar_b200.models.weights import synthetic_weights, weights_to_gguf
from realizar_b200.quant import QType


def test_apr_round_trip_header_fields_and_compression():
    w = synthetic_weights(named_config("tiny-llama"), seed=0)
    blob = weights_to_apr(w)
    assert blob[:4] == b"APR2" and struct.unpack_from("<I", blob, 8)[0] == len(w.tensors)
    flags = struct.unpack_from("<H", blob, 6)[0]
    assert flags & apr.FLAG_QUANTIZED and struct.unpack_from("<Q", blob, 32)[0] % 64 == 0
    m = AprModel.from_bytes(blob)
    assert m.metadata["hidden_size"] == 256 and set(m.tensors) == set(w.tensors)
    name = "blk.0.attn_q.weight"
    assert np.array_equal(m.tensor_data(name), w[name].numpy_bytes()) and m.qtype_of(name) == QType.Q4_K
    assert all(t["offset"] % 64 == 0 for t in m.tensors.values())
    for comp in ("lz4", "zstd"):
        c = weights_to_apr(w, compression=comp)
        assert len(c) < len(blob) * 1.01
        m2 = AprModel.from_bytes(c)
        assert np.array_equal(m2.tensor_data(name), w[name].numpy_bytes())


def test_apr_rejects_bad_input_and_normalises_aliases():
    with pytest.raises(AprError, match="too small"):
        AprModel.from_bytes(b"APR2" + b"\0" * 10)
    with pytest.raises(AprError, match="magic"):
        AprModel.from_bytes(b"XXXX" + b"\0" * 100)
    with pytest.raises(AprError, match="v1"):
        AprModel.from_bytes(b"APR1" + b"\0" * 100)
    blob = bytearray(AprBuilder({"n_embd": 8, "n_layer": 2, "n_head": 2}).add_tensor_raw("t", (4,), 0, np.zeros(4, np.float32)).build())
    m = AprModel.from_bytes(bytes(blob))
    assert m.metadata["hidden_size"] == 8 and m.metadata["num_layers"] == 2 and m.metadata["num_heads"] == 2
    struct.pack_into("<I", blob, 8, 7)                       # claims more tensors than the index holds
    with pytest.raises(AprError):
        AprModel.from_bytes(bytes(blob))
    assert to_gguf_name("model.layers.3.self_attn.q_proj.weight") == "blk.3.attn_q.weight"
    assert to_gguf_name("model.layers.0.mlp.down_proj.weight") == "blk.0.ffn_down.weight"
    assert to_gguf_name("lm_head.weight") == "output.weight" and to_gguf_name("model.embed_tokens.weight") == "token_embd.weight"
    assert to_gguf_name("transformer.h.1.attn.c_attn.bias") == "blk.1.attn_qkv.bias" and to_gguf_name("rotary.inv_freq") is None


def test_safetensors_reader_writer_and_errors(tmp_path):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    blob = write_safetensors({"a": a, "b": a.astype(np.float16), "c": a}, metadata={"format": "pt"}, bf16={"c"})
    f = SafeTensorsFile.from_bytes(blob)
    assert f.metadata == {"format": "pt"} and f.tensors["c"]["dtype"] == "BF16"
    assert np.array_equal(f.numpy("a"), a) and np.array_equal(f.numpy("b"), a.astype(np.float16)) and np.array_equal(f.numpy("c"), a)
    with pytest.raises(SafeTensorsError):
        SafeTensorsFile.from_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafeTensorsError):
        SafeTensorsFile.from_bytes(struct.pack("<Q", 2) + b"{x")
    bad = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    with pytest.raises(SafeTensorsError, match="do not match"):
        SafeTensorsFile.from_bytes(struct.pack("<Q", len(bad)) + bad + b"\0" * 16)


def test_detect_and_load_all_three_formats_agree(tmp_path):
    cfg = named_config("tiny-llama")
    w = synthetic_weights(cfg, scheme="F16", seed=3, std=0.05)
    (tmp_path / "m.gguf").write_bytes(weights_to_gguf(w))
    (tmp_path / "m.apr").write_bytes(weights_to_apr(w))
    st_dir = tmp_path / "hf"
    st_dir.mkdir()
    hf = {}
    rename = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}
    lay = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
           "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
    for name, t in w.tensors.items():
        parts = name.split(".")
        hn = f"model.layers.{parts[1]}.{lay[parts[2]]}.{parts[3]}" if parts[0] == "blk" else f"{rename[parts[0]]}.{parts[1]}"
        hf[hn] = t.to_f32()
    write_safetensors(hf, st_dir / "model.safetensors")
    (st_dir / "config.json").write_text(json.dumps({"model_type": "llama", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
                                                    "num_key_value_heads": 2, "intermediate_size": 512, "vocab_size": 512, "rope_theta": 1e4,
                                                    "rms_norm_eps": 1e-5, "max_position_embeddings": 512}))
    assert [detect.detect_format(p) for p in (tmp_path / "m.gguf", tmp_path / "m.apr", st_dir)] == ["gguf", "apr", "safetensors"]
    toks = [5, 9, 100, 7]
    logits = [CpuModel(detect.load_model(p), 32).prefill(toks) for p in (tmp_path / "m.gguf", tmp_path / "m.apr", st_dir)]
    assert np.allclose(logits[0], logits[1], atol=1e-5) and np.allclose(logits[0], logits[2], atol=2e-3)
    (tmp_path / "junk.gguf").write_bytes(b"not a model at all")
    with pytest.raises(detect.FormatError):
        detect.detect_format(tmp_path / "junk.gguf")
    with pytest.raises(detect.FormatError):
        detect.detect_format(tmp_path / "missing.apr")


def test_convert_requantize_and_validation(tmp_path):
    w = synthetic_weights(named_config("tiny-llama"), scheme="F32", seed=1, std=0.05)
    (tmp_path / "f32.gguf").write_bytes(weights_to_gguf(w))
    info = convert(tmp_path / "f32.gguf", tmp_path / "q.apr", to="apr", qtype="Q4_K", compression="zstd")
    assert "Q4_K" in info["quantization"] and info["bytes"] < w.total_bytes() / 3
    wq = detect.load_model(tmp_path / "q.apr")
    assert wq["blk.0.attn_q.weight"].qtype == QType.Q4_K
    ref, got = CpuModel(w, 16).prefill([1, 2, 3]), CpuModel(wq, 16).prefill([1, 2, 3])
    assert float(ref @ got / np.linalg.norm(ref) / np.linalg.norm(got)) > 0.95        # 4-bit everything on a tiny random model
    broken = requantize(w, QType.Q8_0)
    del broken.tensors["blk.1.ffn_down.weight"]
    with pytest.raises(detect.FormatError, match="missing tensor"):
        detect.validate_weights(broken)
