"""Model configuration: per-architecture constraints and the config derived from checkpoint
metadata (reference parity: ``ArchConstraints`` src/gguf/arch_constraints_fallback.rs:14-261,
``GGUFConfig`` src/gguf/config.rs:229-321 and ``infer_rope_type`` src/gguf/config.rs:176-226).

Unlike the reference, ``rope_dim`` (partial rotary, ``{arch}.rope.dimension_count``) and the
Phi-2 parallel residual are first-class fields so those models run on the GPU path.
"""
from __future__ import annotations

import struct
from dataclasses import asdict, dataclass, field, replace
from typing import Optional

ROPE_NORM = 0   # rotate adjacent pairs (2i, 2i+1)
ROPE_NEOX = 2   # rotate split halves (i, i + rot/2)


@dataclass(frozen=True)
class ArchConstraints:
    norm_type: str = "rmsnorm"          # "rmsnorm" | "layernorm"
    activation: str = "silu"            # "silu" | "gelu"
    positional_encoding: str = "rope"   # "rope" | "absolute" | "relative" | "none"
    mlp_type: str = "swiglu"            # "swiglu" | "gelu_mlp" | "gated_mlp"
    weight_layout: str = "linear"       # "linear" | "conv1d"
    has_bias: bool = False
    tied_embeddings: bool = False
    has_qk_norm: bool = False
    default_eps: float = 1e-5


_LLAMA = ArchConstraints()
_TABLE = {
    "gpt2": ArchConstraints("layernorm", "gelu", "absolute", "gelu_mlp", "conv1d", True, True, False, 1e-5),
    "llama": _LLAMA, "llama3": _LLAMA,
    "qwen2": ArchConstraints(has_bias=True, default_eps=1e-6),
    "qwen2.5": ArchConstraints(has_bias=True, default_eps=1e-6),
    "qwen": ArchConstraints(has_bias=True, default_eps=1e-6),
    "qwen3": ArchConstraints(has_qk_norm=True, default_eps=1e-6),
    "mistral": _LLAMA,
    "phi2": ArchConstraints("layernorm", "gelu", "rope", "gelu_mlp", "linear", True, False, False, 1e-5),
    "phi": ArchConstraints("layernorm", "silu", "rope", "swiglu", "linear", True, False, False, 1e-5),
    "phi3": ArchConstraints("layernorm", "silu", "rope", "swiglu", "linear", True, False, False, 1e-5),
    "gemma": ArchConstraints("rmsnorm", "gelu", "rope", "gated_mlp", "linear", False, True, False, 1e-6),
    "gemma2": ArchConstraints("rmsnorm", "gelu", "rope", "gated_mlp", "linear", False, True, False, 1e-6),
    "deepseek": ArchConstraints(default_eps=1e-6), "deepseek2": ArchConstraints(default_eps=1e-6),
    "bert": ArchConstraints("layernorm", "gelu", "absolute", "gelu_mlp", "linear", True, True, False, 1e-12),
    "whisper": ArchConstraints("layernorm", "gelu", "absolute", "gelu_mlp", "linear", True, False, False, 1e-5),
    "t5": ArchConstraints("layernorm", "gelu", "relative", "gelu_mlp", "linear", False, True, False, 1e-6),
    "encoder-decoder": ArchConstraints("layernorm", "gelu", "relative", "gelu_mlp", "linear", False, True, False, 1e-6),
    "mamba": ArchConstraints("rmsnorm", "silu", "none", "swiglu", "linear", False, True, False, 1e-5),
    "qwen3_5": ArchConstraints(default_eps=1e-6), "qwen3.5": ArchConstraints(default_eps=1e-6),
    "qwen3_moe": ArchConstraints(has_qk_norm=True, default_eps=1e-6),
    "qwen3_5_moe": ArchConstraints(has_qk_norm=True, default_eps=1e-6),
    "falcon_h1": ArchConstraints(default_eps=1e-6), "falcon-h1": ArchConstraints(default_eps=1e-6),
    "openelm": ArchConstraints(default_eps=1e-6),
    "moonshine": ArchConstraints("layernorm", "silu", "rope", "gated_mlp", "linear", False, True, False, 1e-5),
    "rwkv7": ArchConstraints("layernorm", "gelu", "none", "gelu_mlp", "linear", False, False, False, 1e-5),
    "rwkv": ArchConstraints("layernorm", "gelu", "none", "gelu_mlp", "linear", False, False, False, 1e-5),
}

_NEOX_ARCHS = ("qwen", "stablelm", "phi", "gemma", "starcoder2", "gptneox", "gpt_neox", "falcon", "codeshell",
               "orion", "bert", "dbrx", "olmo2", "olmoe", "plamo", "openelm", "exaone", "minicpm3", "nemotron",
               "internlm2", "deepseek")

_DEFAULT_BOS = {"qwen2": 151643, "qwen3": 151643, "qwen3moe": 151643, "llama": 128000, "mistral": 1,
                "gemma": 2, "gemma2": 2, "deepseek": 0, "deepseek2": 0, "phi3": 1}
_DEFAULT_EOS = {"qwen2": 151645, "qwen3": 151645, "qwen3moe": 151645, "qwen3_5": 248044, "llama": 128001,
                "mistral": 2, "gemma": 1, "gemma2": 1, "deepseek": 1, "deepseek2": 1, "phi3": 32000,
                "phi2": 50256, "phi": 50256, "gpt2": 50256}
_DEFAULT_THETA = {"qwen2": 1e6, "qwen3": 1e6, "llama": 5e5, "llama3": 5e5, "mistral": 1e6, "phi2": 1e4,
                  "phi3": 1e4, "gemma": 1e4, "gemma2": 1e4, "deepseek": 1e4, "deepseek2": 1e4}


def arch_constraints(arch: str) -> ArchConstraints:
    """Constraints for a ``general.architecture`` value; unknown names are LLaMA-like."""
    return _TABLE.get(arch.lower(), _LLAMA)


def infer_rope_type(arch: str) -> int:
    a = arch.lower()
    return ROPE_NEOX if any(n in a for n in _NEOX_ARCHS) else ROPE_NORM


def is_encoder_decoder(arch: str) -> bool:
    return arch.lower() in ("t5", "whisper", "encoder-decoder", "moonshine")


@dataclass
class ModelConfig:
    architecture: str = "llama"
    hidden_dim: int = 0
    num_layers: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    intermediate_dim: int = 0
    vocab_size: int = 0
    context_length: int = 4096
    rope_theta: float = 10000.0
    rope_dim: int = 0                    # rotated dims per head (0 -> head_dim)
    rope_type: int = ROPE_NORM
    eps: float = 1e-5
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    constraints: ArchConstraints = field(default_factory=ArchConstraints)
    parallel_residual: bool = False      # x + attn(norm x) + mlp(norm x)   (Phi-2, GPT-J style)
    fused_qkv: bool = False              # checkpoint stores attn_qkv as one tensor
    rope_scaling_type: str = "none"
    rope_scaling_factor: float = 1.0
    rope_original_context: int = 0       # pre-scaling context length (YaRN / dynamic NTK)
    sliding_window: Optional[int] = None # attend to the last N positions only (Mistral style)

    def __post_init__(self):
        if self.head_dim == 0 and self.num_heads:
            self.head_dim = self.hidden_dim // self.num_heads
        if self.num_kv_heads == 0:
            self.num_kv_heads = self.num_heads
        if self.rope_dim == 0:
            self.rope_dim = self.head_dim

    # -- derived ---------------------------------------------------------------------------
    @property
    def q_dim(self) -> int: return self.num_heads * self.head_dim
    @property
    def kv_dim(self) -> int: return self.num_kv_heads * self.head_dim
    @property
    def gated_ffn(self) -> bool: return self.constraints.mlp_type in ("swiglu", "gated_mlp")
    @property
    def uses_layernorm(self) -> bool: return self.constraints.norm_type == "layernorm"
    @property
    def uses_rope(self) -> bool: return self.constraints.positional_encoding == "rope"

    def validate(self) -> None:
        for f in ("hidden_dim", "num_layers", "num_heads", "num_kv_heads", "head_dim", "intermediate_dim", "vocab_size"):
            if getattr(self, f) <= 0:
                raise ValueError(f"model config: {f} must be positive (got {getattr(self, f)})")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads {self.num_heads} is not a multiple of num_kv_heads {self.num_kv_heads}")
        if self.rope_dim > self.head_dim or self.rope_dim % 2:
            raise ValueError(f"rope_dim {self.rope_dim} must be even and <= head_dim {self.head_dim}")

    def to_dict(self) -> dict:
        return asdict(self)

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)

    def pack_for_cpu_engine(self, max_seq: int) -> bytes:
        """Binary layout of ``struct Config`` in csrc/cpu_engine.cpp."""
        return struct.pack(
            "<13i2f", self.num_layers, self.hidden_dim, self.num_heads, self.num_kv_heads, self.head_dim,
            self.intermediate_dim, self.vocab_size, self.rope_dim if self.uses_rope else 0, self.rope_type,
            1 if self.uses_layernorm else 0, 1 if self.gated_ffn else 0, 1 if self.parallel_residual else 0,
            max_seq, self.rope_theta, self.eps)

    # -- constructors -----------------------------------------------------------------------
    @classmethod
    def from_gguf(cls, g) -> "ModelConfig":
        """Build from a parsed GGUF (``realizar_b200.formats.gguf.GGUFModel``)."""
        arch = g.architecture
        c = arch_constraints(arch)
        k = g.arch_key
        hidden = int(k("embedding_length", 0))
        heads = int(k("attention.head_count", 0))
        kv = k("attention.head_count_kv", heads)
        kv = int(kv[0] if isinstance(kv, list) else kv) or heads
        head_dim = int(k("attention.key_length", 0)) or (hidden // heads if heads else 0)
        vocab = k("vocab_size")
        if vocab is None:
            toks = g.get("tokenizer.ggml.tokens")
            if toks:
                vocab = len(toks)
            elif "token_embd.weight" in g.tensors:
                vocab = g.tensors["token_embd.weight"].shape[0]
        eps = k("attention.layer_norm_rms_epsilon") if c.norm_type == "rmsnorm" else k("attention.layer_norm_epsilon")
        if eps is None:
            eps = k("attention.layer_norm_rms_epsilon", k("attention.layer_norm_epsilon", c.default_eps))
        inter = int(k("feed_forward_length", 0))
        if not inter and "blk.0.ffn_up.weight" in g.tensors:
            inter = g.tensors["blk.0.ffn_up.weight"].shape[0]
        cfg = cls(
            architecture=arch, hidden_dim=hidden, num_layers=int(k("block_count", 0)), num_heads=heads,
            num_kv_heads=kv, head_dim=head_dim, intermediate_dim=inter, vocab_size=int(vocab or 0),
            context_length=int(k("context_length", 4096)),
            rope_theta=float(k("rope.freq_base", _DEFAULT_THETA.get(arch, 10000.0))),
            rope_dim=int(k("rope.dimension_count", 0)), rope_type=infer_rope_type(arch), eps=float(eps),
            bos_token_id=g.get("tokenizer.ggml.bos_token_id", _DEFAULT_BOS.get(arch)),
            eos_token_id=g.get("tokenizer.ggml.eos_token_id", _DEFAULT_EOS.get(arch)),
            constraints=c, parallel_residual=(arch == "phi2" or arch == "gptj"),
            fused_qkv="blk.0.attn_qkv.weight" in g.tensors,
            rope_scaling_type=str(k("rope.scaling.type", "none")), rope_scaling_factor=float(k("rope.scaling.factor", 1.0)),
            rope_original_context=int(k("rope.scaling.original_context_length", 0)),
            sliding_window=(int(k("attention.sliding_window", 0)) or None),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_hf_dict(cls, d: dict, architecture: Optional[str] = None) -> "ModelConfig":
        """Build from a HuggingFace-style ``config.json`` / APR metadata dictionary (aliases as
        accepted by the reference's APR metadata reader, src/apr/metadata.rs:15-90)."""
        def pick(*names, default=None):
            for n in names:
                if n in d and d[n] is not None:
                    return d[n]
            return default
        arch = architecture or pick("architecture", "model_type", default="llama")
        arch = {"qwen2.5": "qwen2", "phi-2": "phi2", "phi": "phi2" if pick("partial_rotary_factor") else "phi"}.get(arch, arch)
        c = arch_constraints(arch)
        hidden = int(pick("hidden_size", "hidden_dim", "n_embd", "d_model", default=0))
        heads = int(pick("num_attention_heads", "num_heads", "n_head", default=0))
        head_dim = int(pick("head_dim", default=0)) or (hidden // heads if heads else 0)
        prf = pick("partial_rotary_factor")
        rope_dim = int(pick("rope_dim", "rotary_dim", default=0)) or (int(head_dim * float(prf)) if prf else 0)
        cfg = cls(
            architecture=arch, hidden_dim=hidden, num_layers=int(pick("num_hidden_layers", "num_layers", "n_layer", default=0)),
            num_heads=heads, num_kv_heads=int(pick("num_key_value_heads", "num_kv_heads", default=heads)), head_dim=head_dim,
            intermediate_dim=int(pick("intermediate_size", "intermediate_dim", "n_inner", default=0) or 4 * hidden),
            vocab_size=int(pick("vocab_size", default=0)), context_length=int(pick("max_position_embeddings", "context_length", default=4096)),
            rope_theta=float(pick("rope_theta", default=_DEFAULT_THETA.get(arch, 10000.0))), rope_dim=rope_dim,
            rope_type=infer_rope_type(arch), eps=float(pick("rms_norm_eps", "layer_norm_eps", "layer_norm_epsilon", "eps", default=c.default_eps)),
            bos_token_id=pick("bos_token_id", default=_DEFAULT_BOS.get(arch)), eos_token_id=pick("eos_token_id", default=_DEFAULT_EOS.get(arch)),
            constraints=c, parallel_residual=(arch == "phi2"),
            rope_scaling_type=str((pick("rope_scaling") or {}).get("rope_type", (pick("rope_scaling") or {}).get("type", "none"))),
            rope_scaling_factor=float((pick("rope_scaling") or {}).get("factor", 1.0)),
            rope_original_context=int((pick("rope_scaling") or {}).get("original_max_position_embeddings", 0)),
            sliding_window=(int(pick("sliding_window", default=0) or 0) or None),
        )
        cfg.validate()
        return cfg


# Named shapes used by the benchmarks (architecture only; weights are random-initialised).
def named_config(name: str) -> ModelConfig:
    name = name.lower()
    if name in ("qwen2.5-0.5b", "qwen2-0.5b"):
        return ModelConfig("qwen2", 896, 24, 14, 2, 64, 4864, 151936, 32768, 1e6, 64, ROPE_NEOX, 1e-6, 151643, 151645,
                           replace(arch_constraints("qwen2"), tied_embeddings=True))
    if name in ("phi-2", "phi2"):
        return ModelConfig("phi2", 2560, 32, 32, 32, 80, 10240, 51200, 2048, 1e4, 32, ROPE_NEOX, 1e-5, None, 50256,
                           arch_constraints("phi2"), parallel_residual=True, fused_qkv=True)
    if name in ("llama-3-8b", "llama3-8b"):
        return ModelConfig("llama", 4096, 32, 32, 8, 128, 14336, 128256, 8192, 5e5, 128, ROPE_NORM, 1e-5, 128000, 128001, _LLAMA)
    if name in ("llama-3-70b", "llama3-70b"):
        return ModelConfig("llama", 8192, 80, 64, 8, 128, 28672, 128256, 8192, 5e5, 128, ROPE_NORM, 1e-5, 128000, 128001, _LLAMA)
    if name in ("tiny-llama", "tiny"):
        return ModelConfig("llama", 256, 2, 4, 2, 64, 512, 512, 512, 1e4, 64, ROPE_NORM, 1e-5, 1, 2, _LLAMA)
    if name == "tiny-phi2":
        return ModelConfig("phi2", 320, 2, 4, 4, 80, 1280, 512, 512, 1e4, 32, ROPE_NEOX, 1e-5, None, 2,
                           arch_constraints("phi2"), parallel_residual=True, fused_qkv=True)
    if name == "tiny-qwen2":
        return ModelConfig("qwen2", 256, 2, 4, 2, 64, 512, 512, 512, 1e6, 64, ROPE_NEOX, 1e-6, 1, 2,
                           replace(arch_constraints("qwen2"), tied_embeddings=True))
    raise KeyError(f"unknown model config '{name}'")
