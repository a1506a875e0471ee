"""High-level inference: load a checkpoint, pick the backend (GPU engine, else the C++ CPU
engine), apply the chat template, generate, and report the same result record as the reference's
``run_inference`` (text, tokens, counts, timings, tok/s, format, used_gpu; src/infer/mod.rs:44-210,
src/infer/inference_result.rs:4-31)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, List, Optional, Sequence

from .formats.detect import detect_format, load_model
from .models.weights import ModelWeights
from .serving.chat_template import ChatMessage, ChatTemplate, RawTemplate, auto_detect_template, create_template, detect_format_from_vocab
from .serving.tokenizer import BPETokenizer, ByteTokenizer, tokenizer_from_gguf
from .utils.trace import InferenceTracer

VALID_EXTENSIONS = (".gguf", ".safetensors", ".apr", ".bin", ".json")


@dataclass
class InferenceConfig:
    model_path: str
    prompt: Optional[str] = None
    input_tokens: Optional[Sequence[int]] = None
    max_tokens: int = 32
    temperature: float = 0.0
    top_k: int = 1
    top_p: float = 1.0
    use_gpu: Optional[bool] = None          # None = GPU when available
    chat: bool = False                      # wrap the prompt as a single user turn
    system_prompt: Optional[str] = None
    trace: bool = False
    trace_output: Optional[str] = None
    max_seq_len: int = 2048
    verbose: bool = False
    kv_dtype: str = "bf16"                 # "q8": int8 KV cache on the GPU engine

    def with_prompt(self, p): self.prompt = p; return self
    def with_max_tokens(self, n): self.max_tokens = n; return self
    def with_temperature(self, t): self.temperature = t; return self
    def without_gpu(self): self.use_gpu = False; return self


@dataclass
class InferenceResult:
    text: str
    tokens: List[int]
    input_token_count: int
    generated_token_count: int
    inference_ms: float
    tok_per_sec: float
    load_ms: float
    format: str
    used_gpu: bool
    trace_events: Optional[list] = None


def validate_model_path(path: str) -> Path:
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"model not found: {path}")
    if p.is_file() and p.suffix.lower() not in VALID_EXTENSIONS:
        raise ValueError(f"unsupported model extension '{p.suffix}' (expected one of {', '.join(VALID_EXTENSIONS)})")
    return p


def build_tokenizer(w: ModelWeights):
    g = w._keepalive
    if g is not None and hasattr(g, "get") and hasattr(g, "architecture"):
        t = tokenizer_from_gguf(g)
        if t is not None:
            return t
    if w.vocabulary:
        return BPETokenizer(w.vocabulary, w.metadata.get("merges"), bos_token_id=w.config.bos_token_id, eos_token_id=w.config.eos_token_id)
    return ByteTokenizer(w.config.vocab_size, w.config.eos_token_id)


def build_template(w: ModelWeights, model_name: str = "") -> ChatTemplate:
    tc = w.metadata.get("tokenizer_config") or {}
    if tc.get("chat_template"):
        from .serving.chat_template import HuggingFaceTemplate
        return HuggingFaceTemplate.from_tokenizer_config(tc)
    fmt = auto_detect_template(model_name or w.config.architecture).format
    if fmt == "raw" and w.vocabulary:
        fmt = detect_format_from_vocab(w.vocabulary)
    return create_template(fmt)


class LLM:
    """A loaded model with tokenizer, chat template and a generation backend."""

    def __init__(self, model_path: str, use_gpu: Optional[bool] = None, max_seq_len: int = 2048, max_batch: int = 4, kv_dtype: str = "bf16"):
        import torch
        t0 = time.perf_counter()
        self.path = validate_model_path(model_path)
        self.format = detect_format(self.path)
        self.weights = load_model(self.path)
        self.cfg = self.weights.config
        self.tokenizer = build_tokenizer(self.weights)
        self.template = build_template(self.weights, self.path.stem)
        if use_gpu is None:
            # automatic choice: the GPU when there is one, unless the model is so small that moving it there costs more than
            # running it here (the hybrid dispatch heuristic; weights count as operands that are not on the device yet)
            from .runtime.memory import ComputeBackend, HybridScheduler
            pick = HybridScheduler(gpu_available=torch.cuda.is_available()).choose(self.weights.total_bytes())
            self.used_gpu = pick == ComputeBackend.GPU
        else:
            self.used_gpu = bool(use_gpu)
        self.max_seq_len = min(max_seq_len, self.cfg.context_length)
        if self.used_gpu:
            from .runtime.engine import DecodeEngine, EngineConfig
            self.engine = DecodeEngine(self.weights, EngineConfig(max_batch=max_batch, max_seq_len=self.max_seq_len, kv_dtype=kv_dtype))
            self.cpu = None
        else:
            from .models.cpu_model import CpuModel
            self.engine, self.cpu = None, CpuModel(self.weights, self.max_seq_len)
        self.load_ms = 1e3 * (time.perf_counter() - t0)

    def encode_prompt(self, prompt: str, chat: bool = False, system: Optional[str] = None) -> List[int]:
        if chat:
            msgs = ([ChatMessage.system(system)] if system else []) + [ChatMessage.user(prompt)]
            prompt = self.template.format_conversation(msgs)
        ids = self.tokenizer.encode(prompt)
        if not ids:
            raise ValueError("prompt is empty after tokenisation")
        return ids[-(self.max_seq_len - 1):]

    def generate_tokens(self, ids: Sequence[int], max_tokens: int = 32, temperature: float = 0.0, top_k: int = 1, top_p: float = 1.0,
                        on_token: Optional[Callable[[int], None]] = None, tracer: Optional[InferenceTracer] = None) -> List[int]:
        eos = self.cfg.eos_token_id
        max_tokens = max(1, min(max_tokens, self.max_seq_len - len(ids)))
        if self.engine is not None:
            from .runtime.engine import SamplingParams
            sp = SamplingParams(temperature, top_k, top_p, max_tokens=max_tokens, stop_token_ids=[eos] if eos is not None else [])
            if tracer:
                tracer.enter("TRANSFORMER_BLOCK", tokens=len(ids))
            out = self.engine.generate(list(ids), sp, on_token)
            if tracer:
                tracer.exit("TRANSFORMER_BLOCK", generated=len(out))
            return out
        if temperature <= 0 or top_k == 1:
            if tracer:
                tracer.enter("TRANSFORMER_BLOCK", tokens=len(ids))
            out, _, _ = self.cpu.generate_greedy(list(ids), max_tokens, eos)
            if tracer:
                tracer.exit("TRANSFORMER_BLOCK", generated=len(out), layer_norms=[float(x) for x in self.cpu.layer_trace()])
            if on_token:
                for t in out:
                    on_token(t)
            return out
        from .serving.sampling import GenerationConfig, SamplerChain
        chain = SamplerChain(GenerationConfig(max_tokens=max_tokens, temperature=temperature, top_k=top_k, top_p=top_p))
        logits = self.cpu.prefill(list(ids))
        out: List[int] = []
        for i in range(max_tokens):
            t = chain.sample(logits, list(ids) + out)
            out.append(t)
            if on_token:
                on_token(t)
            if t == eos:
                break
            logits = self.cpu.forward(t, len(ids) + i)
        return out

    def generate(self, prompt: str, **kw) -> str:
        chat, system = kw.pop("chat", False), kw.pop("system", None)
        toks = self.generate_tokens(self.encode_prompt(prompt, chat, system), **kw)
        eos = self.cfg.eos_token_id
        return self.tokenizer.decode([t for t in toks if t != eos])


def run_inference(config: InferenceConfig) -> InferenceResult:
    tracer = InferenceTracer(enabled=config.trace)
    tracer.enter("LOAD", path=str(config.model_path))
    llm = LLM(config.model_path, config.use_gpu, config.max_seq_len, max_batch=1, kv_dtype=config.kv_dtype)
    tracer.exit("LOAD", format=llm.format, load_ms=llm.load_ms)
    tracer.enter("TOKENIZE")
    if config.input_tokens is not None:
        ids = list(config.input_tokens)
    elif config.prompt is not None:
        ids = llm.encode_prompt(config.prompt, config.chat, config.system_prompt)
    else:
        raise ValueError("either prompt or input_tokens is required")
    tracer.exit("TOKENIZE", input_tokens=len(ids))
    t0 = time.perf_counter()
    out = llm.generate_tokens(ids, config.max_tokens, config.temperature, config.top_k, config.top_p, tracer=tracer)
    ms = 1e3 * (time.perf_counter() - t0)
    tracer.enter("DECODE")
    eos = llm.cfg.eos_token_id
    text = llm.tokenizer.decode([t for t in out if t != eos]).strip("\x00")
    tracer.exit("DECODE", chars=len(text))
    if config.trace_output:
        tracer.write(config.trace_output)
    return InferenceResult(text, list(ids) + out, len(ids), len(out), ms, len(out) / (ms / 1e3) if ms > 0 else 0.0, llm.load_ms, llm.format,
                           llm.used_gpu, tracer.events if config.trace else None)


def run_batch_inference(configs: Sequence[InferenceConfig]) -> List[InferenceResult]:
    return [run_inference(c) for c in configs]
