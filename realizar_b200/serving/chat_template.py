"""Chat templates: conversation -> prompt string for the model families the engine serves.

Formats: ChatML (Qwen2, OpenHermes, Yi), Qwen3 with thinking disabled, Llama-2, Llama-3,
Mistral, Zephyr (TinyLlama, StableLM), Phi (``Instruct:/Output:``), Alpaca, Raw, and any
HuggingFace Jinja2 template from ``tokenizer_config.json``.  User content is sanitised so that it
cannot smuggle control tokens (``<|`` gets a zero-width space), and inputs are bounded
(100 KB per message, 10 000 messages).

Behavioural parity with the reference's ``chat_template`` module (formats and detection rules:
src/chat_template.rs:45-400, src/chat_template_helpers.rs:52-162, src/chat_template_llama2.rs:6-430).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence

MAX_MESSAGE_BYTES = 100 * 1024
MAX_MESSAGES = 10_000


class ChatTemplateError(ValueError):
    pass


@dataclass
class ChatMessage:
    role: str
    content: str
    name: Optional[str] = None

    @classmethod
    def system(cls, c): return cls("system", c)
    @classmethod
    def user(cls, c): return cls("user", c)
    @classmethod
    def assistant(cls, c): return cls("assistant", c)


@dataclass
class SpecialTokens:
    bos_token: Optional[str] = None
    eos_token: Optional[str] = None
    unk_token: Optional[str] = None
    pad_token: Optional[str] = None
    im_start_token: Optional[str] = None
    im_end_token: Optional[str] = None
    inst_start: Optional[str] = None
    inst_end: Optional[str] = None
    sys_start: Optional[str] = None
    sys_end: Optional[str] = None


def sanitize_special_tokens(text: str) -> str:
    """Break ``<|`` so user text cannot form a control token (``<|im_end|>`` etc.)."""
    return text.replace("<|", "<​|")


def _check(messages: Sequence[ChatMessage]) -> List[ChatMessage]:
    if len(messages) > MAX_MESSAGES:
        raise ChatTemplateError(f"too many messages ({len(messages)} > {MAX_MESSAGES})")
    out = []
    for m in messages:
        if isinstance(m, dict):
            m = ChatMessage(m.get("role", "user"), m.get("content", "") or "", m.get("name"))
        if len(m.content.encode("utf-8", "ignore")) > MAX_MESSAGE_BYTES:
            raise ChatTemplateError(f"message exceeds {MAX_MESSAGE_BYTES} bytes")
        out.append(m)
    return out


class ChatTemplate:
    format = "raw"
    supports_system_prompt = True
    special_tokens = SpecialTokens()

    def format_message(self, role: str, content: str) -> str:
        return sanitize_special_tokens(content)

    def format_conversation(self, messages: Sequence[ChatMessage]) -> str:
        return "".join(self.format_message(m.role, m.content) for m in _check(messages))


class RawTemplate(ChatTemplate):
    pass


class ChatMLTemplate(ChatTemplate):
    format = "chatml"
    special_tokens = SpecialTokens(bos_token="<|endoftext|>", eos_token="<|im_end|>", im_start_token="<|im_start|>", im_end_token="<|im_end|>")

    def format_message(self, role, content):
        return f"<|im_start|>{role}\n{sanitize_special_tokens(content)}<|im_end|>\n"

    def format_conversation(self, messages):
        return "".join(self.format_message(m.role, m.content) for m in _check(messages)) + "<|im_start|>assistant\n"


class Qwen3NoThinkTemplate(ChatMLTemplate):
    format = "qwen3_nothink"

    def format_conversation(self, messages):
        return "".join(self.format_message(m.role, m.content) for m in _check(messages)) + "<|im_start|>assistant\n<think>\n</think>\n"


class Llama2Template(ChatTemplate):
    format = "llama2"
    special_tokens = SpecialTokens(bos_token="<s>", eos_token="</s>", inst_start="[INST]", inst_end="[/INST]", sys_start="<<SYS>>", sys_end="<</SYS>>")

    def format_message(self, role, content):
        c = sanitize_special_tokens(content)
        if role == "system":
            return f"<<SYS>>\n{c}\n<</SYS>>\n\n"
        if role == "user":
            return f"[INST] {c} [/INST]"
        return f" {c}</s>" if role == "assistant" else c

    def format_conversation(self, messages):
        out, system, in_user = "<s>", None, False
        for i, m in enumerate(_check(messages)):
            c = sanitize_special_tokens(m.content)
            if m.role == "system":
                system = c
            elif m.role == "user":
                if i > 0 and not in_user:
                    out += "<s>"
                out += "[INST] "
                if system is not None:
                    out += f"<<SYS>>\n{system}\n<</SYS>>\n\n"
                    system = None
                out += c + " [/INST]"
                in_user = True
            elif m.role == "assistant":
                out += f" {c}</s>"
                in_user = False
        return out


class MistralTemplate(ChatTemplate):
    format = "mistral"
    supports_system_prompt = False
    special_tokens = SpecialTokens(bos_token="<s>", eos_token="</s>", inst_start="[INST]", inst_end="[/INST]")

    def format_message(self, role, content):
        c = sanitize_special_tokens(content)
        return f"[INST] {c} [/INST]" if role == "user" else (f" {c}</s>" if role == "assistant" else "")

    def format_conversation(self, messages):
        out = "<s>"
        for m in _check(messages):
            out += self.format_message(m.role, m.content)     # system messages are dropped: the format has none
        return out


class Llama3Template(ChatTemplate):
    format = "llama3"
    special_tokens = SpecialTokens(bos_token="<|begin_of_text|>", eos_token="<|eot_id|>")

    def format_message(self, role, content):
        return f"<|start_header_id|>{role}<|end_header_id|>\n\n{sanitize_special_tokens(content)}<|eot_id|>"

    def format_conversation(self, messages):
        return "<|begin_of_text|>" + "".join(self.format_message(m.role, m.content) for m in _check(messages)) + \
            "<|start_header_id|>assistant<|end_header_id|>\n\n"


class ZephyrTemplate(ChatTemplate):
    format = "zephyr"
    special_tokens = SpecialTokens(bos_token="<s>", eos_token="</s>")

    def format_message(self, role, content):
        return f"<|{role}|>\n{sanitize_special_tokens(content)}</s>\n" if role in ("system", "user", "assistant") else ""

    def format_conversation(self, messages):
        return "".join(self.format_message(m.role, m.content) for m in _check(messages)) + "<|assistant|>\n"


class PhiTemplate(ChatTemplate):
    format = "phi"
    special_tokens = SpecialTokens(eos_token="<|endoftext|>")

    def format_message(self, role, content):
        c = sanitize_special_tokens(content)
        return {"user": f"Instruct: {c}\n", "assistant": f"Output: {c}\n", "system": f"{c}\n"}.get(role, "")

    def format_conversation(self, messages):
        return "".join(self.format_message(m.role, m.content) for m in _check(messages)) + "Output:"


class AlpacaTemplate(ChatTemplate):
    format = "alpaca"

    def format_message(self, role, content):
        c = sanitize_special_tokens(content)
        return {"system": f"{c}\n\n", "user": f"### Instruction:\n{c}\n\n", "assistant": f"### Response:\n{c}\n\n"}.get(role, "")

    def format_conversation(self, messages):
        return "".join(self.format_message(m.role, m.content) for m in _check(messages)) + "### Response:\n"


class HuggingFaceTemplate(ChatTemplate):
    """A Jinja2 ``chat_template`` as shipped in ``tokenizer_config.json`` (sandboxed environment)."""
    format = "custom"

    def __init__(self, template_str: str, special_tokens: Optional[SpecialTokens] = None):
        from jinja2.sandbox import ImmutableSandboxedEnvironment
        if len(template_str) > MAX_MESSAGE_BYTES:
            raise ChatTemplateError("template too large")
        self.template_str = template_str
        self.special_tokens = special_tokens or SpecialTokens()
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)

        def raise_exception(msg):
            raise ChatTemplateError(msg)
        env.globals["raise_exception"] = raise_exception
        try:
            self._tpl = env.from_string(template_str)
        except Exception as e:
            raise ChatTemplateError(f"invalid chat template: {e}") from e
        self.supports_system_prompt = "system" in template_str
        self.format = detect_format_from_template(template_str)

    @classmethod
    def from_tokenizer_config(cls, path_or_dict) -> "HuggingFaceTemplate":
        cfg = path_or_dict if isinstance(path_or_dict, dict) else json.loads(Path(path_or_dict).read_text())
        tpl = cfg.get("chat_template")
        if not tpl:
            raise ChatTemplateError("tokenizer config has no chat_template")

        def tok(v):
            return v.get("content") if isinstance(v, dict) else v
        return cls(tpl, SpecialTokens(bos_token=tok(cfg.get("bos_token")), eos_token=tok(cfg.get("eos_token")),
                                      unk_token=tok(cfg.get("unk_token")), pad_token=tok(cfg.get("pad_token"))))

    def format_message(self, role, content):
        return self.format_conversation([ChatMessage(role, content)])

    def format_conversation(self, messages, add_generation_prompt: bool = True):
        msgs = [{"role": m.role, "content": sanitize_special_tokens(m.content)} for m in _check(messages)]
        try:
            return self._tpl.render(messages=msgs, add_generation_prompt=add_generation_prompt,
                                    bos_token=self.special_tokens.bos_token or "", eos_token=self.special_tokens.eos_token or "")
        except ChatTemplateError:
            raise
        except Exception as e:
            raise ChatTemplateError(f"chat template failed to render: {e}") from e


_TEMPLATES = {"chatml": ChatMLTemplate, "qwen3_nothink": Qwen3NoThinkTemplate, "llama2": Llama2Template, "llama3": Llama3Template,
              "mistral": MistralTemplate, "zephyr": ZephyrTemplate, "phi": PhiTemplate, "alpaca": AlpacaTemplate, "raw": RawTemplate,
              "custom": RawTemplate}


def detect_format_from_name(model_name: str) -> str:
    n = model_name.lower()
    if "qwen3" in n:
        return "qwen3_nothink"
    rules = ((("qwen", "openhermes", "yi-"), "chatml"), (("tinyllama", "zephyr", "stablelm"), "zephyr"), (("mistral", "mixtral"), "mistral"),
             (("llama-3", "llama3"), "llama3"), (("llama", "vicuna"), "llama2"), (("phi-", "phi2", "phi3"), "phi"), (("alpaca",), "alpaca"))
    for pats, fmt in rules:
        if any(p in n for p in pats):
            return fmt
    return "raw"


def detect_format_from_tokens(tokens: SpecialTokens) -> str:
    if tokens.im_start_token or tokens.im_end_token:
        return "chatml"
    if tokens.inst_start or tokens.inst_end:
        return "llama2"
    return "raw"


def detect_format_from_template(template: str) -> str:
    if "<|im_start|>" in template:
        return "chatml"
    if "<|start_header_id|>" in template:
        return "llama3"
    if "[INST]" in template:
        return "llama2" if "<<SYS>>" in template else "mistral"
    if "<|user|>" in template:
        return "zephyr"
    return "custom"


def detect_format_from_vocab(vocab: Sequence[str]) -> str:
    v = set(vocab) if not isinstance(vocab, (set, dict)) else vocab
    if "<|im_start|>" in v:
        return "chatml"
    if "<|start_header_id|>" in v:
        return "llama3"
    if "[INST]" in v:
        return "llama2"
    return "raw"


def create_template(fmt: str) -> ChatTemplate:
    return _TEMPLATES.get(fmt, RawTemplate)()


def auto_detect_template(model_name: str) -> ChatTemplate:
    return create_template(detect_format_from_name(model_name))


def format_messages(messages: Sequence, model_name: Optional[str] = None) -> str:
    """Main entry point of the API layer: model-specific prompt for a conversation."""
    tpl = auto_detect_template(model_name) if model_name else RawTemplate()
    return tpl.format_conversation([ChatMessage(**m) if isinstance(m, dict) else m for m in messages])
