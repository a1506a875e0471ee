"""HTTP clients for benchmarking against other inference servers (OpenAI-style ``/v1/completions``
as served by vLLM, Ollama's ``/api/generate``, llama.cpp's ``/completion``) and against this
framework's own server, with per-request timing.  Pure standard library (``urllib``); the
transport is injectable for tests.  Reference parity: ``ModelHttpClient`` /
``CompletionRequest`` / ``OllamaRequest`` / ``InferenceTiming`` (src/http_client/mod.rs:35-432)."""
from __future__ import annotations

import json
import time
import urllib.request
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional


@dataclass
class InferenceTiming:
    text: str
    tokens_generated: int
    total_ms: float
    ttft_ms: Optional[float] = None

    @property
    def tok_per_sec(self) -> float:
        return self.tokens_generated / (self.total_ms / 1e3) if self.total_ms > 0 else 0.0


def _post(url: str, body: dict, timeout: float) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


class ModelHttpClient:
    def __init__(self, base_url: str, timeout: float = 60.0, transport: Optional[Callable[[str, dict, float], dict]] = None):
        self.base, self.timeout, self.post = base_url.rstrip("/"), timeout, transport or _post

    def _timed(self, path: str, body: dict, extract) -> InferenceTiming:
        t = time.perf_counter()
        resp = self.post(self.base + path, body, self.timeout)
        ms = 1e3 * (time.perf_counter() - t)
        text, n = extract(resp)
        return InferenceTiming(text, n, ms)

    def openai_completion(self, model: str, prompt: str, max_tokens: int = 64, temperature: float = 0.0) -> InferenceTiming:
        return self._timed("/v1/completions", {"model": model, "prompt": prompt, "max_tokens": max_tokens, "temperature": temperature},
                           lambda r: (r["choices"][0].get("text", ""), int(r.get("usage", {}).get("completion_tokens", 0))))

    def openai_chat(self, model: str, messages: List[Dict[str, str]], max_tokens: int = 64, temperature: float = 0.0) -> InferenceTiming:
        return self._timed("/v1/chat/completions", {"model": model, "messages": messages, "max_tokens": max_tokens, "temperature": temperature},
                           lambda r: (r["choices"][0]["message"]["content"], int(r.get("usage", {}).get("completion_tokens", 0))))

    def ollama_generate(self, model: str, prompt: str, max_tokens: int = 64) -> InferenceTiming:
        return self._timed("/api/generate", {"model": model, "prompt": prompt, "stream": False, "options": {"num_predict": max_tokens}},
                           lambda r: (r.get("response", ""), int(r.get("eval_count", 0))))

    def llamacpp_completion(self, prompt: str, max_tokens: int = 64) -> InferenceTiming:
        return self._timed("/completion", {"prompt": prompt, "n_predict": max_tokens},
                           lambda r: (r.get("content", ""), int(r.get("tokens_predicted", 0))))

    def native_generate(self, prompt: str, max_tokens: int = 64) -> InferenceTiming:
        return self._timed("/generate", {"prompt": prompt, "max_tokens": max_tokens, "strategy": "greedy"},
                           lambda r: (r.get("text", ""), int(r.get("num_generated", 0))))

    def health(self) -> bool:
        try:
            with urllib.request.urlopen(self.base + "/health", timeout=self.timeout) as r:
                return r.status == 200
        except Exception:
            return False
