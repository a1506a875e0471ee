"""Multi-model management: a thread-safe registry of loaded models, an LRU cache with hit/miss
statistics, start-up warm-up with health reporting, and ``pacha://`` / ``file://`` / ``hf://``
model URIs resolved against a local model directory (there is no network client).
Reference parity: ``ModelRegistry`` (src/registry.rs:40-317), ``ModelCache`` (src/cache.rs:43-286),
``ModelWarmer`` / ``WarmupConfig`` / ``ModelHealth`` (src/warmup.rs:47-424), ``PachaUri`` (src/uri.rs:32-455)."""
from __future__ import annotations

import os
import re
import threading
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional


class RegistryError(KeyError):
    pass


@dataclass
class ModelInfo:
    id: str
    name: str
    description: str = ""
    format: str = ""
    loaded: bool = True
    path: Optional[str] = None


class ModelRegistry:
    def __init__(self, default_id: Optional[str] = None):
        self._models: Dict[str, tuple] = {}
        self._lock = threading.RLock()
        self.default_id = default_id

    def register(self, model_id: str, model: Any, tokenizer: Any = None, info: Optional[ModelInfo] = None) -> None:
        with self._lock:
            if model_id in self._models:
                raise RegistryError(f"model '{model_id}' is already registered")
            self._models[model_id] = (model, tokenizer, info or ModelInfo(model_id, model_id))
            if self.default_id is None:
                self.default_id = model_id

    def replace(self, model_id: str, model: Any, tokenizer: Any = None) -> None:
        """Atomic hot reload: readers see the old or the new entry, never a gap."""
        with self._lock:
            if model_id not in self._models:
                raise RegistryError(f"model '{model_id}' not found")
            _, tok, info = self._models[model_id]
            self._models[model_id] = (model, tokenizer or tok, info)

    def unregister(self, model_id: str) -> None:
        with self._lock:
            if self._models.pop(model_id, None) is None:
                raise RegistryError(f"model '{model_id}' not found")
            if self.default_id == model_id:
                self.default_id = next(iter(self._models), None)

    def get(self, model_id: Optional[str] = None) -> tuple:
        with self._lock:
            mid = model_id or self.default_id
            if mid is None or mid not in self._models:
                raise RegistryError(f"model '{mid}' not found")
            m, t, _ = self._models[mid]
            return m, t

    def contains(self, model_id: str) -> bool:
        with self._lock:
            return model_id in self._models

    def list(self) -> List[ModelInfo]:
        with self._lock:
            return [i for _, _, i in self._models.values()]

    def __len__(self) -> int:
        return len(self._models)


@dataclass
class CacheMetrics:
    hits: int = 0
    misses: int = 0
    evictions: int = 0

    @property
    def hit_rate(self) -> float:
        t = self.hits + self.misses
        return self.hits / t if t else 0.0


class ModelCache:
    """LRU cache keyed by ``(path, variant)``; the loader runs outside the lock so that a slow load
    does not block hits on other keys (a second caller of the same key waits on a per-key event)."""

    def __init__(self, capacity: int = 2, on_evict: Optional[Callable[[Any, Any], None]] = None):
        if capacity < 1:
            raise ValueError("capacity must be >= 1")
        self.capacity = capacity
        self._d: "OrderedDict[Any, Any]" = OrderedDict()
        self._loading: Dict[Any, threading.Event] = {}
        self._lock = threading.Lock()
        self.metrics = CacheMetrics()
        self.on_evict = on_evict

    def get_or_load(self, key, loader: Callable[[], Any]):
        while True:
            with self._lock:
                if key in self._d:
                    self._d.move_to_end(key)
                    self.metrics.hits += 1
                    return self._d[key]
                ev = self._loading.get(key)
                if ev is None:
                    self._loading[key] = threading.Event()
                    self.metrics.misses += 1
                    break
            ev.wait()
        try:
            val = loader()
        except BaseException:
            with self._lock:
                self._loading.pop(key).set()
            raise
        with self._lock:
            self._d[key] = val
            while len(self._d) > self.capacity:
                k, v = self._d.popitem(last=False)
                self.metrics.evictions += 1
                if self.on_evict:
                    self.on_evict(k, v)
            self._loading.pop(key).set()
        return val

    def invalidate(self, key) -> bool:
        with self._lock:
            return self._d.pop(key, None) is not None

    def clear(self) -> None:
        with self._lock:
            self._d.clear()

    def __len__(self) -> int:
        return len(self._d)

    def keys(self) -> list:
        return list(self._d)


# -- warm-up ----------------------------------------------------------------------------------------
@dataclass
class WarmupConfig:
    iterations: int = 3
    prompt_tokens: int = 8
    max_tokens: int = 4
    timeout_s: float = 30.0
    sample_requests: List[List[int]] = field(default_factory=list)


@dataclass
class WarmupResult:
    success: bool
    iterations_completed: int
    total_ms: float
    latencies_ms: List[float]
    error: Optional[str] = None

    @property
    def mean_ms(self) -> float:
        return sum(self.latencies_ms) / len(self.latencies_ms) if self.latencies_ms else 0.0

    @property
    def speedup(self) -> float:
        """First (cold) iteration relative to the last (warm) one."""
        return self.latencies_ms[0] / self.latencies_ms[-1] if len(self.latencies_ms) > 1 and self.latencies_ms[-1] > 0 else 1.0


class ModelHealth:
    def __init__(self, unhealthy_after: int = 3):
        self.state, self.consecutive_failures, self.unhealthy_after = "unknown", 0, unhealthy_after
        self.total_requests = self.failed_requests = 0
        self.last_check: Optional[float] = None

    def record(self, ok: bool) -> None:
        self.total_requests += 1
        self.last_check = time.time()
        if ok:
            self.consecutive_failures, self.state = 0, "ready"
        else:
            self.failed_requests += 1
            self.consecutive_failures += 1
            self.state = "unhealthy" if self.consecutive_failures >= self.unhealthy_after else "degraded"

    @property
    def is_ready(self) -> bool:
        return self.state in ("ready", "degraded")


class ModelWarmer:
    """Runs a few generations through ``generate(prompt_tokens, max_tokens)`` before the model takes
    traffic: populates graph captures, page tables and caches, and proves that the path works."""

    def __init__(self, cfg: Optional[WarmupConfig] = None):
        self.cfg = cfg or WarmupConfig()

    def warm(self, generate: Callable[[List[int], int], Any], vocab_size: int = 256, health: Optional[ModelHealth] = None) -> WarmupResult:
        cfg = self.cfg
        t0 = time.perf_counter()
        lats: List[float] = []
        prompts = cfg.sample_requests or [[(7 * i + 3) % max(2, vocab_size - 1) + 1 for i in range(cfg.prompt_tokens)]]
        try:
            for it in range(cfg.iterations):
                t = time.perf_counter()
                generate(list(prompts[it % len(prompts)]), cfg.max_tokens)
                lats.append(1e3 * (time.perf_counter() - t))
                if time.perf_counter() - t0 > cfg.timeout_s:
                    raise TimeoutError(f"warm-up exceeded {cfg.timeout_s}s")
            if health:
                health.record(True)
            return WarmupResult(True, len(lats), 1e3 * (time.perf_counter() - t0), lats)
        except Exception as e:
            if health:
                health.record(False)
            return WarmupResult(False, len(lats), 1e3 * (time.perf_counter() - t0), lats, repr(e))


# -- URIs ---------------------------------------------------------------------------------------------
_NAME = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._\-/]*$")


@dataclass(frozen=True)
class ModelUri:
    scheme: str            # pacha | file | hf | path
    name: str
    version: Optional[str] = None

    @classmethod
    def parse(cls, uri: str) -> "ModelUri":
        if not uri:
            raise ValueError("empty model URI")
        if "://" not in uri:
            return cls("path", uri)
        scheme, rest = uri.split("://", 1)
        if scheme == "file":
            return cls("file", rest)
        if scheme not in ("pacha", "hf"):
            raise ValueError(f"unsupported URI scheme '{scheme}'")
        if scheme == "pacha" and rest.startswith("model/"):
            rest = rest[len("model/"):]
        name, _, ver = rest.partition(":")
        if not name or not _NAME.match(name) or ".." in name:
            raise ValueError(f"invalid model name in URI '{uri}'")
        if _ and not ver:
            raise ValueError("empty version in URI")
        return cls(scheme, name, ver or None)

    def __str__(self) -> str:
        if self.scheme == "path":
            return self.name
        if self.scheme == "file":
            return f"file://{self.name}"
        return f"{self.scheme}://{self.name}" + (f":{self.version}" if self.version else "")


def model_home() -> Path:
    return Path(os.environ.get("REALIZAR_HOME", Path.home() / ".realizar")) / "models"


def resolve_uri(uri: str, home: Optional[Path] = None) -> Path:
    """Map a URI to a local file.  Registry schemes look under ``<home>/<name>[/<version>]`` for
    a single model file; pulling from a remote registry is not available offline."""
    u = ModelUri.parse(uri)
    if u.scheme in ("path", "file"):
        p = Path(u.name)
        if not p.exists():
            raise FileNotFoundError(f"model not found: {p}")
        return p
    base = (home or model_home()) / u.name
    if u.version:
        base = base / u.version
    if base.is_file():
        return base
    if base.is_dir():
        for ext in (".gguf", ".apr", ".safetensors"):
            hits = sorted(base.glob(f"*{ext}"))
            if hits:
                return hits[0] if ext != ".safetensors" or len(hits) == 1 else base
    for ext in (".gguf", ".apr", ".safetensors"):
        if base.with_suffix(ext).is_file():
            return base.with_suffix(ext)
    raise FileNotFoundError(f"model '{u}' is not in the local store {home or model_home()} (remote pull needs a network)")


def list_local_models(home: Optional[Path] = None) -> List[dict]:
    root = home or model_home()
    out = []
    if root.is_dir():
        for p in sorted(root.rglob("*")):
            if p.is_file() and p.suffix.lower() in (".gguf", ".apr", ".safetensors"):
                out.append({"name": str(p.relative_to(root)), "path": str(p), "size_bytes": p.stat().st_size, "format": p.suffix[1:].lower(),
                            "modified": p.stat().st_mtime})
    return out
