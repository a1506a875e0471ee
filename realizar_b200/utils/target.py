"""Deployment targets: detect where the process runs, what each target can do, and generate the
container recipe / build manifest for it.  Reference parity: ``DeployTarget`` /
``TargetCapabilities`` / ``DockerConfig`` / ``BuildManifest`` (src/target.rs:34-443); the WASM
and Cloudflare-worker targets of the reference have no counterpart for a CUDA engine and are
listed as unsupported capabilities rather than emitted."""
from __future__ import annotations

import json
import os
import platform
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Dict, List, Optional


class DeployTarget(Enum):
    NATIVE = "native"
    LAMBDA = "lambda"
    DOCKER = "docker"
    KUBERNETES = "kubernetes"
    WASM = "wasm"

    @classmethod
    def detect(cls, env: Optional[Dict[str, str]] = None) -> "DeployTarget":
        e = os.environ if env is None else env
        if e.get("AWS_LAMBDA_FUNCTION_NAME") or e.get("AWS_LAMBDA_RUNTIME_API"):
            return cls.LAMBDA
        if e.get("KUBERNETES_SERVICE_HOST"):
            return cls.KUBERNETES
        if e.get("REALIZAR_IN_DOCKER") or os.path.exists("/.dockerenv"):
            return cls.DOCKER
        return cls.NATIVE


@dataclass
class TargetCapabilities:
    gpu: bool
    multi_gpu: bool
    filesystem: bool
    threads: bool
    streaming: bool
    max_memory_mb: Optional[int]

    @classmethod
    def of(cls, t: DeployTarget) -> "TargetCapabilities":
        return {DeployTarget.NATIVE: cls(True, True, True, True, True, None), DeployTarget.DOCKER: cls(True, True, True, True, True, None),
                DeployTarget.KUBERNETES: cls(True, True, True, True, True, None), DeployTarget.LAMBDA: cls(False, False, False, True, False, 10240),
                DeployTarget.WASM: cls(False, False, False, False, False, 4096)}[t]

    def supports(self, feature: str) -> bool:
        return bool(getattr(self, feature))


@dataclass
class DockerConfig:
    base_image: str = "nvidia/cuda:12.9.0-runtime-ubuntu24.04"
    python: str = "python3"
    port: int = 8080
    model_path: Optional[str] = None
    gpus: int = 1
    extra_env: Dict[str, str] = field(default_factory=dict)

    def generate_dockerfile(self) -> str:
        env = "".join(f"ENV {k}={v}\n" for k, v in {"REALIZAR_IN_DOCKER": "1", **self.extra_env}.items())
        model = f"COPY {self.model_path} /models/\n" if self.model_path else ""
        arg = f"/models/{os.path.basename(self.model_path)}" if self.model_path else "$MODEL"
        return (f"FROM {self.base_image}\nWORKDIR /app\nCOPY realizar_b200 /app/realizar_b200\nCOPY csrc /app/csrc\n{model}{env}"
                f"RUN {self.python} -c \"import realizar_b200._build as b; b.build_all()\"\nEXPOSE {self.port}\n"
                f"ENTRYPOINT [\"{self.python}\", \"-m\", \"realizar_b200\", \"serve\", \"--host\", \"0.0.0.0\", \"--port\", \"{self.port}\", \"--model\", \"{arg}\"]\n")

    def run_command(self, image: str) -> str:
        return f"docker run --gpus {self.gpus if self.gpus else 'all'} -p {self.port}:{self.port} {image}"


@dataclass
class BuildTarget:
    name: str
    arch: str
    features: List[str]


@dataclass
class BuildManifest:
    version: str
    targets: List[BuildTarget]
    host: str = field(default_factory=platform.machine)

    @classmethod
    def default(cls, version: str) -> "BuildManifest":
        return cls(version, [BuildTarget("cuda-sm100a", "sm_100a", ["tcgen05", "tma", "pdl", "cuda-graphs", "nvlink-p2p"]),
                             BuildTarget("cpu-x86_64", "x86_64", ["avx2", "fma", "threads"])])

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)
