"""Start the HTTP server (demo engine when no model is given) and query it in-process."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
import sys

from fastapi.testclient import TestClient

from realizar_b200.cli import build_app_state
from realizar_b200.serving.api import create_app

state = build_app_state(sys.argv[1] if len(sys.argv) > 1 else None, None, 4, 2048)
client = TestClient(create_app(state))
print(client.get("/health").json())
print(client.post("/v1/chat/completions", json={"model": "default", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8}).json())
print(client.post("/generate", json={"prompt": "abc", "max_tokens": 5, "strategy": "greedy"}).json())
print(client.get("/metrics").text[:300])
state.serving.stop()
