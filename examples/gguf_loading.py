"""Inspect a checkpoint: format, architecture, tensor types, load-time validation."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
import json
import sys

from realizar_b200.cli import model_info

print(json.dumps(model_info(sys.argv[1]), indent=1, default=str) if len(sys.argv) > 1 else "usage: gguf_loading.py <model.gguf|.apr|.safetensors>")
