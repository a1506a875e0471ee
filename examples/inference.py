"""Generate from a checkpoint (or from a tiny synthetic model when no path is given)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
import sys
import tempfile

from realizar_b200.infer import InferenceConfig, run_inference

if len(sys.argv) > 1:
    path = sys.argv[1]
else:
    from realizar_b200.models.config import named_config
    from realizar_b200.models.weights import synthetic_weights, weights_to_gguf
    from realizar_b200.serving.tokenizer import bytes_to_unicode
    b2u = bytes_to_unicode()
    vocab = [b2u[i] for i in range(256)] + [f"<t{i}>" for i in range(256)]
    path = tempfile.mktemp(suffix=".gguf")
    open(path, "wb").write(weights_to_gguf(synthetic_weights(named_config("tiny-llama"), seed=0, std=0.05), vocabulary=vocab))
r = run_inference(InferenceConfig(path, prompt=sys.argv[2] if len(sys.argv) > 2 else "hello world", max_tokens=16, trace=True))
print(repr(r.text))
print(f"{r.generated_token_count} tokens, {r.tok_per_sec:.1f} tok/s, load {r.load_ms:.0f} ms, format {r.format}, gpu={r.used_gpu}")
