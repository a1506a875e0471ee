"""Grammar-constrained decoding: a JSON schema becomes a GBNF grammar and a per-step token mask."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
import json

import numpy as np

from realizar_b200.serving.grammar import GrammarTokenMasker, grammar_from_json_schema, json_schema_to_gbnf

schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}}, "required": ["name", "age"]}
print(json_schema_to_gbnf(schema).splitlines()[0])
vocab = list('{}":, 0123456789abcdefghijklmnopqrstuvwxyz') + ['"name"', '"age"', "<eos>"]
masker = GrammarTokenMasker(grammar_from_json_schema(schema), vocab, eos_token_id=len(vocab) - 1)
rng, text = np.random.default_rng(0), ""
for _ in range(200):                       # random "logits": the mask alone keeps the output valid
    logits = masker.apply(rng.normal(size=len(vocab)))
    if masker.matcher.is_complete:
        logits[-1] += 4
    t = int(np.argmax(logits))
    masker.accept_token(t)
    if t == len(vocab) - 1:
        break
    text += vocab[t]
print(text, "->", json.loads(text))
