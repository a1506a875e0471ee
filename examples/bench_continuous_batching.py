"""Convoy and saturation tests of the continuous-batching loop (fake engine: no model needed)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
import json

from realizar_b200.runtime.scheduler import FakeEngine, ServingEngine
from realizar_b200.utils.benchlib import convoy_test, saturation_test

s = ServingEngine(FakeEngine(max_batch=8, vocab=1000)).start()
print(json.dumps(convoy_test(s, vocab=900), indent=1))
print(json.dumps(saturation_test(s, concurrency=16, requests=64, vocab=900), indent=1))
s.stop()
