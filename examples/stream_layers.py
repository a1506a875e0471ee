"""Layer streaming with two buffers: a stack of layers whose weights do not all fit "on the device" runs from two buffers while
the next layer's weights are copied in.  With CUDA the copies go on a side stream and overlap with the compute; on a CPU-only
machine the same schedule runs in order.  (The serving engine applies this schedule inside its launch plans when a checkpoint
is larger than the GPU: ``EngineConfig(resident_layers=...)``.)

    python examples/stream_layers.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run from a source checkout
from realizar_b200.runtime.memory import LayerStreamer, StreamingMode, check_vram_sufficient


def main() -> None:
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    layers, dim = 6, 256
    host = [torch.randn(dim, dim) / dim ** 0.5 for _ in range(layers)]
    if dev.type == "cuda":
        host = [w.pin_memory() for w in host]
    plan = check_vram_sufficient(weight_bytes=layers * dim * dim * 4, kv_bytes=0, free_bytes=3 * dim * dim * 4 + (1 << 20), num_layers=layers,
                                 workspace_bytes=1 << 19, headroom=0.0)
    assert plan.mode == StreamingMode.LAYER_STREAMING
    print(f"plan: {plan.mode.value}, {plan.resident_layers} of {layers} layers could stay resident, {plan.layer_bytes} bytes per layer")
    buffers = [torch.empty(dim, dim, device=dev) for _ in range(2)]
    x = torch.randn(4, dim, device=dev)
    state = {"x": x}

    def copy(layer: int, buf: int) -> None:
        buffers[buf].copy_(host[layer], non_blocking=True)

    def compute(layer: int, buf: int) -> None:
        state["x"] = torch.tanh(state["x"] @ buffers[buf])

    LayerStreamer(layers, copy, compute).run()
    if dev.type == "cuda":
        torch.cuda.synchronize()
    want = x.cpu()
    for w in host:
        want = torch.tanh(want @ w)
    err = float((state["x"].cpu() - want).abs().max())
    print(f"streamed result matches the resident one: max |diff| = {err:.2e}")
    assert err < 1e-3


if __name__ == "__main__":
    main()
