"""Contracts: declarative invariants in ``contracts/*.yaml`` and the checks that hold the code to
them (struct sizes shared between Python and CUDA, block layouts, load-time requirements).
Reference parity: the reference generates pre/post-condition macros from ``contracts/*.yaml`` at
build time and checks kernel structure in ``ptx_parity`` (build.rs:1-60, src/ptx_parity.rs:13-340);
here the same documents are read at test time."""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Dict, List

import yaml

CONTRACT_DIR = Path(__file__).resolve().parents[2] / "contracts"


def load(name: str) -> dict:
    with open(CONTRACT_DIR / f"{name}.yaml") as f:
        return yaml.safe_load(f)


def check_abi(lib=None) -> List[str]:
    """Compare sizeof of every parameter block as compiled with its ctypes mirror.  Returns mismatches."""
    from ..ops import _signatures as S
    if lib is None:
        from .. import ops
        lib = ops.lib()
    bad = []
    for e in load("kernel_abi")["structs"]:
        c_size = int(getattr(lib, e["c"])())
        py_size = ctypes.sizeof(getattr(S, e["py"]))
        if c_size != py_size:
            bad.append(f"{e['py']}: C {c_size} bytes, ctypes {py_size} bytes")
    return bad


def check_block_layouts() -> List[str]:
    from ..quant import BLOCK_SPECS, QType
    from ..quant.device_layout import dev_row_bytes
    doc = load("block_layouts")
    bad = []
    for name, spec in doc["checkpoint_blocks"].items():
        sp = BLOCK_SPECS[QType[name]]
        be, bb = sp.elems, sp.nbytes
        if (bb, be) != (spec["bytes"], spec["elems"]):
            bad.append(f"{name}: code has {bb} bytes / {be} weights, contract {spec['bytes']} / {spec['elems']}")
    for name, expr in doc["device_rows"].items():
        for k in (256, 2560, 8192):
            want = int(eval(expr, {"k": k}))
            got = dev_row_bytes(int(QType[name]), k)
            if want != got or got % doc["alignment"]["device_row_multiple"]:
                bad.append(f"{name} device row at k={k}: code {got}, contract {want}")
    return bad


def required_tensors(fused_qkv: bool, gated: bool, parallel_residual: bool, layers: int) -> List[str]:
    doc = load("model_load")
    per = list(doc["required_per_layer"]["fused_qkv" if fused_qkv else "separate_qkv"])
    if gated:
        per += doc["gated_ffn_extra"]
    if not parallel_residual:
        per += doc["non_parallel_residual_extra"]
    return list(doc["required_global"]) + [f"blk.{l}.{t}" for l in range(layers) for t in per]
