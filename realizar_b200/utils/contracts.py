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


def parse_ptxas_report(text: str) -> List[dict]:
    """Entries of a ptxas ``-v`` report: mangled name, kernel base name, registers, barriers, spill bytes, stack, static smem."""
    import re
    out = []
    pat = re.compile(r"Compiling entry function '(\S+)' for 'sm_100a'\n.*?\n\s+(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads\n"
                     r".*?Used (\d+) registers(?:, used (\d+) barriers)?(?:, \d+ bytes cumulative stack size)?(?:, (\d+) bytes smem)?")
    for m in pat.finditer(text):
        name = m.group(1)
        b = re.search(r"_ZN3rlz(\d+)", name)
        base = name
        if b:
            i = b.end()
            base = name[i:i + int(b.group(1))]
        out.append({"name": name, "kernel": base, "stack": int(m.group(2)), "spill_stores": int(m.group(3)), "spill_loads": int(m.group(4)),
                    "registers": int(m.group(5)), "barriers": int(m.group(6) or 0), "static_smem": int(m.group(7) or 0)})
    return out


def check_kernel_parity(report_dir=None) -> List[str]:
    """Hold the compiled kernels to ``contracts/kernel_parity.yaml``.  Returns the violations; raises FileNotFoundError when the
    build's resource reports are not there (nothing built in this tree yet)."""
    report_dir = Path(report_dir) if report_dir else Path(__file__).resolve().parents[1] / "_lib" / "obj"
    bad, cache = [], {}
    for fam in load("kernel_parity")["families"]:
        path = report_dir / f"{fam['file']}.ptxas.txt"
        if fam["file"] not in cache:
            if not path.exists():
                raise FileNotFoundError(path)
            cache[fam["file"]] = parse_ptxas_report(path.read_text())
        ks = [e for e in cache[fam["file"]] if e["kernel"] == fam["kernel"]]
        tag = fam["kernel"]
        if len(ks) < fam.get("min_instantiations", 1):
            bad.append(f"{tag}: {len(ks)} instantiations, contract wants at least {fam.get('min_instantiations', 1)}")
            continue
        worst = max(e["registers"] for e in ks)
        if worst > fam["max_registers"]:
            bad.append(f"{tag}: {worst} registers > {fam['max_registers']}")
        spill = max(e["spill_stores"] for e in ks)
        if spill > fam.get("max_spill_bytes", 0):
            bad.append(f"{tag}: {spill} bytes of spill stores > {fam.get('max_spill_bytes', 0)}")
        if fam.get("same_static_smem") and len({e["static_smem"] for e in ks}) != 1:
            bad.append(f"{tag}: variants differ in static shared memory {sorted({e['static_smem'] for e in ks})}")
        if fam.get("same_barriers") and len({e["barriers"] for e in ks}) != 1:
            bad.append(f"{tag}: variants differ in barrier count {sorted({e['barriers'] for e in ks})}")
    return bad


def required_tensors(fused_qkv: bool, gated: bool, parallel_residual: bool, layers: int) -> List[str]:
    doc = load("model_load")
    per = list(doc["required_per_layer"]["fused_qkv" if fused_qkv else "separate_qkv"])
    if gated:
        per += doc["gated_ffn_extra"]
    if not parallel_residual:
        per += doc["non_parallel_residual_extra"]
    return list(doc["required_global"]) + [f"blk.{l}.{t}" for l in range(layers) for t in per]
