"""The C++ host library (quantisers, fused dots, GGUF / APR parsers, CPU decoder) under AddressSanitizer +
UndefinedBehaviorSanitizer: a second build of the library is loaded in a child process with the sanitizer runtime preloaded and
driven through the same Python entry points as the regular tests, including truncated and corrupted files.  Any report from
the sanitizers makes the child exit non-zero."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

EXERCISE = textwrap.dedent("""
    import sys
    import numpy as np
    sys.path.insert(0, %r)
    from realizar_b200 import quant
    from realizar_b200.quant import QType
    from realizar_b200.formats import gguf as G
    from realizar_b200.models.config import named_config
    from realizar_b200.models.cpu_model import CpuModel
    from realizar_b200.models.weights import synthetic_weights, weights_to_gguf

    rng = np.random.default_rng(0)
    for qt in (QType.Q4_0, QType.Q4_1, QType.Q5_0, QType.Q5_1, QType.Q8_0, QType.Q4_K, QType.Q5_K, QType.Q6_K):
        for n, k in ((3, 256), (5, 768), (1, 2560)):
            w = rng.standard_normal((n, k)).astype(np.float32)
            q = quant.quantize(w, qt)
            d = quant.dequantize(q, qt, (n, k))
            x = rng.standard_normal(k).astype(np.float32)
            y = quant.matvec(q, qt, n, k, x)
            assert np.abs(y - d @ x).max() < 0.05 * np.abs(d @ x).max() + 0.5, (qt, n, k)
    for name in ("tiny-llama", "tiny-phi2"):
        w = synthetic_weights(named_config(name), scheme="Q4_K_M", seed=0)
        m = CpuModel(w, 64)
        out = m.generate_greedy([1, 5, 9, 2], 6)
        assert len(out[0]) == 6
        m.close()
    blob = weights_to_gguf(w)
    model = G.GGUFModel.from_bytes(blob)
    assert len(model.tensors) > 4
    rejected = 0
    for cut in (0, 3, 8, 24, 100, 1000, len(blob) // 2, len(blob) - 1):
        try:
            G.GGUFModel.from_bytes(blob[:cut])
        except Exception:
            rejected += 1
    for _ in range(40):
        b = bytearray(blob[:8192])
        for i in rng.integers(4, len(b), 24):
            b[i] = int(rng.integers(0, 256))
        try:
            G.GGUFModel.from_bytes(bytes(b))
        except Exception:
            rejected += 1
    assert rejected >= 8
    # APR v2 container: build one (plain and LZ4-compressed), parse it back, then truncated and corrupted copies
    from realizar_b200.formats import apr as A
    for comp in (None, "lz4"):
        bld = A.AprBuilder({"architecture": "llama", "hidden_size": 64, "vocab_size": 10}, compression=comp)
        bld.add_tensor_raw("model.embed_tokens.weight", (10, 64), 0, rng.standard_normal((10, 64)).astype(np.float32))
        bld.add_tensor_raw("model.norm.weight", (64,), 0, np.ones(64, np.float32))
        ab = bld.build()
        am = A.AprModel.from_bytes(ab)
        assert am.tensor_data("model.norm.weight").size == 64 * 4
        for cut in (0, 7, 31, 64, len(ab) // 2, len(ab) - 3):
            try:
                A.AprModel.from_bytes(ab[:cut])
            except Exception:
                rejected += 1
        for _ in range(30):
            b = bytearray(ab)
            for i in rng.integers(0, len(b), 12):
                b[i] = int(rng.integers(0, 256))
            try:
                m2 = A.AprModel.from_bytes(bytes(b))
                for nm in ("model.embed_tokens.weight", "model.norm.weight"):
                    try:
                        m2.tensor_data(nm)
                    except Exception:
                        pass
            except Exception:
                rejected += 1
    print("SANITIZED-OK", rejected)
""") % ROOT


def _runtime(name: str) -> str:
    out = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True)
    path = out.stdout.strip()
    return path if out.returncode == 0 and os.path.isabs(path) and os.path.exists(path) else ""


def test_host_library_under_address_and_ub_sanitizers():
    asan = _runtime("libasan.so")
    if not asan:
        pytest.skip("no AddressSanitizer runtime with this compiler")
    from realizar_b200 import _build
    try:
        lib = _build.build_cpu(sanitize="address")
    except subprocess.CalledProcessError:
        pytest.skip("the sanitizer flavour of the host library does not build here")
    # libstdc++ has to be there when the sanitizer runtime starts (it wraps __cxa_throw; the interpreter itself is not linked to it)
    preload = ":".join(p for p in (asan, _runtime("libstdc++.so.6") or _runtime("libstdc++.so")) if p)
    env = dict(os.environ, LD_PRELOAD=preload, RLZ_CPU_LIB=str(lib), ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=23",
               UBSAN_OPTIONS="halt_on_error=1:exitcode=24:print_stacktrace=1", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-c", EXERCISE], capture_output=True, text=True, env=env, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0 and "SANITIZED-OK" in r.stdout, tail
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error:" not in r.stderr, tail


def test_thread_pool_under_thread_sanitizer(tmp_path):
    """The host library's spin-then-sleep thread pool under ThreadSanitizer, driven by a small C++ program (no interpreter in
    the process): three caller threads issue batched products and parallel loops at once; every result must equal the
    single-caller one and the sanitizer must stay silent."""
    if not _runtime("libtsan.so"):
        pytest.skip("no ThreadSanitizer runtime with this compiler")
    csrc = os.path.join(ROOT, "realizar_b200", "csrc")
    exe = str(tmp_path / "pool_stress")
    build = subprocess.run(["g++", "-O1", "-g", "-fsanitize=thread", "-std=c++17", "-pthread", "-fno-math-errno", "-I", csrc, "-o", exe,
                            os.path.join(ROOT, "tests", "native", "pool_stress.cpp"), os.path.join(csrc, "quant_cpu.cpp")],
                           capture_output=True, text=True, timeout=600)
    if build.returncode != 0:
        pytest.skip("the ThreadSanitizer build of the stress program does not link here: " + build.stderr[-300:])
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66"))
    if "FATAL: ThreadSanitizer" in r.stderr and "unexpected memory mapping" in r.stderr:
        pytest.skip("ThreadSanitizer cannot map its shadow memory in this environment")
    assert r.returncode == 0 and "POOL-STRESS OK" in r.stdout, (r.stdout + r.stderr)[-2000:]
    assert "ThreadSanitizer" not in r.stderr, r.stderr[-2000:]
