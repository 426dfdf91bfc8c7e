"""CPU-only checks of the host side: synthetic artifacts, GGUF reading, planner
admission, the C ABI's exported surface, selection strings."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from tuckmill_b200 import cuda, engine as E, testing as T

ROOT = Path(__file__).resolve().parent.parent


def test_generator_is_a_pure_function_of_seed_tensor_and_index():
    a = T.q8_0_matrix(0, 3, 64, 256)
    b = T.q8_0_rows(0, 3, 16, 20, 256)
    np.testing.assert_array_equal(a[16:36], b)
    assert not np.array_equal(a, T.q8_0_matrix(1, 3, 64, 256))
    assert not np.array_equal(a, T.q8_0_matrix(0, 4, 64, 256))
    q = np.ascontiguousarray(a[:, :, 2:]).view(np.int8)
    assert q.min() >= -127 and q.max() <= 127
    big = T.uniform_quants(0, 9, 0, 1 << 20)
    assert big.min() == -127 and big.max() == 127 and abs(float(big.mean())) < 0.5
    d = T.block_scales(0, 9, 0, 1 << 16).astype(np.float32)
    assert abs(d.mean() * 127 / (0.02 * np.sqrt(2 / np.pi)) - 1) < 0.02  # E|N(0, 0.02)|
    assert (d < 6.1e-5).mean() > 0.2  # f16 subnormal scales are kept
    x = T.activations(0, 1, 1 << 16)
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1) < 0.02


def test_gguf_round_trip_and_plan(tmp_path):
    path = tmp_path / "t.gguf"
    index = T.write_gguf(path, T.TINY_GEMMA3, seed=2)
    meta, tensors, data = T.read_gguf(path)
    assert meta["general.architecture"] == "gemma3" and meta["gemma3.attention.sliding_window"] == 8
    assert "output.weight" not in tensors and set(tensors) == set(index)
    ty, dims, off, nbytes = tensors["blk.3.ffn_down.weight"]
    assert ty == 8 and dims == [128, 64] and nbytes == 64 * 4 * 34 and off % 32 == 0
    info = E.plan(path, 64, 8 << 30)
    s = T.TINY_GEMMA3
    assert info.architecture == b"gemma3" and info.layers == 6 and info.vocab == 256
    assert info.plan_state == s.layers * 2 * s.kv_heads * 64 * s.head_dim * 2
    mats = sum(cuda.packed_bytes(o, i) for l in range(s.layers) for o, i in
               [(s.heads * s.head_dim + 2 * s.kv_heads * s.head_dim, s.hidden), (s.hidden, s.heads * s.head_dim),
                (2 * s.ffn, s.hidden), (s.hidden, s.ffn)]) + cuda.packed_bytes(s.vocab, s.hidden)
    norms = 4 * (s.layers * (4 * s.hidden + 2 * s.head_dim) + s.hidden)
    assert info.plan_weights == mats + norms


def test_admission_rule_r_plus_u_plus_h(tmp_path):
    """R + U + H <= B with H = max(12.5% B, 192 MiB) (crates/planner/src/lib.rs:
    75-110, crates/manifest/src/plan.rs:68-96)."""
    path = tmp_path / "t.gguf"
    T.write_gguf(path, T.TINY_QWEN3, seed=2)
    B = 64 << 30
    info = E.plan(path, 128, B)
    assert info.safety_reserve == B // 8 and info.overhead == 192 << 20
    kv = 2 * 2 * (32 + 32) * 2 * 128
    assert info.reservation == info.plan_weights + kv + (2048 << 20) + (16 << 20)
    small = E.plan(path, 128, 3 << 30)
    assert small.safety_reserve == 3 * (1 << 30) // 8
    with pytest.raises(E.EngineError) as e:
        E.plan(path, 128, 2 << 30)
    assert e.value.code == "MODEL_EXCEEDS_BUDGET"
    with pytest.raises(E.EngineError) as e:
        E.plan(path, 1 << 24, 4 << 30)  # KV alone outgrows the budget
    assert e.value.code == "CONTEXT_EXCEEDS_BUDGET"
    k = __import__("json").loads((ROOT / "tests/golden/reference_kats.json").read_text())["kv_example"]
    assert k["layers"] * k["kv_heads"] * (k["key"] + k["value"]) * k["bytes"] * k["tokens"] == k["total"]


def test_adapters_refuse_what_they_do_not_express(tmp_path):
    for extra, arch in (({"gemma3.final_logit_softcapping": 30.0}, T.TINY_GEMMA3),
                        ({"gemma3.attention.sliding_window_pattern": 4}, T.TINY_GEMMA3)):
        shape = T.DecoderShape(**{**arch.__dict__, "extra_kv": extra})
        path = tmp_path / "bad.gguf"
        T.write_gguf(path, shape, seed=1)
        with pytest.raises(E.EngineError) as e:
            E.plan(path, 16, 8 << 30)
        assert e.value.code == "UNSUPPORTED_ARCHITECTURE"
    shape = T.DecoderShape(**{**T.TINY_QWEN3.__dict__, "arch": "qwen35"})
    path = tmp_path / "hybrid.gguf"
    T.write_gguf(path, shape, seed=1)
    with pytest.raises(E.EngineError) as e:
        E.plan(path, 16, 8 << 30)
    assert e.value.code == "UNSUPPORTED_ARCHITECTURE"
    (tmp_path / "junk.gguf").write_bytes(b"GGUF" + b"\0" * 40)
    with pytest.raises(E.EngineError) as e:
        E.plan(tmp_path / "junk.gguf", 16, 8 << 30)
    assert e.value.code == "INVALID_ARTIFACT"
    trunc = tmp_path / "trunc.gguf"
    T.write_gguf(trunc, T.TINY_QWEN3, seed=1)
    trunc.write_bytes(trunc.read_bytes()[:-4096])
    with pytest.raises(E.EngineError) as e:
        E.plan(trunc, 16, 8 << 30)
    assert e.value.code == "INVALID_ARTIFACT"


def test_library_exports_every_declared_symbol():
    """The shared libraries load and export every entry point the headers declare."""
    for header, lib in (("tm_cuda.h", cuda.load_library()), ("tm_engine.h", E.load_library())):
        text = (ROOT / "include" / header).read_text()
        names = set(re.findall(r"\b(tm_(?:cuda|engine)_[a-z0-9_]+)\s*\(", text))
        assert len(names) > 10
        for n in sorted(names):
            assert hasattr(lib, n), f"{n} declared in {header} but not exported"
    assert cuda.available() >= 0 and isinstance(cuda.runtime_info(), str)
    assert cuda.packed_bytes(3, 64) == 256 + 3 * 2 * 2 and cuda.packed_bytes(3, 48) == 0


def test_no_device_is_a_typed_refusal_not_a_fallback(tmp_path):
    if cuda.available() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(cuda.CudaError) as e:
        cuda.CudaContext(0)
    assert e.value.code == -1
    path = tmp_path / "t.gguf"
    T.write_gguf(path, T.TINY_QWEN3, seed=2)
    with pytest.raises(E.EngineError) as e:
        E.Engine(path, context=16)
    assert e.value.code == "UNAVAILABLE"
    with pytest.raises(E.EngineError) as e:
        E.Engine(path, context=16, kernels="bogus")
    assert e.value.code == "INVALID_REQUEST"


def test_product_never_touches_the_oracle():
    """Only tests/, the smoke check and bench.py's CPU legs may use oracle/."""
    for p in (ROOT / "tuckmill_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".cpp", ".hpp", ".h") and "build" not in p.parts:
            text = p.read_text()
            assert "liboracle" not in text and "import oracle" not in text and "tm_oracle" not in text, p
