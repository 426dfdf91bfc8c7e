"""The CPU oracle against the reference's own known-answer vectors
(tests/golden/reference_kats.json) and against independent arithmetic."""
import json
import math
from pathlib import Path

import numpy as np
import pytest

from tuckmill_b200 import testing as T

KATS = json.loads((Path(__file__).parent / "golden" / "reference_kats.json").read_text())


def num(v):
    return float(v) if isinstance(v, str) else v


def test_f16_decode_table(oracle):
    for bits, want in KATS["f16_decode"]["cases"]:
        got = oracle.f16_to_f32(int(bits, 16))
        want = num(want)
        assert (math.isnan(got) and math.isnan(want)) or got == want, bits


def test_f16_encode_tables(oracle):
    for key in ("f16_encode", "f16_encode_device_list"):
        for value, bits in KATS[key]["cases"]:
            assert oracle.f32_to_f16_bits(num(value)) == int(bits, 16), (key, value)


def test_f16_codec_agrees_with_ieee_on_every_pattern(oracle):
    """Beyond the KATs: all 65536 patterns decode like IEEE binary16, and
    random f32 values encode like a correctly rounded RNE conversion."""
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits], np.float32)
    nan = np.isnan(want)
    assert np.array_equal(nan, np.isnan(got)) and np.array_equal(got[~nan], want[~nan])
    assert np.array_equal(np.signbit(got[~nan]), np.signbit(want[~nan]))
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 3e4, 1e6)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16_bits(v) for v in vals], np.uint16)
    assert np.array_equal(got, want)


def test_q8_0_dequant_kat(oracle):
    k = KATS["q8_0_dequant"]
    q = np.zeros((1, 32), np.int8)
    q[0, :3] = k["q_head"]
    d = np.array([[int(k["d_bits"], 16)]], np.uint16).view(np.float16)
    out = oracle.dequant_q8_0(T.q8_0_from_parts(d, q))
    assert out.size == k["elems"] and list(out[:3]) == k["out_head"] and np.all(out[3:] == 0)
    raw = T.boundary_weights(1, 5, 96)
    np.testing.assert_array_equal(oracle.dequant_q8_0(raw).reshape(5, 96), T.q8_0_dequant(raw))


def test_gemv_ones_is_exactly_64_and_zero_cases(oracle):
    k = KATS["gemv_ones"]
    raw = T.q8_0_from_parts(np.full((1, 1), k["d"], np.float16), np.full((1, 32), k["q"], np.int8))
    assert oracle.dot_q8_0_x_f32(raw, np.full(32, k["x"], np.float32)) == k["y"]
    raw = T.q8_0_matrix(1, 2, 3, 64)
    assert np.all(oracle.matmul_q8_0(raw, 3, 64, np.zeros(64, np.float32)) == 0.0)
    zero = T.q8_0_from_parts(np.ones((1, 2), np.float16), np.zeros((1, 64), np.int8))
    assert oracle.dot_q8_0_x_f32(zero, np.ones(64, np.float32)) == 0.0


def test_dot_follows_the_reference_order_exactly(oracle):
    """Per block a sequential f32 sum from 0.0, then acc += d * block_sum, blocks
    in order, no fused multiply-add (crates/tuckcore/src/kernels.rs:186-204)."""
    rows, cols = 7, 256
    raw = T.q8_0_matrix(3, 5, rows, cols)
    x = T.activations(3, 6, cols)
    d = np.ascontiguousarray(raw[:, :, :2]).view(np.float16).reshape(rows, cols // 32).astype(np.float32)
    q = np.ascontiguousarray(raw[:, :, 2:]).view(np.int8).reshape(rows, cols // 32, 32).astype(np.float32)
    want = np.zeros(rows, np.float32)
    for r in range(rows):
        acc = np.float32(0)
        for b in range(cols // 32):
            s = np.float32(0)
            for l in range(32):
                s = np.float32(s + np.float32(q[r, b, l] * x[b * 32 + l]))
            acc = np.float32(acc + np.float32(d[r, b] * s))
        want[r] = acc
    got = oracle.matmul_q8_0(raw, rows, cols, x, threads=1)
    np.testing.assert_array_equal(got, want)
    # batched and threaded calls change no bit
    X = T.activations(3, 7, 19 * cols).reshape(19, cols)
    Y = oracle.matmul_q8_0(raw, rows, cols, X, threads=3)
    for b in range(19):
        np.testing.assert_array_equal(Y[b], oracle.matmul_q8_0(raw, rows, cols, X[b], threads=1))


def test_malformed_shapes_are_rejected(oracle):
    """crates/tuckcore/src/kernels.rs:560-587."""
    row = np.zeros(68, np.uint8)
    with pytest.raises(ValueError):
        oracle.dot_q8_0_x_f32(row[:33], np.zeros(32, np.float32))
    with pytest.raises(ValueError):
        oracle.dot_q8_0_x_f32(row[:0], np.zeros(0, np.float32))
    with pytest.raises(ValueError):
        oracle.dot_q8_0_x_f32(row, np.zeros(32, np.float32))
    with pytest.raises(ValueError):
        oracle.dot_q8_0_x_f32(row, np.zeros(65, np.float32))


def test_rmsnorm_rope_silu_argmax_kats(oracle):
    k = KATS["rmsnorm"]
    y = oracle.rmsnorm(np.array(k["x"], np.float32), np.array(k["w"], np.float32), k["eps"])
    np.testing.assert_allclose(y, np.array(k["x"]) / math.sqrt(k["rms_sq"]), atol=1e-6)
    k = KATS["rope"]
    x = oracle.rope_apply(np.array(k["x"], np.float32), k["pos"], np.array(k["inv_freq"], np.float32))
    s3, c3, s15, c15 = math.sin(3), math.cos(3), math.sin(1.5), math.cos(1.5)
    np.testing.assert_allclose(x, [c3 - 0.5 * s3, -1.5 * s15, s3 + 0.5 * c3, 1.5 * c15], atol=1e-6)
    assert abs(float(np.sum(x * x)) - float(np.sum(np.square(k["x"])))) < 1e-5
    assert abs(oracle.silu(0.0)) < 1e-8 and abs(oracle.silu(10.0) - 10.0) < 1e-3
    assert abs(oracle.gelu_tanh(1.0) - 0.841192) < 1e-5
    for vals, want in KATS["argmax"]["cases"]:
        assert oracle.argmax(np.array([num(v) for v in vals], np.float32)) == want
    inv = oracle.rope_inv_freq(128, 1e6)
    want = (1.0 / np.power(np.float64(np.float32(1e6)), 2.0 * np.arange(64) / 128.0)).astype(np.float32)
    np.testing.assert_array_equal(inv, want)


def test_attention_head_matches_direct_softmax(oracle):
    hd, cap = 32, 20
    k = T.activations(0, 1, cap * hd).reshape(cap, hd)
    v = T.activations(0, 2, cap * hd).reshape(cap, hd)
    q = T.activations(0, 3, hd)
    for start, seq in ((0, 1), (0, 13), (5, 13), (12, 13)):
        got = oracle.attend_head(q, k, v, start, seq, 0.25)
        s = (k[start:seq].astype(np.float64) @ q.astype(np.float64)) * 0.25
        w = np.exp(s - s.max())
        w /= w.sum()
        np.testing.assert_allclose(got, w @ v[start:seq].astype(np.float64), rtol=2e-5, atol=2e-6)


def test_forward_is_deterministic_and_chunking_changes_nothing(oracle, tmp_path):
    """crates/tuckcore/src/forward.rs:1141-1186 (streamed == resident, bit exact)
    restated for this oracle's batched prefill."""
    for shape in (T.TINY_QWEN3, T.TINY_GEMMA3):
        path = tmp_path / f"{shape.arch}.gguf"
        T.write_gguf(path, shape, seed=4, norm_jitter=0.1)
        toks = T.token_ids(1, 21, shape.vocab)
        m = oracle.Model(path, threads=2)
        m.reset(32)
        a = m.forward(toks)
        m.reset(32)
        for t in toks[:-1]:
            m.forward([t], want_logits=False)
        b = m.forward([toks[-1]])
        np.testing.assert_array_equal(a, b)
        m.reset(32)
        m.forward(toks[:9], want_logits=False)
        np.testing.assert_array_equal(m.forward(toks[9:]), a)
        with pytest.raises(ValueError):
            m.forward([shape.vocab])
        m.reset(4)
        with pytest.raises(ValueError):
            m.forward(toks[:5])


def test_f16_kv_rounding_is_visible(oracle, tmp_path):
    """crates/tuckcore/src/forward.rs:1078-1138."""
    path = tmp_path / "q.gguf"
    T.write_gguf(path, T.TINY_QWEN3, seed=5)
    toks = T.token_ids(2, 12, T.TINY_QWEN3.vocab)
    outs = []
    for f16 in (True, False):
        m = oracle.Model(path, kv_f16=f16, threads=1)
        m.reset(16)
        outs.append(m.forward(toks))
    assert not np.array_equal(outs[0], outs[1])
    assert np.max(np.abs(outs[0] - outs[1])) < 0.05 * max(1.0, float(np.max(np.abs(outs[1]))))


def test_f16_dot_and_the_reference_fixture_values(oracle, tmp_path):
    """The F16 dot (crates/tuckcore/src/kernels.rs:223-232: widen each weight, multiply,
    add in element order) and the tensor contents of the reference's synthetic fixtures
    (crates/manifest/src/testing.rs:611-614: element e = ((31 e + 7) mod 64 - 32) / 64;
    :678-690: Q8_0 d = 1/128, q = (11 e + 5) mod 128 - 64)."""
    v = T.fixture_values(130)
    assert v[0] == (7 - 32) / 64 and v[1] == (38 - 32) / 64 and v[2] == (5 - 32) / 64 and v[64] == v[0]
    assert np.array_equal(v.astype(np.float16).astype(np.float32), v) and v.min() >= -0.5 and v.max() < 0.5
    blocks = T.fixture_q8_0(3)
    assert blocks.shape == (1, 3, 34) and bytes(blocks[0, 0, :2]) == np.float16(1 / 128).tobytes()
    q = blocks[0, :, 2:].view(np.int8).reshape(-1)
    assert q[0] == 5 - 64 and q[1] == 16 - 64 and q[12] == (11 * 12 + 5) % 128 - 64
    rows, cols = 9, 70
    w = (T.normals(1, 2, 3, 0, rows * cols).reshape(rows, cols) * 0.5).astype(np.float16)
    x = T.activations(4, 5, 2 * cols).reshape(2, cols)
    got = oracle.matmul_f16(w, rows, cols, x)
    for b in range(2):
        for r in range(rows):
            acc = np.float32(0)
            for c in range(cols):
                acc = np.float32(acc + np.float32(w[r, c]) * x[b, c])
            assert got[b, r] == acc
    # the fixture artifact: an F16 model end to end, one token at a time == batched
    path = tmp_path / "f16.gguf"
    T.write_gguf(path, T.TINY_QWEN3, fill="fixture-f16")
    _, tensors, data = T.read_gguf(path)
    ty, dims, off, nbytes = tensors["blk.1.ffn_down.weight"]
    assert ty == T.GGML_F16 and dims == [256, 128] and nbytes == 256 * 128 * 2
    np.testing.assert_array_equal(np.frombuffer(data[off:off + 64], np.float16).astype(np.float32), T.fixture_values(32))
    m = oracle.Model(path, threads=1)
    assert m.weight_type == 1
    toks = T.token_ids(3, 7, 512)
    m.reset(16)
    a = m.forward(toks)
    m.reset(16)
    for t in toks[:-1]:
        m.forward([t], want_logits=False)
    np.testing.assert_array_equal(m.forward([toks[-1]]), a)
    assert np.isfinite(a).all()
