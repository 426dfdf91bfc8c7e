"""Seeded synthetic artifacts: Q8_0 tensors, activations and whole GGUF files.

Counterpart of the reference's fixture writer
(crates/manifest/src/testing.rs:225-700), which emits tiny *valid* GGUFs with
deterministic values.  Here the values follow the benchmark's distributions:
quants uniform integers in [-127, 127], one f16 scale |N(0, 0.02)|/127 per
32-quant block, f32 activations N(0, 1).  Every value is a pure function of
``(seed, tensor_id, element index)`` (a splitmix64 counter hash), so a shard of
a tensor can be generated without generating the rest.

The files are ordinary GGUF v3: a tensor's dims are ``[in_dim, out_dim]``
(innermost first, testing.rs:349-351) and a Q8_0 row is ``in_dim/32`` blocks of
``[f16 d little-endian][i8 q x 32]`` (crates/tuckcore/src/tensor.rs:94-104).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

GGML_F32, GGML_F16, GGML_Q8_0 = 0, 1, 8
Q8_BLOCK, Q8_BLOCK_BYTES = 32, 34

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)
_GOLDEN = 0x9E3779B97F4A7C15
_TENSOR_MUL = 0xD1B54A32D192ED03
_STREAM_MUL = 0x8CB92BA72F3D8DD7


def _mix_scalar(z: int) -> int:
    z &= 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def _mix(z: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser over a uint64 array (wrapping arithmetic)."""
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def hashes(seed: int, tensor_id: int, stream: int, start: int, count: int) -> np.ndarray:
    """``count`` 64-bit hashes of counters ``start..start+count`` of one stream."""
    key = _mix_scalar(seed * _GOLDEN + tensor_id * _TENSOR_MUL + stream * _STREAM_MUL + 1)
    idx = np.arange(start, start + count, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return _mix(np.uint64(key) + idx * np.uint64(_GOLDEN))


def uniform_quants(seed: int, tensor_id: int, start: int, count: int) -> np.ndarray:
    """int8 values uniform in [-127, 127]; element e uses 16 bits of hash e//4."""
    assert start % 4 == 0
    h = hashes(seed, tensor_id, 0, start // 4, (count + 3) // 4)
    u16 = h.view("<u2").astype(np.uint32)
    return (((u16 * np.uint32(255)) >> np.uint32(16)).astype(np.int16) - 127).astype(np.int8)[:count]


def normals(seed: int, tensor_id: int, stream: int, start: int, count: int) -> np.ndarray:
    """float64 N(0,1) by Box-Muller on the two 32-bit halves of one hash each."""
    h = hashes(seed, tensor_id, stream, start, count)
    hi = (h >> np.uint64(32)).astype(np.float64)
    lo = (h & np.uint64(0xFFFFFFFF)).astype(np.float64)
    u1 = (hi + 1.0) / 4294967296.0
    u2 = lo / 4294967296.0
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def block_scales(seed: int, tensor_id: int, start: int, count: int) -> np.ndarray:
    """f16 scales |N(0, 0.02)| / 127, rounded to nearest even (subnormals kept)."""
    z = normals(seed, tensor_id, 1, start, count)
    return (np.abs(z * 0.02) / 127.0).astype(np.float32).astype(np.float16)


def activations(seed: int, tensor_id: int, count: int) -> np.ndarray:
    """f32 N(0, 1) activations."""
    return normals(seed, tensor_id, 2, 0, count).astype(np.float32)


def token_ids(seed: int, count: int, vocab: int, tensor_id: int = 0xA11CE) -> np.ndarray:
    h = hashes(seed, tensor_id, 3, 0, count)
    return ((h >> np.uint64(11)) % np.uint64(vocab)).astype(np.uint32)


def q8_0_rows(seed: int, tensor_id: int, row0: int, rows: int, cols: int) -> np.ndarray:
    """Raw GGUF bytes ``[rows, cols/32, 34]`` of rows row0.. of a Q8_0 tensor."""
    assert cols % Q8_BLOCK == 0 and cols > 0
    nb = cols // Q8_BLOCK
    out = np.empty((rows, nb, Q8_BLOCK_BYTES), dtype=np.uint8)
    step = max(1, (1 << 24) // cols)
    for r in range(0, rows, step):
        n = min(step, rows - r)
        q = uniform_quants(seed, tensor_id, (row0 + r) * cols, n * cols)
        d = block_scales(seed, tensor_id, (row0 + r) * nb, n * nb)
        out[r:r + n, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
        out[r:r + n, :, 2:] = q.view(np.uint8).reshape(n, nb, Q8_BLOCK)
    return out


def q8_0_matrix(seed: int, tensor_id: int, rows: int, cols: int) -> np.ndarray:
    return q8_0_rows(seed, tensor_id, 0, rows, cols)


def q8_0_from_parts(d_f16: np.ndarray, q_i8: np.ndarray) -> np.ndarray:
    """Assemble raw bytes from scales ``[rows, cols/32]`` and quants ``[rows, cols]``."""
    rows, nb = d_f16.shape
    out = np.empty((rows, nb, Q8_BLOCK_BYTES), dtype=np.uint8)
    out[:, :, 0:2] = np.ascontiguousarray(d_f16.astype(np.float16)).view(np.uint8).reshape(rows, nb, 2)
    out[:, :, 2:] = np.ascontiguousarray(q_i8.astype(np.int8)).view(np.uint8).reshape(rows, nb, Q8_BLOCK)
    return out


def q8_0_dequant(raw: np.ndarray) -> np.ndarray:
    """f32 ``[rows, cols]`` = d * q of raw ``[rows, nb, 34]`` bytes (exact in f32)."""
    rows, nb, _ = raw.shape
    d = np.ascontiguousarray(raw[:, :, 0:2]).view(np.float16).reshape(rows, nb).astype(np.float32)
    q = np.ascontiguousarray(raw[:, :, 2:]).view(np.int8).astype(np.float32)
    return (d[:, :, None] * q).reshape(rows, nb * Q8_BLOCK)


# --------------------------------------------------------------------------
# Boundary data of the reference's device tests (crates/metal/src/tests.rs:
# 119-162): adversarial scales and quants, restated with this generator.
# --------------------------------------------------------------------------

BOUNDARY_SCALES = np.array(
    [1.0, -0.5, 2.0 ** -12, 65504.0, -65504.0, 5.96e-8, 0.0, -0.0, 448.0, 6e-5], dtype=np.float32
).astype(np.float16)


def boundary_weights(seed: int, rows: int, cols: int) -> np.ndarray:
    """Scales cycle the boundary list; quants include -128, 127 and 0."""
    nb = cols // Q8_BLOCK
    idx = (np.arange(rows * nb) % len(BOUNDARY_SCALES)).reshape(rows, nb)
    d = BOUNDARY_SCALES[idx]
    q = uniform_quants(seed, 0xB0DA, 0, rows * cols).reshape(rows, cols).copy()
    q[:, 0::97] = -128
    q[:, 1::89] = 127
    q[:, 2::83] = 0
    return q8_0_from_parts(d, q)


def boundary_input(seed: int, cols: int) -> np.ndarray:
    """Activations mixing 0, -1, +-1e3 with U(-10, 10)."""
    h = hashes(seed, 0xB1, 4, 0, cols)
    u = ((h >> np.uint64(11)).astype(np.float64) / float(1 << 53) * 20.0 - 10.0).astype(np.float32)
    u[0::7] = 0.0
    u[1::11] = -1.0
    u[2::13] = 1e3
    u[3::17] = -1e3
    return u


# --------------------------------------------------------------------------
# Dense-decoder shapes and GGUF files
# --------------------------------------------------------------------------

@dataclass
class DecoderShape:
    """Geometry of a dense decoder artifact (the metadata an adapter reads)."""

    arch: str  # "qwen3" | "gemma3"
    layers: int
    hidden: int
    ffn: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    rope_base: float = 1e6
    eps: float = 1e-6
    context: int = 4096
    window: int = 0  # gemma3 sliding window
    tied_head: bool = False
    extra_kv: dict = field(default_factory=dict)

    def matrices(self, layer: int) -> list[tuple[str, int, int]]:
        """(name, out_dim, in_dim) of one layer's seven projections."""
        p = f"blk.{layer}."
        qo, kvo, h, f = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.hidden, self.ffn
        return [
            (p + "attn_q.weight", qo, h), (p + "attn_k.weight", kvo, h), (p + "attn_v.weight", kvo, h),
            (p + "attn_output.weight", h, qo), (p + "ffn_gate.weight", f, h), (p + "ffn_up.weight", f, h),
            (p + "ffn_down.weight", h, f),
        ]

    def norms(self, layer: int) -> list[tuple[str, int]]:
        p = f"blk.{layer}."
        out = [(p + "attn_norm.weight", self.hidden), (p + "attn_q_norm.weight", self.head_dim),
               (p + "attn_k_norm.weight", self.head_dim), (p + "ffn_norm.weight", self.hidden)]
        if self.arch == "gemma3":
            out += [(p + "post_attention_norm.weight", self.hidden), (p + "post_ffw_norm.weight", self.hidden)]
        return out

    def decode_weight_bytes(self) -> int:
        """Q8_0 bytes one decode token reads: every projection and the head."""
        per = sum(o * (i // 32) * 34 for _, o, i in self.matrices(0))
        return per * self.layers + self.vocab * (self.hidden // 32) * 34


QWEN3_0_6B = DecoderShape("qwen3", 28, 1024, 3072, 16, 8, 128, 151936, rope_base=1e6, context=40960)
GEMMA3_1B = DecoderShape("gemma3", 26, 1152, 6912, 4, 1, 256, 262144, rope_base=1e6, window=512,
                         tied_head=True, context=32768)
QWEN3_8B = DecoderShape("qwen3", 36, 4096, 12288, 32, 8, 128, 151936, rope_base=1e6, context=40960)
TINY_QWEN3 = DecoderShape("qwen3", 2, 128, 256, 4, 2, 32, 512, rope_base=1e6, context=256)
TINY_GEMMA3 = DecoderShape("gemma3", 6, 64, 128, 4, 1, 32, 256, rope_base=1e6, window=8,
                           tied_head=True, context=256)
# Small decoders with the head sizes of the benchmark models (128 and 256), which the persistent
# decode kernel serves; the two above (head size 32) take the per-operator graph.
SMALL_QWEN3 = DecoderShape("qwen3", 3, 256, 512, 4, 2, 128, 1024, rope_base=1e6, context=512)
SMALL_GEMMA3 = DecoderShape("gemma3", 6, 128, 320, 4, 1, 256, 512, rope_base=1e6, window=40,
                            tied_head=True, context=512)


def _gguf_str(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _gguf_kv(key: str, value) -> bytes:
    out = _gguf_str(key)
    if isinstance(value, str):
        return out + struct.pack("<I", 8) + _gguf_str(value)
    if isinstance(value, bool):
        return out + struct.pack("<IB", 7, int(value))
    if isinstance(value, float):
        return out + struct.pack("<If", 6, value)
    if isinstance(value, int):
        return out + struct.pack("<II", 4, value)
    raise TypeError(type(value))


def fixture_values(count: int) -> np.ndarray:
    """Element e of every F32 / F16 tensor of the reference's synthetic model fixtures:
    ((31 e + 7) mod 64 - 32) / 64, multiples of 1/64 in [-0.5, 0.5), exact in binary16
    (crates/manifest/src/testing.rs:611-614)."""
    e = np.arange(count, dtype=np.uint64)
    return (((e * np.uint64(31) + np.uint64(7)) % np.uint64(64)).astype(np.float32) - 32.0) / 64.0


def fixture_q8_0(blocks: int) -> np.ndarray:
    """Q8_0 blocks of the same fixtures: d = 1/128, q[e] = (11 e + 5) mod 128 - 64
    (crates/manifest/src/testing.rs:678-690)."""
    e = np.arange(blocks * 32, dtype=np.uint64)
    q = (((e * np.uint64(11) + np.uint64(5)) % np.uint64(128)).astype(np.int32) - 64).astype(np.int8)
    return q8_0_from_parts(np.full((1, blocks), 0.0078125, dtype=np.float16), q.reshape(1, blocks * 32))


def write_gguf(path, shape: DecoderShape, seed: int = 0, norm_jitter: float = 0.0,
               alignment: int = 32, fill: str = "seeded") -> dict:
    """Write a valid GGUF v3 with Q8_0 or F16 matrices and f32 norm vectors.

    ``fill="seeded"``: seeded Q8_0 matrices, norm vectors 1.0 (+ ``norm_jitter`` * N(0,1)
    when asked); ``"seeded-f16"``: the same matrices dequantised and rounded to binary16 (an
    F16 twin whose rows differ, unlike the reference fixture's).  ``fill="fixture-f16"`` / ``"fixture-q8_0"``: the tensor contents of the
    reference's synthetic fixtures (crates/manifest/src/testing.rs:236-396, 611-690) -- with
    TINY_QWEN3 and "fixture-f16" every tensor equals the reference's ``tiny_qwen3`` artifact
    byte for byte (the tokenizer metadata, which no engine path reads, is left out).
    Returns ``{name: (type, dims, absolute file offset, bytes)}``.
    """
    if fill not in ("seeded", "seeded-f16", "fixture-f16", "fixture-q8_0"):
        raise ValueError(fill)
    a = shape.arch
    kv = {
        "general.architecture": a, "general.alignment": alignment,
        f"{a}.block_count": shape.layers, f"{a}.context_length": shape.context,
        f"{a}.embedding_length": shape.hidden, f"{a}.feed_forward_length": shape.ffn,
        f"{a}.attention.head_count": shape.heads, f"{a}.attention.head_count_kv": shape.kv_heads,
        f"{a}.attention.key_length": shape.head_dim, f"{a}.attention.value_length": shape.head_dim,
        f"{a}.attention.layer_norm_rms_epsilon": float(shape.eps), f"{a}.rope.freq_base": float(shape.rope_base),
    }
    if a == "gemma3":
        kv[f"{a}.attention.sliding_window"] = shape.window
    kv.update(shape.extra_kv)

    tensors: list[tuple[str, list[int], int, int]] = []  # name, dims, type, bytes

    def q8(name, out_dim, in_dim):
        if fill in ("fixture-f16", "seeded-f16"):
            tensors.append((name, [in_dim, out_dim], GGML_F16, out_dim * in_dim * 2))
        else:
            tensors.append((name, [in_dim, out_dim], GGML_Q8_0, out_dim * (in_dim // 32) * 34))

    def f32(name, n):
        tensors.append((name, [n], GGML_F32, n * 4))

    q8("token_embd.weight", shape.vocab, shape.hidden)
    f32("output_norm.weight", shape.hidden)
    if not shape.tied_head:
        q8("output.weight", shape.vocab, shape.hidden)
    for l in range(shape.layers):
        for name, o, i in shape.matrices(l):
            q8(name, o, i)
        for name, n in shape.norms(l):
            f32(name, n)

    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv))
    head += b"".join(_gguf_kv(k, v) for k, v in kv.items())
    infos, off = b"", 0
    rel = []
    for name, dims, ty, nbytes in tensors:
        infos += _gguf_str(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
        infos += struct.pack("<IQ", ty, off)
        rel.append(off)
        off += (nbytes + alignment - 1) // alignment * alignment
    start = (len(head) + len(infos) + alignment - 1) // alignment * alignment
    index = {}
    with open(path, "wb") as f:
        f.write(head + infos)
        f.write(b"\0" * (start - len(head) - len(infos)))
        for tid, ((name, dims, ty, nbytes), r) in enumerate(zip(tensors, rel)):
            f.seek(start + r)
            if fill == "seeded-f16" and ty == GGML_F16:
                rows, cols = dims[1], dims[0]
                step = max(1, (1 << 25) // cols)
                for r0 in range(0, rows, step):
                    f.write(q8_0_dequant(q8_0_rows(seed, tid, r0, min(step, rows - r0), cols)).astype(np.float16).tobytes())
            elif fill.startswith("fixture"):
                if ty == GGML_Q8_0:
                    f.write(fixture_q8_0(dims[0] * dims[1] // 32).tobytes())
                else:
                    v = fixture_values(int(np.prod(dims)))
                    f.write((v.astype(np.float16) if ty == GGML_F16 else v).tobytes())
            elif ty == GGML_Q8_0:
                rows, cols = dims[1], dims[0]
                step = max(1, (1 << 25) // cols)
                for r0 in range(0, rows, step):
                    f.write(q8_0_rows(seed, tid, r0, min(step, rows - r0), cols).tobytes())
            else:
                v = np.ones(dims[0], dtype=np.float32)
                if norm_jitter:
                    v += (norm_jitter * normals(seed, tid, 5, 0, dims[0])).astype(np.float32)
                f.write(v.tobytes())
            index[name] = (ty, dims, start + r, nbytes)
        f.truncate(start + off)
    return index


def read_gguf(path) -> tuple[dict, dict, np.memmap]:
    """Minimal GGUF v2/v3 reader: ``(metadata, {name: (type, dims, offset, bytes)}, mmap)``."""
    data = np.memmap(path, dtype=np.uint8, mode="r")
    buf = memoryview(data)
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, buf, pos)
        pos += struct.calcsize(fmt)
        return v if len(v) > 1 else v[0]

    def string():
        nonlocal pos
        n = take("<Q")
        s = bytes(buf[pos:pos + n]).decode()
        pos += n
        return s

    scalar = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}

    def value(ty):
        if ty == 8:
            return string()
        if ty == 9:
            et, n = take("<I"), take("<Q")
            return [value(et) for _ in range(n)]
        return take(scalar[ty])

    magic, version, n_tensors, n_kv = take("<IIQQ")
    if magic != 0x46554747 or version not in (2, 3):
        raise ValueError("not a GGUF v2/v3 file")
    meta = {}
    for _ in range(n_kv):
        k = string()
        meta[k] = value(take("<I"))
    infos = []
    for _ in range(n_tensors):
        name = string()
        nd = take("<I")
        dims = [take("<Q") for _ in range(nd)]
        ty, off = take("<I"), take("<Q")
        infos.append((name, dims, ty, off))
    align = int(meta.get("general.alignment", 32))
    start = (pos + align - 1) // align * align
    block = {GGML_F32: (1, 4), GGML_F16: (1, 2), GGML_Q8_0: (32, 34)}
    tensors = {}
    for name, dims, ty, off in infos:
        elems = int(np.prod(dims))
        be, bb = block[ty]
        tensors[name] = (ty, dims, start + off, elems // be * bb)
    return meta, tensors, data
