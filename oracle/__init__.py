"""ctypes front-end of the CPU oracle (``tm_oracle.c``).

TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against.
Nothing in the product package imports this module; only the test-suite, the
smoke check and the bench's CPU-baseline leg do.  Build with ``make -C oracle``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None


def build(force: bool = False) -> Path:
    so = _HERE / "liboracle.so"
    src = _HERE / "tm_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        so = _HERE / "liboracle.so"
        if not so.exists():
            build()
        L = C.CDLL(str(so))
        L.tmo_f16_to_f32.restype = C.c_float
        L.tmo_f16_to_f32.argtypes = [C.c_uint16]
        L.tmo_f32_to_f16_bits.restype = C.c_uint16
        L.tmo_f32_to_f16_bits.argtypes = [C.c_float]
        L.tmo_dot_q8_0_x_f32.restype = C.c_float
        L.tmo_dot_q8_0_x_f32.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.tmo_validate_q8_0_row.restype = C.c_long
        L.tmo_validate_q8_0_row.argtypes = [C.c_size_t, C.c_size_t]
        L.tmo_dequant_q8_0.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.tmo_matmul_q8_0.restype = C.c_int
        L.tmo_matmul_q8_0.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                                      C.c_void_p, C.c_int]
        L.tmo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_size_t, C.c_void_p]
        L.tmo_rope_inv_freq.argtypes = [C.c_size_t, C.c_float, C.c_void_p]
        L.tmo_rope_apply.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.tmo_silu.restype = C.c_float
        L.tmo_silu.argtypes = [C.c_float]
        L.tmo_gelu_tanh.restype = C.c_float
        L.tmo_gelu_tanh.argtypes = [C.c_float]
        L.tmo_argmax.restype = C.c_uint32
        L.tmo_argmax.argtypes = [C.c_void_p, C.c_size_t]
        L.tmo_attend_head.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                      C.c_size_t, C.c_float, C.c_void_p, C.c_void_p]
        L.tmo_kv_new.restype = C.c_void_p
        L.tmo_kv_new.argtypes = [C.c_void_p, C.c_size_t]
        L.tmo_kv_free.argtypes = [C.c_void_p]
        L.tmo_forward.restype = C.c_int
        L.tmo_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                  C.c_void_p, C.c_int]
        _LIB = L
    return _LIB


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def f16_to_f32(bits: int) -> float:
    return float(lib().tmo_f16_to_f32(bits))


def f32_to_f16_bits(v: float) -> int:
    return int(lib().tmo_f32_to_f16_bits(np.float32(v)))


def dequant_q8_0(raw: np.ndarray) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    blocks = raw.size // 34
    out = np.empty(blocks * 32, dtype=np.float32)
    lib().tmo_dequant_q8_0(_p(raw), blocks, _p(out))
    return out


def dot_q8_0_x_f32(row: np.ndarray, x: np.ndarray) -> float:
    """Checked entry (kernels.rs:368-381): raises on a malformed row or width."""
    row = np.ascontiguousarray(row, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32)
    blocks = lib().tmo_validate_q8_0_row(row.size, x.size)
    if blocks == -1:
        raise ValueError(f"packed Q8_0 row length {row.size} is not a positive multiple of 34 bytes")
    if blocks == -2:
        raise ValueError(f"Q8_0 x f32 dot expects {row.size // 34 * 32} activation elements, got {x.size}")
    return float(lib().tmo_dot_q8_0_x_f32(_p(row), blocks, _p(x)))


def matmul_q8_0(raw: np.ndarray, rows: int, cols: int, x: np.ndarray, threads: int | None = None) -> np.ndarray:
    """y[b, r] = dot(row_r, x[b]); x is [batch, cols] or [cols]."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    assert raw.size == rows * (cols // 32) * 34
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, cols)
    y = np.empty((x2.shape[0], rows), dtype=np.float32)
    rc = lib().tmo_matmul_q8_0(_p(raw), rows, cols, _p(x2), x2.shape[0], _p(y), threads or default_threads())
    if rc != 0:
        raise ValueError("invalid Q8_0 matmul geometry")
    return y[0] if np.ndim(x) == 1 else y


def matmul_f16(w: np.ndarray, rows: int, cols: int, x: np.ndarray, threads: int | None = None) -> np.ndarray:
    """y[b][r] = dot(f32(w[r]), x[b]) over an F16 matrix (`w`: rows * cols float16), the scalar
    order of crates/tuckcore/src/kernels.rs:223-232."""
    w = np.ascontiguousarray(w, dtype=np.float16).reshape(rows, cols)
    x = np.ascontiguousarray(x, dtype=np.float32)
    batch = 1 if x.ndim == 1 else x.shape[0]
    assert x.size == batch * cols
    y = np.empty(batch * rows, dtype=np.float32)
    fn = lib().tmo_matmul_f16
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]
    rc = fn(_p(w), rows, cols, _p(x), batch, _p(y), threads or default_threads())
    if rc != 0:
        raise ValueError("malformed F16 matmul")
    return y if x.ndim == 1 else y.reshape(batch, rows)


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.empty_like(x)
    lib().tmo_rmsnorm(_p(x), _p(w), eps, x.size, _p(y))
    return y


def rope_inv_freq(rope_dims: int, base: float) -> np.ndarray:
    out = np.empty(rope_dims // 2, dtype=np.float32)
    lib().tmo_rope_inv_freq(rope_dims, base, _p(out))
    return out


def rope_apply(x: np.ndarray, pos: int, inv_freq: np.ndarray) -> np.ndarray:
    y = np.array(x, dtype=np.float32)
    f = np.ascontiguousarray(inv_freq, dtype=np.float32)
    lib().tmo_rope_apply(_p(y), 2 * f.size, pos, _p(f))
    return y


def silu(x: float) -> float:
    return float(lib().tmo_silu(np.float32(x)))


def gelu_tanh(x: float) -> float:
    return float(lib().tmo_gelu_tanh(np.float32(x)))


def argmax(logits: np.ndarray) -> int:
    a = np.ascontiguousarray(logits, dtype=np.float32)
    return int(lib().tmo_argmax(_p(a), a.size))


def attend_head(q, k_plane, v_plane, start: int, seq: int, scale: float) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k_plane, dtype=np.float32)
    v = np.ascontiguousarray(v_plane, dtype=np.float32)
    hd = q.size
    scores = np.empty(seq, dtype=np.float32)
    out = np.empty(hd, dtype=np.float32)
    lib().tmo_attend_head(_p(q), _p(k), _p(v), hd, start, seq, scale, _p(scores), _p(out))
    return out


class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("q", "k", "v", "o", "gate", "up", "down", "pre_norm", "post_norm", "q_norm", "k_norm",
                 "mixer_out_norm", "ffn_out_norm")] + \
               [("rope_base", C.c_float), ("window", C.c_uint32), ("act_gelu", C.c_uint32)]


class _Model(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("layers", "hidden", "ffn", "heads", "kv_heads", "head_dim", "vocab")] + \
               [("eps", C.c_float), ("embedding_scale", C.c_float), ("kv_f16", C.c_uint32),
                ("embedding", C.c_void_p), ("head", C.c_void_p), ("final_norm", C.c_void_p),
                ("layer", C.POINTER(_Layer)), ("weight_type", C.c_uint32)]


class Model:
    """A dense decoder over a GGUF artifact, following the typed graph the
    reference's adapters build (crates/tuckcore/src/engine/adapters.rs:130-200
    qwen3, :214-336 gemma3: global layer every 6th, sliding-window RoPE base
    10000, embedding scale sqrt(hidden), tied head, sandwich norms, GeGLU)."""

    def __init__(self, gguf_path, kv_f16: bool = True, threads: int | None = None):
        from tuckmill_b200 import testing  # GGUF reader only; no compute

        meta, tensors, data = testing.read_gguf(gguf_path)
        self._data = data
        self.threads = threads or default_threads()
        a = meta["general.architecture"]
        if a not in ("qwen3", "gemma3"):
            raise ValueError(f"unsupported architecture {a!r}")
        g = lambda k, d=None: meta.get(f"{a}.{k}", d)
        self.arch = a
        base_addr = data.ctypes.data
        self._keep = []

        # every matrix of an artifact has one type: Q8_0 (8) or F16 (1, the reference's fixtures)
        self.weight_type = int(tensors["token_embd.weight"][0])
        if self.weight_type not in (1, 8):
            raise ValueError(f"unsupported matrix type {self.weight_type}")

        def q8(name):
            ty, dims, off, nbytes = tensors[name]
            assert ty == self.weight_type, name
            return base_addr + off

        def f32(name):
            ty, dims, off, nbytes = tensors[name]
            assert ty == 0, name
            v = np.frombuffer(data, dtype=np.float32, count=nbytes // 4, offset=off).copy()
            self._keep.append(v)
            return v.ctypes.data

        layers = int(g("block_count"))
        gemma = a == "gemma3"
        self._layers = (_Layer * layers)()
        for l in range(layers):
            p = f"blk.{l}."
            L = self._layers[l]
            for fld, nm in (("q", "attn_q"), ("k", "attn_k"), ("v", "attn_v"), ("o", "attn_output"),
                            ("gate", "ffn_gate"), ("up", "ffn_up"), ("down", "ffn_down")):
                setattr(L, fld, q8(p + nm + ".weight"))
            for fld, nm in (("pre_norm", "attn_norm"), ("post_norm", "ffn_norm"), ("q_norm", "attn_q_norm"),
                            ("k_norm", "attn_k_norm")):
                setattr(L, fld, f32(p + nm + ".weight"))
            if gemma:
                L.mixer_out_norm = f32(p + "post_attention_norm.weight")
                L.ffn_out_norm = f32(p + "post_ffw_norm.weight")
                is_global = (l + 1) % 6 == 0
                L.rope_base = float(g("rope.freq_base")) if is_global else 10000.0
                L.window = 0 if is_global else int(g("attention.sliding_window"))
                L.act_gelu = 1
            else:
                L.rope_base = float(g("rope.freq_base", 10000.0))
                L.window = 0
                L.act_gelu = 0
        m = _Model()
        m.layers, m.hidden, m.ffn = layers, int(g("embedding_length")), int(g("feed_forward_length"))
        m.heads, m.kv_heads = int(g("attention.head_count")), int(g("attention.head_count_kv"))
        m.head_dim = int(g("attention.key_length"))
        m.vocab = int(tensors["token_embd.weight"][1][1])
        m.eps = float(g("attention.layer_norm_rms_epsilon", 1e-6))
        m.embedding_scale = float(np.sqrt(np.float32(m.hidden))) if gemma else 0.0
        m.kv_f16 = 1 if kv_f16 else 0
        m.embedding = q8("token_embd.weight")
        m.head = q8("output.weight") if "output.weight" in tensors else m.embedding
        m.final_norm = f32("output_norm.weight")
        m.layer = C.cast(self._layers, C.POINTER(_Layer))
        m.weight_type = self.weight_type
        self._m = m
        self.vocab, self.hidden = m.vocab, m.hidden
        self._kv = None
        self.pos = 0

    def reset(self, capacity: int):
        if self._kv:
            lib().tmo_kv_free(self._kv)
        self._kv = lib().tmo_kv_new(C.byref(self._m), capacity)
        if not self._kv:
            raise MemoryError("oracle KV allocation failed")
        self.pos = 0

    def forward(self, tokens, want_logits: bool = True):
        """Feed tokens at the current position; logits of the last one."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty(self.vocab, dtype=np.float32) if want_logits else None
        rc = lib().tmo_forward(C.byref(self._m), self._kv, _p(t), t.size, self.pos,
                               _p(logits) if want_logits else None, self.threads)
        if rc == -1:
            raise ValueError("token id is outside the vocabulary")
        if rc == -2:
            raise ValueError("position exceeds KV capacity")
        if rc != 0:
            raise MemoryError("oracle forward failed")
        self.pos += t.size
        return logits

    def generate_greedy(self, prompt, steps: int, chunk: int = 128):
        """Prefill in chunks, then `steps` greedy tokens; returns (tokens, margins)
        where margin = top1 - top2 logit at each step."""
        prompt = np.asarray(prompt, dtype=np.uint32)
        logits = None
        for i in range(0, prompt.size, chunk):
            last = i + chunk >= prompt.size
            logits = self.forward(prompt[i:i + chunk], want_logits=last)
        out, margins = [], []
        for s in range(steps):
            tok = argmax(logits)
            part = np.partition(logits[~np.isnan(logits)], -2)
            margins.append(float(part[-1] - part[-2]))
            out.append(tok)
            if s + 1 < steps:
                logits = self.forward([tok])
        return np.array(out, dtype=np.uint32), np.array(margins, dtype=np.float32)

    def __del__(self):
        try:
            if self._kv:
                lib().tmo_kv_free(self._kv)
        except Exception:
            pass
