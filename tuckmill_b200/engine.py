"""ctypes front-end of the C++ engine host layer (``include/tm_engine.h``).

Mirrors the executor surface the reference's tests drive
(crates/tuckcore/src/executor.rs:218-854 ``TuckCore: InferenceBackend`` --
load, generate, score -- and ``EngineModel::step``): a test harness, not a
compute path; all arithmetic happens in ``libtm_cuda.so``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import cuda as _cuda

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libtm_engine.so"
_lib = None

ERROR_CODES = {1: "INVALID_REQUEST", 2: "INVALID_ARTIFACT", 3: "UNSUPPORTED_ARCHITECTURE",
               4: "UNSUPPORTED_QUANTIZATION", 5: "CONTEXT_EXCEEDS_BUDGET", 6: "MODEL_EXCEEDS_BUDGET",
               7: "UNAVAILABLE", 8: "CANCELLED", 9: "INTERNAL"}


class EngineError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = ERROR_CODES.get(code, str(code))
        self.message = message


class _Options(C.Structure):
    _fields_ = [("gguf_path", C.c_char_p), ("kernels", C.c_char_p), ("device", C.c_int), ("context", C.c_uint32),
                ("prefill_batch", C.c_uint32), ("exact", C.c_int), ("budget_bytes", C.c_uint64),
                ("shard_rank", C.c_uint32), ("shard_world", C.c_uint32), ("comm_id", C.c_void_p),
                ("persistent_step", C.c_int), ("sequences", C.c_uint32)]


class Info(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("vocab", "hidden", "layers", "context", "prefill_batch")] + \
               [(n, C.c_uint64) for n in ("plan_weights", "plan_state", "plan_scratch", "allocated_bytes", "budget",
                                          "reservation", "overhead", "safety_reserve")] + \
               [("kernel_impl", C.c_char * 16), ("kernel_id", C.c_char * 64), ("architecture", C.c_char * 32)]


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("ttft_ns", "decode_span_ns", "prompt_tokens", "generated",
                                          "kernel_launches", "dispatches", "h2d_bytes", "d2h_bytes")]


def load_library() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    _cuda.load_library()  # libtm_cuda.so first: no CUDA library, no engine
    if not _LIB_PATH.exists():
        raise ImportError(f"{_LIB_PATH} is not built; run `python -m tuckmill_b200.build`")
    L = C.CDLL(str(_LIB_PATH))
    E = [C.c_char_p, C.c_size_t]
    P = C.c_void_p
    L.tm_engine_load.argtypes = [C.POINTER(_Options), C.POINTER(P)] + E
    L.tm_engine_free.argtypes = [P]
    L.tm_engine_comm_id.argtypes = [P] + E
    L.tm_engine_get_info.argtypes = [P, C.POINTER(Info)]
    L.tm_engine_cuda_ctx.restype = P
    L.tm_engine_cuda_ctx.argtypes = [P]
    L.tm_engine_decode_program.restype = P
    L.tm_engine_decode_program.argtypes = [P]
    L.tm_engine_reset.argtypes = [P] + E
    L.tm_engine_prefill.argtypes = [P, P, C.c_uint32, C.c_int] + E
    L.tm_engine_prefill_token.argtypes = [P, C.POINTER(C.c_uint32)] + E
    L.tm_engine_step.argtypes = [P, C.c_uint32, P] + E
    L.tm_engine_logits.argtypes = [P, P] + E
    L.tm_engine_generate.argtypes = [P, P, C.c_uint32, C.c_uint32, C.c_int, P, C.POINTER(C.c_uint32),
                                     C.POINTER(Stats)] + E
    L.tm_engine_decode_steps.argtypes = [P, C.c_uint32] + E
    L.tm_engine_prefill_seq.argtypes = [P, C.c_uint32, P, C.c_uint32, C.c_int] + E
    L.tm_engine_prefill_token_of.argtypes = [P, C.c_uint32, C.POINTER(C.c_uint32)] + E
    L.tm_engine_step_batch.argtypes = [P, P, P] + E
    L.tm_engine_decode_steps_batch.argtypes = [P, C.c_uint32] + E
    L.tm_engine_generate_batch.argtypes = [P, P, P, C.c_uint32, C.c_uint32, C.c_int, P, P, C.POINTER(Stats)] + E
    L.tm_engine_decode_ungrouped.argtypes = [P, C.c_uint32] + E
    L.tm_engine_plan.argtypes = [C.c_char_p, C.c_uint32, C.c_uint64, C.POINTER(Info)] + E
    L.tm_engine_plan_shard.argtypes = [C.c_char_p, C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32, C.POINTER(Info)] + E
    _lib = L
    return L


def _check(rc: int, err) -> None:
    if rc != 0:
        raise EngineError(rc, err.value.decode(errors="replace"))


def plan(gguf_path, context: int, budget_bytes: int, shard_rank: int = 0, shard_world: int = 1) -> Info:
    """Admission arithmetic only (no device): raises when R + U + H > B.  With
    shard_world > 1 the byte classes are those of one rank of the row split."""
    L = load_library()
    info, err = Info(), C.create_string_buffer(1024)
    _check(L.tm_engine_plan_shard(str(gguf_path).encode(), context, budget_bytes, shard_rank, shard_world,
                                  C.byref(info), err, 1024), err)
    return info


def comm_id() -> bytes:
    """128 opaque bytes naming a new communicator; rank 0 makes them and the
    launcher hands them to the other ranks."""
    L = load_library()
    out, err = C.create_string_buffer(128), C.create_string_buffer(1024)
    _check(L.tm_engine_comm_id(out, err, 1024), err)
    return out.raw


class Engine:
    def __init__(self, gguf_path, context: int, kernels: str = "cuda", device: int = 0, prefill_batch: int = 0,
                 exact: bool = False, budget_bytes: int = 0, shard_rank: int = 0, shard_world: int = 1,
                 comm_id: bytes | None = None, persistent_step: bool = False, sequences: int = 1):
        """With shard_world > 1 every rank constructs its Engine with the same
        128-byte `comm_id` (from `comm_id()` on one rank) and then makes the same
        calls in the same order; each call is a collective."""
        self._l = load_library()
        self._path = str(gguf_path).encode()
        self._kernels = kernels.encode()
        self._comm_id = C.create_string_buffer(comm_id, 128) if comm_id is not None else None
        o = _Options(self._path, self._kernels, device, context, prefill_batch, int(exact), budget_bytes,
                     shard_rank, shard_world, C.cast(self._comm_id, C.c_void_p) if self._comm_id is not None else None,
                     int(persistent_step), sequences)
        self.sequences = max(1, sequences)
        h, err = C.c_void_p(), C.create_string_buffer(1024)
        _check(self._l.tm_engine_load(C.byref(o), C.byref(h), err, 1024), err)
        self.handle = h
        self.info = Info()
        self._l.tm_engine_get_info(self.handle, C.byref(self.info))
        self.vocab = self.info.vocab

    def _call(self, fn, *args):
        err = C.create_string_buffer(1024)
        _check(fn(self.handle, *args, err, 1024), err)

    def refresh_info(self) -> Info:
        self._l.tm_engine_get_info(self.handle, C.byref(self.info))
        return self.info

    def cuda_ctx(self) -> int:
        return int(self._l.tm_engine_cuda_ctx(self.handle))

    def decode_program(self) -> int:
        """Handle of the persistent decode program (0 when a step is a graph of kernels)."""
        return int(self._l.tm_engine_decode_program(self.handle) or 0)

    def program_trace(self):
        """Per-operator time stamps of the last decode step (tm_cuda_program_trace): (kinds, stamps[n][4])."""
        L = _cuda.load_library()
        cap = 4096
        out = (C.c_uint64 * (cap * 8))()
        kinds = (C.c_uint32 * cap)()
        err = C.create_string_buffer(256)
        L.tm_cuda_program_trace.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_char_p, C.c_size_t]
        rc = L.tm_cuda_program_trace(self.cuda_ctx(), self.decode_program(), out, cap, kinds, err, 256)
        if rc:
            raise _cuda.CudaError(rc, err.value.decode())
        n = self.info.layers * 8 + 8
        return np.array(kinds[:n]), np.array(out[:n * 8], dtype=np.uint64).reshape(n, 8)

    def stream(self) -> int:
        return int(_cuda.load_library().tm_cuda_stream(self.cuda_ctx()) or 0)

    def fence(self):
        err = C.create_string_buffer(256)
        rc = _cuda.load_library().tm_cuda_fence(self.cuda_ctx(), err, 256)
        if rc:
            raise _cuda.CudaError(rc, err.value.decode())

    def reset(self):
        self._call(self._l.tm_engine_reset)

    def prefill(self, tokens, want_token: bool = True):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        self._call(self._l.tm_engine_prefill, t.ctypes.data, t.size, int(want_token))

    def prefill_token(self) -> int:
        tok = C.c_uint32()
        self._call(self._l.tm_engine_prefill_token, C.byref(tok))
        return tok.value

    def step(self, token: int, want_logits: bool = True):
        out = np.empty(self.vocab, dtype=np.float32) if want_logits else None
        self._call(self._l.tm_engine_step, int(token), out.ctypes.data if want_logits else None)
        return out

    def logits(self) -> np.ndarray:
        out = np.empty(self.vocab, dtype=np.float32)
        self._call(self._l.tm_engine_logits, out.ctypes.data)
        return out

    def decode_steps(self, steps: int):
        self._call(self._l.tm_engine_decode_steps, steps)

    def decode_ungrouped(self, steps: int):
        self._call(self._l.tm_engine_decode_ungrouped, steps)

    def profile(self, enabled: bool):
        _cuda.load_library().tm_cuda_profile_set(self.cuda_ctx(), int(enabled))

    def profile_rows(self):
        L = _cuda.load_library()
        rows, i = [], 0
        name, nanos, count = C.create_string_buffer(128), C.c_uint64(), C.c_uint64()
        while L.tm_cuda_profile_read(self.cuda_ctx(), i, name, 128, C.byref(nanos), C.byref(count)):
            rows.append((name.value.decode(), nanos.value, count.value))
            i += 1
        return rows

    def generate(self, prompt, max_new: int, ignore_eos: bool = True):
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.empty(max_new, dtype=np.uint32)
        n, st = C.c_uint32(), Stats()
        self._call(self._l.tm_engine_generate, p.ctypes.data, p.size, max_new, int(ignore_eos), out.ctypes.data,
                   C.byref(n), C.byref(st))
        return out[:n.value].copy(), st

    # ---- several sequences (Engine(..., sequences=S)) ----
    def prefill_seq(self, seq: int, tokens, want_token: bool = True):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        self._call(self._l.tm_engine_prefill_seq, seq, t.ctypes.data, t.size, int(want_token))

    def prefill_token_of(self, seq: int) -> int:
        tok = C.c_uint32()
        self._call(self._l.tm_engine_prefill_token_of, seq, C.byref(tok))
        return tok.value

    def step_batch(self, tokens, want_logits: bool = True):
        """One decode step of every sequence; returns logits [sequences, vocab] when asked."""
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        if t.size != self.sequences:
            raise ValueError(f"{t.size} tokens for {self.sequences} sequences")
        out = np.empty((self.sequences, self.vocab), dtype=np.float32) if want_logits else None
        self._call(self._l.tm_engine_step_batch, t.ctypes.data, out.ctypes.data if want_logits else None)
        return out

    def decode_steps_batch(self, steps: int):
        self._call(self._l.tm_engine_decode_steps_batch, steps)

    def generate_batch(self, prompts, max_new: int, ignore_eos: bool = True):
        """Greedy generation for len(prompts) <= sequences requests at once: (list of token arrays, Stats)."""
        ps = [np.ascontiguousarray(p, dtype=np.uint32) for p in prompts]
        flat = np.concatenate(ps) if ps else np.zeros(0, np.uint32)
        lens = np.array([p.size for p in ps], dtype=np.uint32)
        out = np.zeros((len(ps), max_new), dtype=np.uint32)
        counts, st = np.zeros(len(ps), dtype=np.uint32), Stats()
        self._call(self._l.tm_engine_generate_batch, flat.ctypes.data, lens.ctypes.data, len(ps), max_new,
                   int(ignore_eos), out.ctypes.data, counts.ctypes.data, C.byref(st))
        return [out[r, :counts[r]].copy() for r in range(len(ps))], st

    def score(self, tokens) -> np.ndarray:
        """Teacher-forced logits at every position (crates/tuckcore/src/executor.rs:716-762)."""
        self.reset()
        return np.stack([self.step(int(t)) for t in tokens])

    def close(self):
        if getattr(self, "handle", None):
            self._l.tm_engine_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
