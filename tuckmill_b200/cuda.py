"""Typed host wrapper over the ``tm_cuda`` C ABI (``include/tm_cuda.h``).

The Python twin of the reference's device wrapper crate
(crates/metal/src/lib.rs:755-2650: ``MetalContext`` with one method per
operator, RAII ``MetalBuffer`` handles, error-code mapping :732-747): the same
method names and argument order, ``CudaError`` carrying the ABI's code and
message.  It calls the shared library only -- there is no fallback: loading
fails loudly when ``libtm_cuda.so`` has not been built.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_PKG = Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libtm_cuda.so"

ERR_NAMES = {0: "OK", -1: "NO_DEVICE", -2: "SOURCE", -3: "ALLOC", -4: "BOUNDS", -5: "UNSUPPORTED", -6: "INTERNAL"}
ARGMAX_NONE = 0xFFFFFFFF
GEMM_MAX_BATCH = 32
GEMM_MMA_MAX_BATCH = 8192
PRO_NONE, PRO_RMSNORM, PRO_SILU_MUL, PRO_GELU_MUL = 0, 1, 2, 3
EPI_STORE, EPI_ADD = 0, 1


class CudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"TM_CUDA_ERR_{ERR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


_lib = None
_P, _U32, _SZ, _F, _I = C.c_void_p, C.c_uint32, C.c_size_t, C.c_float, C.c_int
_ERR = [C.c_char_p, C.c_size_t]

# name -> argument types WITHOUT the trailing (err, err_cap); all return int.
_OPS = {
    "buffer_zero": [_P, _P, _SZ, _SZ],
    "upload": [_P, _P, _SZ, _P, _SZ],
    "download": [_P, _P, _SZ, _P, _SZ],
    "download_after": [_P, _P, _SZ, _P, _SZ, C.c_uint64],
    "f32_scale": [_P, _P, _P, _F, _U32],
    "f32_axpy": [_P, _P, _P, _F, _U32],
    "copy_f32": [_P, _P, _U32, _P, _U32, _U32],
    "cast_f16_f32": [_P, _P, _P, _U32],
    "cast_f32_f16": [_P, _P, _P, _U32],
    "argmax_f32": [_P, _P, _U32, _P, _P, _U32],
    "argmax_f32_dev": [_P, _P, _U32, _P, _P, _U32, _P, _U32, _U32, _P],
    "rmsnorm_f32": [_P, _P, _P, _P, _U32, _U32, _F],
    "rmsnorm_add_f32": [_P, _P, _P, _P, _U32, _U32, _F],
    "silu_mul_f32": [_P, _P, _P, _P, _U32],
    "gelu_tanh_mul_f32": [_P, _P, _P, _P, _U32],
    "q8_0_pack": [_P, _P, _U32, _U32, _P, _SZ, _U32, _U32],
    "q8_0_unpack": [_P, _P, _U32, _U32, _P, _SZ, _U32, _U32],
    "q8_0_gemv": [_P, _P, _P, _P, _U32, _U32],
    "q8_0_gemm": [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32],
    "q8_0_gemm_mma": [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32],
    "q8_0_gemv_fused": [_P, _P, _P, _P, _U32, _U32, _I, _P, _F, _I],
    "q8_0_row_f32": [_P, _P, _P, _U32, _U32, _U32],
    "row_indirect_f32": [_P, _P, _U32, _U32, _U32, _P, _U32, _P],
    "rows_indirect_f32": [_P, _P, _U32, _U32, _P, _U32, _U32, _F, _P],
    "row_indirect_f32_dev": [_P, _P, _U32, _U32, _P, _U32, _P, _U32, C.c_int32, _F, _P],
    "f16_gemv": [_P, _P, _P, _P, _U32, _U32],
    "f16_gemm": [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32],
    "f16_row_f32": [_P, _P, _P, _U32, _U32, _U32],
    "f16_gemv_fused": [_P, _P, _P, _P, _U32, _U32, _I, _P, _F, _I],
    "f16_row_indirect_f32_dev": [_P, _P, _U32, _U32, _P, _U32, _P, _U32, C.c_int32, _F, _P],
    "f16_rows_indirect_f32": [_P, _P, _U32, _U32, _P, _U32, _U32, _F, _P],
    "q8_0_gemm_fused": [_P, _P, _P, _P, _U32, _U32, _U32, _I, _P, _F, _I],
    "attention_decode_batch_dev": [_P] * 13 + [_U32] * 9 + [_F, _F, _I],
    "rows_indirect_seq_f32_dev": [_P, _P, _U32, _U32, _P, _U32, _P, _U32, C.c_int32, _F, _P],
    "argmax_rows_f32_dev": [_P, _P, _U32, _U32, _P, _P, _U32, _U32, _P, _U32, _P],
    "u32_add_sat": [_P, _P, _U32, _U32, _U32, _U32],
    "reduce_ranks_add_f32": [_P, _P, _P, _P, _U32, _U32, _U32, _F],
    "exchange_add_ll_f32": [_P, _P, _P, _P, _U32],
    "prefetch_l2": [_P, _P, _U32],
    "q8_0_gemv_addnorm": [_P, _P, _P, _P, _P, _P, _P, _P, _U32, _U32, _F],
    "begin_group": [_P],
    "end_group": [_P],
    "abort_group": [_P],
    "end_group_retain": [_P, C.POINTER(C.c_void_p)],
    "graph_launch": [_P, _P],
    "begin_program": [_P, _U32, C.c_uint64, C.c_uint64],
    "end_program": [_P, C.POINTER(C.c_void_p)],
    "abort_program": [_P],
    "program_status": [_P, _P, C.POINTER(C.c_uint32)],
    "program_debug": [_P, _P, _U32, _U32],
    "fence": [_P],
    "u32_add": [_P, _P, _U32, _U32],
    "qwen35_rope_partial": [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32],
    "qwen35_rope_partial_chunk": [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _U32],
    "qwen35_kv_store_f16": [_P, _P, _P, _P, _P, _U32, _U32, _U32, _U32],
    "qwen35_kv_store_f16_chunk": [_P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32],
    "qwen35_attention_f16": [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _F],
    "qwen35_attention_f16_chunk": [_P, _P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _F, _U32, _U32],
    "comm_init": [_P, C.c_void_p, _I, _I],
    "all_gather_f32": [_P, _P, _U32, _P, _U32, _U32],
    "all_gather_rows_f32": [_P, _P, _P, _P, _U32, _U32],
    "push_rows_f32": [_P, _P, _P, _U32, _U32],
    "q8_0_gemm_mma_push": [_P, _P, _P, _P, _U32, _U32, _U32],
    "symm_status": [_P, _P, C.POINTER(C.c_uint32)],
    "q8_0_gemm_mma_fused": [_P, _P, _P, _U32, _U32, _U32, _U32, C.POINTER(C.c_void_p), C.POINTER(C.c_uint32), _I, _P, _F, _I],
    "qk_prep_chunk": [_P] * 9 + [_U32] * 7 + [_F],
    "attention_chunk_mma": [_P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _F, _U32, _U32],
    "attention_decode_dev": [_P] * 12 + [_U32, _P] + [_U32] * 6 + [_F, _F, _I],
    "attention_decode_dev_static": [_P] * 11 + [_U32, _P] + [_U32] * 6 + [_F, _F, _I],
}


def load_library() -> C.CDLL:
    """Load ``libtm_cuda.so``; raise (never fall back) when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise ImportError(f"{_LIB_PATH} is not built; run `python -m tuckmill_b200.build` "
                          "(there is no CPU fallback for the CUDA path)")
    L = C.CDLL(str(_LIB_PATH))
    for name, args in _OPS.items():
        fn = getattr(L, "tm_cuda_" + name)
        fn.restype = C.c_int
        fn.argtypes = args + _ERR
    L.tm_cuda_available.restype = C.c_int
    L.tm_cuda_runtime_info.restype = C.c_char_p
    L.tm_cuda_create.restype = _P
    L.tm_cuda_create.argtypes = [_I] + _ERR
    L.tm_cuda_destroy.argtypes = [_P]
    L.tm_cuda_buffer_new.restype = _P
    L.tm_cuda_buffer_new.argtypes = [_P, _SZ, _I] + _ERR
    L.tm_cuda_symm_alloc.restype = _P
    L.tm_cuda_symm_alloc.argtypes = [_P, _SZ] + _ERR
    L.tm_cuda_buffer_view.restype = _P
    L.tm_cuda_buffer_view.argtypes = [_P, _P, _SZ, _SZ] + _ERR
    L.tm_cuda_buffer_free.argtypes = [_P, _P]
    L.tm_cuda_q8_0_row_view.restype = _P
    L.tm_cuda_q8_0_row_view.argtypes = [_P, _P, _U32, _U32, _U32, _U32] + _ERR
    L.tm_cuda_buffer_contents.restype = _P
    L.tm_cuda_buffer_contents.argtypes = [_P, _P]
    L.tm_cuda_buffer_device_ptr.restype = _P
    L.tm_cuda_buffer_device_ptr.argtypes = [_P, _P]
    L.tm_cuda_buffer_len.restype = _SZ
    L.tm_cuda_buffer_len.argtypes = [_P, _P]
    L.tm_cuda_mma_workspace_bytes.restype = _SZ
    L.tm_cuda_mma_workspace_bytes.argtypes = [_U32, _U32]
    L.tm_cuda_mma_workspace_reserve.restype = C.c_int
    L.tm_cuda_mma_workspace_reserve.argtypes = [_P, _SZ] + _ERR
    L.tm_cuda_mma_aborted.restype = C.c_int
    L.tm_cuda_mma_aborted.argtypes = [_P]
    L.tm_cuda_mma_last_tile.restype = C.c_int
    L.tm_cuda_mma_last_tile.argtypes = [_P]
    L.tm_cuda_mma_last_split.restype = C.c_int
    L.tm_cuda_mma_last_split.argtypes = [_P]
    L.tm_cuda_program_bytes.restype = _SZ
    L.tm_cuda_program_bytes.argtypes = [_U32, C.c_uint64, C.c_uint64]
    L.tm_cuda_program_attention_elems.restype = C.c_uint64
    L.tm_cuda_program_attention_elems.argtypes = [_U32, _U32, _U32]
    L.tm_cuda_program_supports_gemv.argtypes = [_U32]
    L.tm_cuda_program_supports_attention.argtypes = [_U32, _U32, _U32, _U32]
    L.tm_cuda_q8_0_packed_bytes.restype = _SZ
    L.tm_cuda_q8_0_packed_bytes.argtypes = [_U32, _U32]
    L.tm_cuda_graph_free.argtypes = [_P, _P]
    for name in ("committed_dispatches", "completed_dispatches", "gpu_nanos_total", "allocated_bytes",
                 "in_flight_bytes", "kernel_launches"):
        fn = getattr(L, "tm_cuda_" + name)
        fn.restype = C.c_uint64
        fn.argtypes = [_P]
    L.tm_cuda_last_gpu_ms.restype = C.c_double
    L.tm_cuda_last_gpu_ms.argtypes = [_P]
    L.tm_cuda_stream.restype = _P
    L.tm_cuda_stream.argtypes = [_P]
    L.tm_cuda_profile_set.argtypes = [_P, _I]
    L.tm_cuda_profile_read.restype = C.c_int
    L.tm_cuda_profile_read.argtypes = [_P, _U32, C.c_char_p, _SZ, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    _lib = L
    return L


def available() -> int:
    return int(load_library().tm_cuda_available())


def comm_unique_id() -> bytes:
    """128 opaque bytes naming a new communicator (made on one rank, handed to the others)."""
    out, err = C.create_string_buffer(128), C.create_string_buffer(512)
    rc = load_library().tm_cuda_comm_unique_id(out, err, 512)
    if rc != 0:
        raise CudaError(rc, err.value.decode())
    return out.raw


def runtime_info() -> str:
    return load_library().tm_cuda_runtime_info().decode()


def decode_attention_scratch_bytes(heads: int, kv_heads: int, head_dim: int, cap: int) -> int:
    L = load_library()
    L.tm_cuda_attention_decode_scratch_bytes.restype = C.c_size_t
    L.tm_cuda_attention_decode_scratch_bytes.argtypes = [_U32] * 4
    return int(L.tm_cuda_attention_decode_scratch_bytes(heads, kv_heads, head_dim, cap))


def decode_attention_static_max_scratch() -> int:
    L = load_library()
    L.tm_cuda_attention_decode_static_max_scratch.restype = C.c_size_t
    return int(L.tm_cuda_attention_decode_static_max_scratch())


def mma_workspace_bytes(cols: int, batch: int) -> int:
    """Context workspace a tensor-core GEMM of `batch` tokens by `cols` columns needs (reserve it with
    CudaContext.mma_workspace_reserve before opening a dispatch group that contains such a call)."""
    return int(load_library().tm_cuda_mma_workspace_bytes(cols, batch))


def packed_bytes(rows: int, cols: int) -> int:
    return int(load_library().tm_cuda_q8_0_packed_bytes(rows, cols))


class CudaBuffer:
    """RAII handle of a context buffer (crates/metal/src/lib.rs:2482-2650)."""

    def __init__(self, ctx: "CudaContext", handle: int, parent: "CudaBuffer | None" = None):
        self.ctx, self.handle, self._parent = ctx, handle, parent

    def __len__(self) -> int:
        return int(self.ctx._l.tm_cuda_buffer_len(self.ctx.handle, self.handle))

    def len(self) -> int:
        return len(self)

    def zero(self, off: int = 0, length: int | None = None):
        self.ctx._call("buffer_zero", self.handle, off, len(self) if length is None else length)

    def upload(self, off: int, data) -> None:
        a = np.ascontiguousarray(data)
        self.ctx._call("upload", self.handle, off, a.ctypes.data, a.nbytes)

    def download(self, off: int, nbytes: int, dtype=np.uint8) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        self.ctx._call("download", self.handle, off, out.ctypes.data, nbytes)
        return out.view(dtype)

    def download_after(self, off: int, nbytes: int, completed_target: int, dtype=np.uint8) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        self.ctx._call("download_after", self.handle, off, out.ctypes.data, nbytes, completed_target)
        return out.view(dtype)

    def view(self, off: int, length: int) -> "CudaBuffer":
        err = C.create_string_buffer(256)
        h = self.ctx._l.tm_cuda_buffer_view(self.ctx.handle, self.handle, off, length, err, 256)
        if not h:
            raise CudaError(-4, err.value.decode())
        return CudaBuffer(self.ctx, h, parent=self)

    def device_ptr(self) -> int:
        return int(self.ctx._l.tm_cuda_buffer_device_ptr(self.ctx.handle, self.handle) or 0)

    def free(self):
        if self.handle and self.ctx.handle:
            self.ctx._l.tm_cuda_buffer_free(self.ctx.handle, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class CudaGraph:
    def __init__(self, ctx: "CudaContext", handle: int):
        self.ctx, self.handle = ctx, handle

    def launch(self):
        self.ctx._call("graph_launch", self.handle)

    def status(self) -> int:
        """Status bits of a persistent program (1: a wait for activations ran out, 2: a weight-stage wait)."""
        st = C.c_uint32()
        self.ctx._call("program_status", self.handle, C.byref(st))
        return st.value

    def debug(self, sequence_skew: int = 0, spin_limit: int = 0):
        self.ctx._call("program_debug", self.handle, sequence_skew, spin_limit)

    def free(self):
        if self.handle and self.ctx.handle:
            self.ctx._l.tm_cuda_graph_free(self.ctx.handle, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class CudaContext:
    """One device + one stream; one method per operator of the ABI."""

    def __init__(self, device: int = 0):
        self._l = load_library()
        err = C.create_string_buffer(512)
        self.handle = self._l.tm_cuda_create(device, err, 512)
        if not self.handle:
            raise CudaError(-1, err.value.decode())
        self.device = device

    def close(self):
        if self.handle:
            self._l.tm_cuda_destroy(self.handle)
            self.handle = None

    def _call(self, name: str, *args):
        err = C.create_string_buffer(512)
        fn = getattr(self._l, "tm_cuda_" + name)
        rc = fn(self.handle, *args, err, 512)
        if rc != 0:
            raise CudaError(rc, err.value.decode())

    @staticmethod
    def _h(b):
        return b.handle if b is not None else None

    # -- buffers -----------------------------------------------------------
    def buffer(self, nbytes: int, shared: bool = False) -> CudaBuffer:
        err = C.create_string_buffer(512)
        h = self._l.tm_cuda_buffer_new(self.handle, nbytes, int(shared), err, 512)
        if not h:
            raise CudaError(-3 if nbytes else -4, err.value.decode())
        return CudaBuffer(self, h)

    def floats(self, data, shared: bool = False) -> CudaBuffer:
        a = np.ascontiguousarray(data, dtype=np.float32)
        b = self.buffer(max(a.nbytes, 4), shared)
        if a.nbytes:
            b.upload(0, a)
        return b

    def from_array(self, a: np.ndarray, shared: bool = False) -> CudaBuffer:
        a = np.ascontiguousarray(a)
        b = self.buffer(a.nbytes, shared)
        b.upload(0, a)
        return b

    def q8_0_matrix(self, raw: np.ndarray, rows: int, cols: int, chunk_rows: int | None = None) -> CudaBuffer:
        """Upload raw GGUF Q8_0 bytes and repack them into the two-plane form
        (the load path of crates/tuckcore/src/engine/metal.rs:119-154, with
        the repack step the CUDA kernels need)."""
        raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
        row_bytes = cols // 32 * 34
        assert raw.size == rows * row_bytes
        dst = self.buffer(packed_bytes(rows, cols))
        step = chunk_rows or max(1, (4 << 20) // row_bytes)
        stage = self.buffer(min(rows, step) * row_bytes)
        for r0 in range(0, rows, step):
            n = min(step, rows - r0)
            stage.upload(0, raw[r0 * row_bytes:(r0 + n) * row_bytes])
            self._call("q8_0_pack", dst.handle, rows, cols, stage.handle, 0, r0, n)
        self.fence()
        stage.free()
        return dst

    def q8_0_row_view(self, w: CudaBuffer, rows: int, cols: int, row0: int, nrows: int) -> CudaBuffer:
        err = C.create_string_buffer(256)
        h = self._l.tm_cuda_q8_0_row_view(self.handle, w.handle, rows, cols, row0, nrows, err, 256)
        if not h:
            raise CudaError(-4, err.value.decode())
        return CudaBuffer(self, h, parent=w)

    def q8_0_unpack(self, w: CudaBuffer, rows: int, cols: int) -> np.ndarray:
        raw = self.buffer(rows * (cols // 32) * 34)
        self._call("q8_0_unpack", w.handle, rows, cols, raw.handle, 0, 0, rows)
        out = raw.download(0, len(raw))
        raw.free()
        return out

    # -- operators (names and argument order of crates/metal/src/lib.rs) ----
    def f32_scale(self, x, y, factor, n): self._call("f32_scale", x.handle, y.handle, factor, n)
    def f32_axpy(self, a, y, alpha, n): self._call("f32_axpy", a.handle, y.handle, alpha, n)
    def copy_f32(self, src, src_off, dst, dst_off, n): self._call("copy_f32", src.handle, src_off, dst.handle, dst_off, n)
    def cast_f16_f32(self, x, y, n): self._call("cast_f16_f32", x.handle, y.handle, n)
    def cast_f32_f16(self, x, y, n): self._call("cast_f32_f16", x.handle, y.handle, n)
    def argmax_f32(self, x, n, partial, out, out_index): self._call("argmax_f32", x.handle, n, partial.handle, out.handle, out_index)
    def rmsnorm_add(self, p, weight, x, rows, cols, eps): self._call("rmsnorm_add_f32", p.handle, weight.handle, x.handle, rows, cols, eps)
    def rmsnorm(self, x, weight, y, rows, cols, eps): self._call("rmsnorm_f32", x.handle, weight.handle, y.handle, rows, cols, eps)
    def silu_mul(self, gate, up, out, n): self._call("silu_mul_f32", gate.handle, up.handle, out.handle, n)
    def gelu_tanh_mul(self, gate, up, out, n): self._call("gelu_tanh_mul_f32", gate.handle, up.handle, out.handle, n)
    def q8_0_gemv(self, w, x, y, rows, cols): self._call("q8_0_gemv", w.handle, x.handle, y.handle, rows, cols)

    def q8_0_gemm(self, w, x, y, rows, cols, batch, x_off=0, y_off=0):
        self._call("q8_0_gemm", w.handle, x.handle, y.handle, rows, cols, batch, x_off, y_off)

    def q8_0_gemm_mma(self, w, x, y, rows, cols, batch, x_off=0, y_off=0):
        self._call("q8_0_gemm_mma", w.handle, x.handle, y.handle, rows, cols, batch, x_off, y_off)

    def mma_workspace_reserve(self, nbytes: int): self._call("mma_workspace_reserve", nbytes)
    def mma_aborted(self) -> bool: return bool(self._l.tm_cuda_mma_aborted(self.handle))
    def mma_last_tile(self) -> int: return int(self._l.tm_cuda_mma_last_tile(self.handle))
    def mma_last_split(self) -> int: return int(self._l.tm_cuda_mma_last_split(self.handle))

    def q8_0_gemv_fused(self, w, x, y, rows, cols, prologue=PRO_NONE, pro=None, eps=0.0, epilogue=EPI_STORE):
        self._call("q8_0_gemv_fused", w.handle, x.handle, y.handle, rows, cols, prologue, self._h(pro), eps, epilogue)

    def q8_0_row(self, w, out, row, cols, out_off=0): self._call("q8_0_row_f32", w.handle, out.handle, row, cols, out_off)

    # F16-weight matrices: rows * cols binary16 values, uploaded verbatim (tm_metal.h:156-179 forms)
    def f16_gemv(self, w, x, y, rows, cols): self._call("f16_gemv", w.handle, x.handle, y.handle, rows, cols)

    def f16_gemm(self, w, x, y, rows, cols, batch, x_off=0, y_off=0):
        self._call("f16_gemm", w.handle, x.handle, y.handle, rows, cols, batch, x_off, y_off)

    def f16_row(self, w, out, row, cols, out_off=0): self._call("f16_row_f32", w.handle, out.handle, row, cols, out_off)

    def f16_gemv_fused(self, w, x, y, rows, cols, prologue=PRO_NONE, pro=None, eps=0.0, epilogue=EPI_STORE):
        self._call("f16_gemv_fused", w.handle, x.handle, y.handle, rows, cols, prologue, self._h(pro), eps, epilogue)

    def f16_row_indirect_dev(self, w, rows, cols, ids, base, pos_buf, pos_index, bias, scale, out):
        self._call("f16_row_indirect_f32_dev", w.handle, rows, cols, ids.handle, base, self._h(pos_buf), pos_index,
                   bias, scale, out.handle)

    def f16_rows_indirect(self, w, rows, cols, ids, first, n, scale, out):
        self._call("f16_rows_indirect_f32", w.handle, rows, cols, ids.handle, first, n, scale, out.handle)

    # decode steps of several sequences (include/tm_cuda.h)
    def q8_0_gemv_addnorm(self, w, x, add_p, add_w, x_out, norm_w, y, rows, cols, eps):
        """y = W rmsnorm(x + rmsnorm(add_p, add_w), norm_w); the updated x goes to x_out (not x itself)."""
        self._call("q8_0_gemv_addnorm", w.handle, x.handle, add_p.handle, add_w.handle, x_out.handle, norm_w.handle,
                   y.handle, rows, cols, eps)

    def q8_0_gemm_fused(self, w, x, y, rows, cols, batch, prologue=PRO_NONE, pro=None, eps=0.0, epilogue=EPI_STORE):
        self._call("q8_0_gemm_fused", w.handle, x.handle, y.handle, rows, cols, batch, prologue, self._h(pro), eps, epilogue)

    def attention_decode_batch(self, q, k, v, q_norm, k_norm, inv_freq, k_cache, v_cache, out, scratch, pos_buf, status,
                               n_seq, heads, kv_heads, head_dim, n_rot, cap, window, eps, scale, exact,
                               q_stride=0, kv_stride=0):
        self._call("attention_decode_batch_dev", q.handle, k.handle, v.handle, q_norm.handle, k_norm.handle,
                   inv_freq.handle, k_cache.handle, v_cache.handle, out.handle, scratch.handle, pos_buf.handle,
                   status.handle, n_seq, q_stride, kv_stride, heads, kv_heads, head_dim, n_rot, cap, window, eps, scale,
                   int(exact))

    def rows_indirect_seq(self, w, rows, cols, ids, ids_stride, pos_buf, n_seq, bias, scale, out):
        self._call("rows_indirect_seq_f32_dev", w.handle, rows, cols, ids.handle, ids_stride, pos_buf.handle, n_seq,
                   bias, scale, out.handle)

    def argmax_rows_dev(self, x, n_rows, n, partial, out, out_stride, base, pos_buf, out_cap, mirror=None):
        self._call("argmax_rows_f32_dev", x.handle, n_rows, n, partial.handle, out.handle, out_stride, base,
                   pos_buf.handle, out_cap, self._h(mirror))

    def u32_add_sat(self, buf, first, count, delta, limit):
        self._call("u32_add_sat", buf.handle, first, count, delta, limit)

    def prefetch_l2(self, bufs):
        """A hint: bring the buffers' bytes into L2 on a side stream (joins at the end of the open group)."""
        arr = (C.c_void_p * len(bufs))(*[b.handle for b in bufs])
        self._call("prefetch_l2", arr, len(bufs))

    def exchange_add_ll(self, src, slots, y, width):
        self._call("exchange_add_ll_f32", src.handle, slots.handle, y.handle, width)

    def reduce_ranks_add(self, slots, x, weight, world, n_rows, cols, eps=0.0):
        self._call("reduce_ranks_add_f32", slots.handle, x.handle, self._h(weight), world, n_rows, cols, eps)

    def row_indirect_f32(self, w, type_id, rows, cols, ids, slot, out):
        self._call("row_indirect_f32", w.handle, type_id, rows, cols, ids.handle, slot, out.handle)

    def qwen35_rope_partial(self, q, k, inv_freq, pos, n_q, n_kv, head_dim, n_rot):
        self._call("qwen35_rope_partial", q.handle, k.handle, inv_freq.handle, pos, n_q, n_kv, head_dim, n_rot)

    def qwen35_rope_partial_chunk(self, q, k, inv_freq, pos0, n_q, n_kv, head_dim, n_rot, n):
        self._call("qwen35_rope_partial_chunk", q.handle, k.handle, inv_freq.handle, pos0, n_q, n_kv, head_dim, n_rot, n)

    def qwen35_kv_store_f16(self, k_src, v_src, k_cache, v_cache, pos, cap, head_dim, kv_heads):
        self._call("qwen35_kv_store_f16", k_src.handle, v_src.handle, k_cache.handle, v_cache.handle, pos, cap, head_dim, kv_heads)

    def qwen35_kv_store_chunk(self, k_src, v_src, k_cache, v_cache, pos0, cap, head_dim, kv_heads, n):
        self._call("qwen35_kv_store_f16_chunk", k_src.handle, v_src.handle, k_cache.handle, v_cache.handle, pos0, cap, head_dim, kv_heads, n)

    def qwen35_attention_f16(self, q, k_cache, v_cache, out, scratch, heads, pos, cap, head_dim, group, scale):
        self._call("qwen35_attention_f16", q.handle, k_cache.handle, v_cache.handle, out.handle, scratch.handle, heads, pos, cap, head_dim, group, scale)

    def q8_0_gemm_mma_fused(self, w, x, rows, cols, batch, ys, part_rows, prologue=PRO_NONE, pro=None, eps=0.0,
                            epilogue=EPI_STORE):
        yp = (C.c_void_p * len(ys))(*[y.handle for y in ys])
        pr = (C.c_uint32 * len(ys))(*part_rows)
        self._call("q8_0_gemm_mma_fused", w.handle, x.handle, rows, cols, batch, len(ys), yp, pr, prologue,
                   self._h(pro), eps, epilogue)

    def qk_prep_chunk(self, q, k, v, q_norm, k_norm, inv_freq, k_cache, v_cache, heads, kv_heads, head_dim, n_rot, pos0,
                      cap, n, eps):
        self._call("qk_prep_chunk", q.handle, k.handle, v.handle, q_norm.handle, k_norm.handle, inv_freq.handle,
                   k_cache.handle, v_cache.handle, heads, kv_heads, head_dim, n_rot, pos0, cap, n, eps)

    def attention_chunk_mma(self, q, k_cache, v_cache, out, heads, pos0, cap, head_dim, group, scale, n, window):
        self._call("attention_chunk_mma", q.handle, k_cache.handle, v_cache.handle, out.handle, heads, pos0, cap, head_dim, group, scale, n, window)

    def qwen35_attention_chunk(self, q, k_cache, v_cache, out, scratch, heads, pos0, cap, head_dim, group, scale, n, window):
        self._call("qwen35_attention_f16_chunk", q.handle, k_cache.handle, v_cache.handle, out.handle, scratch.handle, heads, pos0, cap, head_dim, group, scale, n, window)

    def attention_decode_dev(self, q, k, v, q_norm, k_norm, inv_freq, k_cache, v_cache, out, scratch, pos_buf,
                             pos_index, status, heads, kv_heads, head_dim, n_rot, cap, window, eps, scale, exact=True):
        self._call("attention_decode_dev", q.handle, k.handle, v.handle, q_norm.handle, k_norm.handle,
                   inv_freq.handle, k_cache.handle, v_cache.handle, out.handle, scratch.handle, pos_buf.handle,
                   pos_index, status.handle, heads, kv_heads, head_dim, n_rot, cap, window, eps, scale, int(exact))

    def attention_decode_dev_static(self, q, k, v, q_norm, k_norm, inv_freq, k_cache, v_cache, out, pos_buf, pos_index,
                                    status, heads, kv_heads, head_dim, n_rot, cap, window, eps, scale, exact=True):
        """The decode attention core for callers that may not allocate: no scratch
        argument, the library's built-in scratch array is used instead."""
        self._call("attention_decode_dev_static", q.handle, k.handle, v.handle, q_norm.handle, k_norm.handle,
                   inv_freq.handle, k_cache.handle, v_cache.handle, out.handle, pos_buf.handle, pos_index,
                   status.handle, heads, kv_heads, head_dim, n_rot, cap, window, eps, scale, int(exact))

    def u32_add(self, buf, index, delta): self._call("u32_add", buf.handle, index, delta)

    # -- output-row split across devices (one process per device) ---------------
    def comm_init(self, ident: bytes, rank: int, world: int):
        """Collective: every rank passes the same 128-byte id (`comm_unique_id()` of one rank)."""
        self._comm_id = C.create_string_buffer(ident, 128)
        self._call("comm_init", C.cast(self._comm_id, C.c_void_p), rank, world)

    def all_gather_f32(self, src, src_off, dst, dst_off, count):
        self._call("all_gather_f32", src.handle, src_off, dst.handle, dst_off, count)

    def symm_buffer(self, nbytes: int) -> CudaBuffer:
        """Collective: the same zeroed allocation on every rank, mapped into every other rank."""
        err = C.create_string_buffer(512)
        h = self._l.tm_cuda_symm_alloc(self.handle, nbytes, err, 512)
        if not h:
            raise CudaError(-2, err.value.decode())
        return CudaBuffer(self, h)

    def push_rows_f32(self, src, dst, n_rows, width):
        """All-gather as a push: dst[t][rank*width + c] on every rank (dst: a symmetric buffer or a view of one)."""
        self._call("push_rows_f32", src.handle, dst.handle, n_rows, width)

    def q8_0_gemm_mma_push(self, w, x, dst, rows, cols, batch):
        """The tensor-core GEMM whose epilogue writes this rank's rows into every rank's gathered output."""
        self._call("q8_0_gemm_mma_push", w.handle, x.handle, dst.handle, rows, cols, batch)

    def symm_status(self, buf) -> int:
        v = C.c_uint32(0)
        self._call("symm_status", buf.handle, C.byref(v))
        return int(v.value)

    def all_gather_rows_f32(self, src, stage, dst, n_rows, width):
        self._call("all_gather_rows_f32", src.handle, stage.handle, dst.handle, n_rows, width)

    # -- grouping, fences, measurement ---------------------------------------
    def begin_group(self): self._call("begin_group")
    def end_group(self): self._call("end_group")
    def abort_group(self): self._call("abort_group")

    def end_group_retain(self) -> CudaGraph:
        out = C.c_void_p()
        self._call("end_group_retain", C.byref(out))
        return CudaGraph(self, out.value)

    def begin_program(self, max_ops: int, vector_elems: int = 1 << 20, attention_elems: int = 0):
        """Open a program for at most `max_ops` operators whose outputs total `vector_elems` floats;
        `attention_elems` from program_attention_elems() for its largest attention operator."""
        self._call("begin_program", max_ops, vector_elems, attention_elems)

    def program_attention_elems(self, heads: int, head_dim: int, cap: int) -> int:
        return int(self._l.tm_cuda_program_attention_elems(heads, head_dim, cap))
    def abort_program(self): self._call("abort_program")

    def end_program(self) -> CudaGraph:
        """The operators recorded since begin_program as one persistent kernel."""
        out = C.c_void_p()
        self._call("end_program", C.byref(out))
        return CudaGraph(self, out.value)

    def grouped(self, encode):
        """Encode ``encode()`` into one dispatch; abort it on error
        (crates/tuckcore/src/qwen35_gpu.rs:66-86)."""
        self.begin_group()
        try:
            encode()
        except Exception:
            self.abort_group()
            raise
        self.end_group()

    def fence(self): self._call("fence")
    def committed_dispatches(self) -> int: return int(self._l.tm_cuda_committed_dispatches(self.handle))
    def completed_dispatches(self) -> int: return int(self._l.tm_cuda_completed_dispatches(self.handle))
    def gpu_nanos_total(self) -> int: return int(self._l.tm_cuda_gpu_nanos_total(self.handle))
    def last_gpu_ms(self) -> float: return float(self._l.tm_cuda_last_gpu_ms(self.handle))
    def allocated_bytes(self) -> int: return int(self._l.tm_cuda_allocated_bytes(self.handle))
    def in_flight_bytes(self) -> int: return int(self._l.tm_cuda_in_flight_bytes(self.handle))
    def kernel_launches(self) -> int: return int(self._l.tm_cuda_kernel_launches(self.handle))
    def stream(self) -> int: return int(self._l.tm_cuda_stream(self.handle) or 0)
    def set_profiling(self, enabled: bool): self._l.tm_cuda_profile_set(self.handle, int(enabled))

    def profile_snapshot(self) -> list[tuple[str, int, int]]:
        rows, i = [], 0
        name = C.create_string_buffer(128)
        nanos, count = C.c_uint64(), C.c_uint64()
        while self._l.tm_cuda_profile_read(self.handle, i, name, 128, C.byref(nanos), C.byref(count)):
            rows.append((name.value.decode(), nanos.value, count.value))
            i += 1
        return rows

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
