//! TuckCore CUDA path: typed Rust handles over the narrow C ABI of
//! `include/tm_cuda.h` (NVIDIA B200, sm_100a).
//!
//! The twin of `crates/metal/src/lib.rs`: one [`CudaContext`] owns one device
//! and one in-order stream, [`CudaBuffer`] handles free their storage on drop,
//! every operator is one method returning `Result<()>` with a `TuckmillError`,
//! and every buffer is checked (by the C layer) to belong to the calling
//! context.  The engine (`crates/tuckcore/src/engine`) calls the same method
//! names it calls on `MetalContext`; methods that exist only here (weight
//! packing, retained graphs, device-side positions, the row split) are marked
//! "CUDA only".
//!
//! Without `libtm_cuda.so` at build time (see `build.rs`) every constructor
//! returns `ErrorCode::Unavailable`: `--kernels cuda` is then a typed refusal,
//! never a fallback.

use std::ffi::{c_char, c_int, c_void, CStr};
use std::sync::{Arc, Mutex};

use tuckmill_manifest::{ErrorCode, Result, TuckmillError};

const ERR_CAP: usize = 512;

/// Batch limit of [`CudaContext::q8_0_gemm`] (the exact per-row form).
pub const GEMM_MAX_BATCH: u32 = 32;
/// Batch limit of [`CudaContext::q8_0_gemm_mma`] (the reference's 512 raised
/// to what one tensor-core launch tiles).
pub const GEMM_MMA_MAX_BATCH: u32 = 8192;
/// Bytes of scratch [`CudaContext::argmax_f32`] needs.
pub const ARGMAX_PARTIAL_BYTES: usize = 512;
/// [`CudaContext::argmax_f32`]'s result when every input was NaN.
pub const ARGMAX_NONE: u32 = u32::MAX;

/// Prologue folded into a fused GEMV / GEMM (CUDA only).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
#[repr(i32)]
pub enum Prologue {
    None = 0,
    RmsNorm = 1,
    SiluMul = 2,
    GeluMul = 3,
}

/// Epilogue of a fused GEMV / GEMM (CUDA only).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
#[repr(i32)]
pub enum Epilogue {
    Store = 0,
    Add = 1,
}

#[allow(non_camel_case_types, dead_code)]
mod ffi {
    use std::ffi::{c_char, c_int, c_void};

    #[repr(C)]
    pub struct TmCudaCtx {
        _private: [u8; 0],
    }
    #[repr(C)]
    pub struct TmCudaBuffer {
        _private: [u8; 0],
    }
    #[repr(C)]
    pub struct TmCudaGraph {
        _private: [u8; 0],
    }

    pub const TM_CUDA_OK: c_int = 0;
    pub const TM_CUDA_ERR_NO_DEVICE: c_int = -1;
    pub const TM_CUDA_ERR_SOURCE: c_int = -2;
    pub const TM_CUDA_ERR_ALLOC: c_int = -3;
    pub const TM_CUDA_ERR_BOUNDS: c_int = -4;
    pub const TM_CUDA_ERR_UNSUPPORTED: c_int = -5;
    pub const TM_CUDA_ERR_INTERNAL: c_int = -6;

    // One line per declaration of include/tm_cuda.h, in its order.
    #[cfg(tm_cuda_linked)]
    extern "C" {
        pub fn tm_cuda_available() -> c_int;
        pub fn tm_cuda_runtime_info() -> *const c_char;
        pub fn tm_cuda_create(device: c_int, err: *mut c_char, err_cap: usize) -> *mut TmCudaCtx;
        pub fn tm_cuda_destroy(ctx: *mut TmCudaCtx);
        pub fn tm_cuda_buffer_new(ctx: *mut TmCudaCtx, bytes: usize, shared: c_int, err: *mut c_char, err_cap: usize) -> *mut TmCudaBuffer;
        pub fn tm_cuda_buffer_free(ctx: *mut TmCudaCtx, buffer: *mut TmCudaBuffer);
        pub fn tm_cuda_buffer_contents(ctx: *mut TmCudaCtx, buffer: *mut TmCudaBuffer) -> *mut c_void;
        pub fn tm_cuda_buffer_len(ctx: *const TmCudaCtx, buffer: *const TmCudaBuffer) -> usize;
        pub fn tm_cuda_buffer_zero(ctx: *mut TmCudaCtx, buffer: *mut TmCudaBuffer, off: usize, len: usize, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_upload(ctx: *mut TmCudaCtx, dst: *mut TmCudaBuffer, off: usize, src: *const c_void, len: usize, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_download(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, off: usize, dst: *mut c_void, len: usize, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_buffer_view(ctx: *mut TmCudaCtx, parent: *mut TmCudaBuffer, off: usize, len: usize, err: *mut c_char, err_cap: usize) -> *mut TmCudaBuffer;
        pub fn tm_cuda_buffer_device_ptr(ctx: *mut TmCudaCtx, buffer: *mut TmCudaBuffer) -> *mut c_void;
        pub fn tm_cuda_f32_scale(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, factor: f32, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f32_axpy(ctx: *mut TmCudaCtx, a: *mut TmCudaBuffer, y: *mut TmCudaBuffer, alpha: f32, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_copy_f32(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, src_off: u32, dst: *mut TmCudaBuffer, dst_off: u32, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_cast_f16_f32(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_cast_f32_f16(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_argmax_f32(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, n: u32, partial: *mut TmCudaBuffer, out: *mut TmCudaBuffer, out_index: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_rmsnorm_f32(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, weight: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, eps: f32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_rmsnorm_add_f32(ctx: *mut TmCudaCtx, p: *mut TmCudaBuffer, weight: *mut TmCudaBuffer, x: *mut TmCudaBuffer, rows: u32, cols: u32, eps: f32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_silu_mul_f32(ctx: *mut TmCudaCtx, gate: *mut TmCudaBuffer, up: *mut TmCudaBuffer, out: *mut TmCudaBuffer, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_gelu_tanh_mul_f32(ctx: *mut TmCudaCtx, gate: *mut TmCudaBuffer, up: *mut TmCudaBuffer, out: *mut TmCudaBuffer, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_packed_bytes(rows: u32, cols: u32) -> usize;
        pub fn tm_cuda_q8_0_pack(ctx: *mut TmCudaCtx, dst: *mut TmCudaBuffer, rows: u32, cols: u32, raw: *mut TmCudaBuffer, raw_off: usize, row0: u32, nrows: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_row_view(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, rows: u32, cols: u32, row0: u32, nrows: u32, err: *mut c_char, err_cap: usize) -> *mut TmCudaBuffer;
        pub fn tm_cuda_q8_0_unpack(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, rows: u32, cols: u32, raw: *mut TmCudaBuffer, raw_off: usize, row0: u32, nrows: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemv(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemm(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, batch: u32, x_off: u32, y_off: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemm_mma(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, batch: u32, x_off: u32, y_off: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_mma_workspace_bytes(cols: u32, batch: u32) -> usize;
        pub fn tm_cuda_mma_workspace_reserve(ctx: *mut TmCudaCtx, bytes: usize, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_mma_aborted(ctx: *mut TmCudaCtx) -> c_int;
        pub fn tm_cuda_mma_last_tile(ctx: *mut TmCudaCtx) -> c_int;
        pub fn tm_cuda_mma_last_split(ctx: *mut TmCudaCtx) -> c_int;
        pub fn tm_cuda_q8_0_row_f32(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, out: *mut TmCudaBuffer, row: u32, cols: u32, out_off: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f16_gemv(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f16_gemm(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, batch: u32, x_off: u32, y_off: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f16_row_f32(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, out: *mut TmCudaBuffer, row: u32, cols: u32, out_off: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f16_gemv_fused(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, prologue: c_int, pro: *mut TmCudaBuffer, eps: f32, epilogue: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f16_row_indirect_f32_dev(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, rows: u32, cols: u32, ids: *mut TmCudaBuffer, base: u32, pos_buf: *mut TmCudaBuffer, pos_index: u32, bias: i32, scale: f32, out: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_f16_rows_indirect_f32(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, rows: u32, cols: u32, ids: *mut TmCudaBuffer, first: u32, n: u32, scale: f32, out: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_row_indirect_f32(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, type_id: u32, rows: u32, cols: u32, ids: *mut TmCudaBuffer, slot: u32, out: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_rows_indirect_f32(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, rows: u32, cols: u32, ids: *mut TmCudaBuffer, first: u32, n: u32, scale: f32, out: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemv_fused(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, prologue: c_int, pro: *mut TmCudaBuffer, eps: f32, epilogue: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemv_addnorm(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, add_p: *mut TmCudaBuffer, add_w: *mut TmCudaBuffer, x_out: *mut TmCudaBuffer, norm_w: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, eps: f32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemm_fused(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, y: *mut TmCudaBuffer, rows: u32, cols: u32, batch: u32, prologue: c_int, pro: *mut TmCudaBuffer, eps: f32, epilogue: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_begin_group(ctx: *mut TmCudaCtx, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_end_group(ctx: *mut TmCudaCtx, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_abort_group(ctx: *mut TmCudaCtx, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_end_group_retain(ctx: *mut TmCudaCtx, out: *mut *mut TmCudaGraph, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_graph_launch(ctx: *mut TmCudaCtx, graph: *mut TmCudaGraph, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_graph_free(ctx: *mut TmCudaCtx, graph: *mut TmCudaGraph);
        pub fn tm_cuda_prefetch_l2(ctx: *mut TmCudaCtx, bufs: *const *mut TmCudaBuffer, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_program_bytes(max_ops: u32, vector_elems: u64, attention_elems: u64) -> usize;
        pub fn tm_cuda_program_attention_elems(heads: u32, head_dim: u32, cap: u32) -> u64;
        pub fn tm_cuda_program_supports_gemv(cols: u32) -> c_int;
        pub fn tm_cuda_program_supports_attention(heads: u32, kv_heads: u32, head_dim: u32, n_rot: u32) -> c_int;
        pub fn tm_cuda_begin_program(ctx: *mut TmCudaCtx, max_ops: u32, vector_elems: u64, attention_elems: u64, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_end_program(ctx: *mut TmCudaCtx, out: *mut *mut TmCudaGraph, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_abort_program(ctx: *mut TmCudaCtx, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_program_status(ctx: *mut TmCudaCtx, program: *mut TmCudaGraph, status: *mut u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_program_trace(ctx: *mut TmCudaCtx, program: *mut TmCudaGraph, out: *mut u64, max_ops: u32, kinds: *mut u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_program_debug(ctx: *mut TmCudaCtx, program: *mut TmCudaGraph, sequence_skew: u32, spin_limit: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_fence(ctx: *mut TmCudaCtx, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_committed_dispatches(ctx: *const TmCudaCtx) -> u64;
        pub fn tm_cuda_completed_dispatches(ctx: *const TmCudaCtx) -> u64;
        pub fn tm_cuda_download_after(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, off: usize, dst: *mut c_void, len: usize, completed_target: u64, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_last_gpu_ms(ctx: *const TmCudaCtx) -> f64;
        pub fn tm_cuda_gpu_nanos_total(ctx: *const TmCudaCtx) -> u64;
        pub fn tm_cuda_profile_set(ctx: *mut TmCudaCtx, enabled: c_int) -> c_int;
        pub fn tm_cuda_profile_read(ctx: *mut TmCudaCtx, index: u32, name: *mut c_char, name_cap: usize, nanos: *mut u64, count: *mut u64) -> c_int;
        pub fn tm_cuda_allocated_bytes(ctx: *const TmCudaCtx) -> u64;
        pub fn tm_cuda_in_flight_bytes(ctx: *const TmCudaCtx) -> u64;
        pub fn tm_cuda_kernel_launches(ctx: *const TmCudaCtx) -> u64;
        pub fn tm_cuda_device_memory(ctx: *mut TmCudaCtx, free_bytes: *mut u64, total_bytes: *mut u64) -> c_int;
        pub fn tm_cuda_stream(ctx: *mut TmCudaCtx) -> *mut c_void;
        pub fn tm_cuda_qwen35_rope_partial(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k: *mut TmCudaBuffer, inv_freq: *mut TmCudaBuffer, pos: u32, n_q_heads: u32, n_kv_heads: u32, head_dim: u32, n_rot: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_qwen35_rope_partial_chunk(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k: *mut TmCudaBuffer, inv_freq: *mut TmCudaBuffer, pos0: u32, n_q_heads: u32, n_kv_heads: u32, head_dim: u32, n_rot: u32, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_qwen35_kv_store_f16(ctx: *mut TmCudaCtx, k_src: *mut TmCudaBuffer, v_src: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, pos: u32, cap: u32, head_dim: u32, kv_heads: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_qwen35_kv_store_f16_chunk(ctx: *mut TmCudaCtx, k_src: *mut TmCudaBuffer, v_src: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, pos0: u32, cap: u32, head_dim: u32, kv_heads: u32, n: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_qwen35_attention_f16(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, out: *mut TmCudaBuffer, scratch: *mut TmCudaBuffer, heads: u32, pos: u32, cap: u32, head_dim: u32, group: u32, scale: f32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_qwen35_attention_f16_chunk(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, out: *mut TmCudaBuffer, scratch: *mut TmCudaBuffer, heads: u32, pos0: u32, cap: u32, head_dim: u32, group: u32, scale: f32, n: u32, window: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_q8_0_gemm_mma_fused(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, rows: u32, cols: u32, batch: u32, n_parts: u32, y_parts: *const *mut TmCudaBuffer, part_rows: *const u32, prologue: c_int, pro: *mut TmCudaBuffer, eps: f32, epilogue: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_qk_prep_chunk(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k: *mut TmCudaBuffer, v: *mut TmCudaBuffer, q_norm: *mut TmCudaBuffer, k_norm: *mut TmCudaBuffer, inv_freq: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, heads: u32, kv_heads: u32, head_dim: u32, n_rot: u32, pos0: u32, cap: u32, n: u32, eps: f32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_attention_chunk_mma_supported(head_dim: u32) -> c_int;
        pub fn tm_cuda_attention_chunk_mma(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, out: *mut TmCudaBuffer, heads: u32, pos0: u32, cap: u32, head_dim: u32, group: u32, scale: f32, n: u32, window: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_attention_decode_scratch_bytes(heads: u32, kv_heads: u32, head_dim: u32, cap: u32) -> usize;
        pub fn tm_cuda_attention_decode_dev(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k: *mut TmCudaBuffer, v: *mut TmCudaBuffer, q_norm: *mut TmCudaBuffer, k_norm: *mut TmCudaBuffer, inv_freq: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, out: *mut TmCudaBuffer, scratch: *mut TmCudaBuffer, pos_buf: *mut TmCudaBuffer, pos_index: u32, status: *mut TmCudaBuffer, heads: u32, kv_heads: u32, head_dim: u32, n_rot: u32, cap: u32, window: u32, eps: f32, scale: f32, exact: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_attention_decode_static_max_scratch() -> usize;
        pub fn tm_cuda_attention_decode_dev_static(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k: *mut TmCudaBuffer, v: *mut TmCudaBuffer, q_norm: *mut TmCudaBuffer, k_norm: *mut TmCudaBuffer, inv_freq: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, out: *mut TmCudaBuffer, pos_buf: *mut TmCudaBuffer, pos_index: u32, status: *mut TmCudaBuffer, heads: u32, kv_heads: u32, head_dim: u32, n_rot: u32, cap: u32, window: u32, eps: f32, scale: f32, exact: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_attention_decode_batch_dev(ctx: *mut TmCudaCtx, q: *mut TmCudaBuffer, k: *mut TmCudaBuffer, v: *mut TmCudaBuffer, q_norm: *mut TmCudaBuffer, k_norm: *mut TmCudaBuffer, inv_freq: *mut TmCudaBuffer, k_cache: *mut TmCudaBuffer, v_cache: *mut TmCudaBuffer, out: *mut TmCudaBuffer, scratch: *mut TmCudaBuffer, pos_buf: *mut TmCudaBuffer, status: *mut TmCudaBuffer, n_seq: u32, q_stride: u32, kv_stride: u32, heads: u32, kv_heads: u32, head_dim: u32, n_rot: u32, cap: u32, window: u32, eps: f32, scale: f32, exact: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_rows_indirect_seq_f32_dev(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, rows: u32, cols: u32, ids: *mut TmCudaBuffer, ids_stride: u32, pos_buf: *mut TmCudaBuffer, n_seq: u32, bias: i32, scale: f32, out: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_argmax_rows_f32_dev(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, n_rows: u32, n: u32, partial: *mut TmCudaBuffer, out: *mut TmCudaBuffer, out_stride: u32, base: u32, pos_buf: *mut TmCudaBuffer, out_cap: u32, mirror: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_u32_add_sat(ctx: *mut TmCudaCtx, buf: *mut TmCudaBuffer, first: u32, count: u32, delta: u32, limit: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_u32_add(ctx: *mut TmCudaCtx, buf: *mut TmCudaBuffer, index: u32, delta: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_argmax_f32_dev(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, n: u32, partial: *mut TmCudaBuffer, out: *mut TmCudaBuffer, base: u32, pos_buf: *mut TmCudaBuffer, pos_index: u32, out_cap: u32, mirror: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_row_indirect_f32_dev(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, rows: u32, cols: u32, ids: *mut TmCudaBuffer, base: u32, pos_buf: *mut TmCudaBuffer, pos_index: u32, bias: i32, scale: f32, out: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_comm_unique_id(out128: *mut c_void, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_comm_init(ctx: *mut TmCudaCtx, id128: *const c_void, rank: c_int, world: c_int, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_comm_rank(ctx: *const TmCudaCtx, rank: *mut c_int, world: *mut c_int) -> c_int;
        pub fn tm_cuda_all_gather_f32(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, src_off: u32, dst: *mut TmCudaBuffer, dst_off: u32, count: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_all_gather_rows_f32(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, stage: *mut TmCudaBuffer, dst: *mut TmCudaBuffer, n_rows: u32, width: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_symm_alloc(ctx: *mut TmCudaCtx, bytes: usize, err: *mut c_char, err_cap: usize) -> *mut TmCudaBuffer;
        pub fn tm_cuda_q8_0_gemm_mma_push(ctx: *mut TmCudaCtx, w: *mut TmCudaBuffer, x: *mut TmCudaBuffer, dst: *mut TmCudaBuffer, rows: u32, cols: u32, batch: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_push_rows_f32(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, dst: *mut TmCudaBuffer, n_rows: u32, width: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_symm_status(ctx: *mut TmCudaCtx, buf: *mut TmCudaBuffer, status: *mut u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_argmax_sharded_dev(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, n: u32, index_offset: u32, partial: *mut TmCudaBuffer, pairs: *mut TmCudaBuffer, out: *mut TmCudaBuffer, base: u32, pos_buf: *mut TmCudaBuffer, pos_index: u32, out_cap: u32, mirror: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_reduce_ranks_add_f32(ctx: *mut TmCudaCtx, slots: *mut TmCudaBuffer, x: *mut TmCudaBuffer, weight: *mut TmCudaBuffer, world: u32, n_rows: u32, cols: u32, eps: f32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_exchange_add_ll_f32(ctx: *mut TmCudaCtx, src: *mut TmCudaBuffer, slots: *mut TmCudaBuffer, y: *mut TmCudaBuffer, width: u32, err: *mut c_char, err_cap: usize) -> c_int;
        pub fn tm_cuda_argmax_rows_sharded_dev(ctx: *mut TmCudaCtx, x: *mut TmCudaBuffer, n_rows: u32, n: u32, index_offset: u32, partial: *mut TmCudaBuffer, pairs: *mut TmCudaBuffer, out: *mut TmCudaBuffer, out_stride: u32, base: u32, pos_buf: *mut TmCudaBuffer, out_cap: u32, mirror: *mut TmCudaBuffer, err: *mut c_char, err_cap: usize) -> c_int;
    }
}

/// Result of [`probe`].
#[derive(Clone, Debug)]
pub struct Probe {
    pub available: bool,
    pub info: String,
}

/// Whether a usable sm_100 device and the library are present.
pub fn probe() -> Probe {
    #[cfg(tm_cuda_linked)]
    {
        // SAFETY: both functions take no arguments; runtime_info returns a
        // static NUL-terminated string.
        let n = unsafe { ffi::tm_cuda_available() };
        let info = unsafe { CStr::from_ptr(ffi::tm_cuda_runtime_info()) }
            .to_string_lossy()
            .into_owned();
        Probe { available: n > 0, info }
    }
    #[cfg(not(tm_cuda_linked))]
    Probe {
        available: false,
        info: "tuckmill-cuda was built without libtm_cuda (set TM_CUDA_LIB_DIR)".to_string(),
    }
}

fn err_text(buf: &[c_char]) -> String {
    // SAFETY: the C layer always NUL-terminates within err_cap.
    let text = unsafe { CStr::from_ptr(buf.as_ptr()) }
        .to_string_lossy()
        .into_owned();
    if text.is_empty() {
        "unknown error".to_string()
    } else {
        text
    }
}

/// ABI code -> typed error (the mapping of `crates/metal/src/lib.rs`).
fn cuda_error(code: c_int, text: String, context: &str) -> TuckmillError {
    let mapped = match code {
        ffi::TM_CUDA_ERR_NO_DEVICE | ffi::TM_CUDA_ERR_ALLOC => ErrorCode::Unavailable,
        ffi::TM_CUDA_ERR_BOUNDS | ffi::TM_CUDA_ERR_UNSUPPORTED => ErrorCode::InvalidRequest,
        _ => ErrorCode::Internal,
    };
    TuckmillError::new(mapped, format!("CUDA {context}: {text}"))
}

#[cfg(not(tm_cuda_linked))]
fn unavailable<T>() -> Result<T> {
    Err(TuckmillError::new(
        ErrorCode::Unavailable,
        "CUDA kernels were requested but this build carries no libtm_cuda",
    )
    .with_action("Build tuckmill_b200/csrc with nvcc for sm_100a and set TM_CUDA_LIB_DIR."))
}

struct ContextInner {
    raw: *mut ffi::TmCudaCtx,
    /// Serializes dispatches: the ABI is used from one thread at a time.
    lock: Mutex<()>,
}

// SAFETY: the raw context is only touched under `lock`; the C layer's counters
// are atomics.
unsafe impl Send for ContextInner {}
unsafe impl Sync for ContextInner {}

impl Drop for ContextInner {
    fn drop(&mut self) {
        #[cfg(tm_cuda_linked)]
        unsafe {
            // SAFETY: created by tm_cuda_create; every buffer holds an Arc to
            // this inner and has been dropped before the last reference.
            ffi::tm_cuda_destroy(self.raw);
        }
    }
}

/// One device, one in-order stream, and the kernels of the C ABI.
#[derive(Clone)]
pub struct CudaContext {
    inner: Arc<ContextInner>,
}

/// A device (or pinned, host-visible) allocation; freed on drop.
pub struct CudaBuffer {
    ctx: Arc<ContextInner>,
    raw: *mut ffi::TmCudaBuffer,
    len: usize,
    shared: bool,
}

// SAFETY: the handle is only used under the owning context's lock.
unsafe impl Send for CudaBuffer {}
unsafe impl Sync for CudaBuffer {}

impl Drop for CudaBuffer {
    fn drop(&mut self) {
        #[cfg(tm_cuda_linked)]
        {
            let _g = self.ctx.lock.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: raw was returned by this context and is freed exactly once.
            unsafe { ffi::tm_cuda_buffer_free(self.ctx.raw, self.raw) };
        }
    }
}

/// A retained dispatch group (or a persistent decode program): replayed with
/// [`CudaContext::graph_launch`].  CUDA only.
pub struct CudaGraph {
    ctx: Arc<ContextInner>,
    raw: *mut ffi::TmCudaGraph,
}

unsafe impl Send for CudaGraph {}
unsafe impl Sync for CudaGraph {}

impl Drop for CudaGraph {
    fn drop(&mut self) {
        #[cfg(tm_cuda_linked)]
        {
            let _g = self.ctx.lock.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: raw was returned by this context and is freed exactly once.
            unsafe { ffi::tm_cuda_graph_free(self.ctx.raw, self.raw) };
        }
    }
}

/// Calls one `int`-returning ABI function under the context lock and maps its
/// code; `$ctx` is a `&CudaContext`.
macro_rules! call {
    ($ctx:expr, $what:literal, $f:ident ( $($arg:expr),* )) => {{
        #[cfg(tm_cuda_linked)]
        {
            let _g = $ctx.inner.lock.lock().unwrap_or_else(|e| e.into_inner());
            let mut err = [0 as c_char; ERR_CAP];
            // SAFETY: handles come from this context; `err` is ERR_CAP writable bytes.
            let rc = unsafe { ffi::$f($ctx.inner.raw, $($arg,)* err.as_mut_ptr(), ERR_CAP) };
            if rc == ffi::TM_CUDA_OK {
                Ok(())
            } else {
                Err(cuda_error(rc, err_text(&err), $what))
            }
        }
        #[cfg(not(tm_cuda_linked))]
        {
            $( let _ = &$arg; )*
            let _ = $ctx;
            unavailable::<()>()
        }
    }};
}

impl CudaBuffer {
    pub fn len(&self) -> usize {
        self.len
    }
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }
    pub fn is_shared(&self) -> bool {
        self.shared
    }
    fn raw(&self) -> *mut ffi::TmCudaBuffer {
        self.raw
    }
}

impl CudaContext {
    /// Open device `device` (0-based).
    pub fn open(device: i32) -> Result<Self> {
        #[cfg(tm_cuda_linked)]
        {
            let mut err = [0 as c_char; ERR_CAP];
            // SAFETY: err points to ERR_CAP writable bytes.
            let raw = unsafe { ffi::tm_cuda_create(device as c_int, err.as_mut_ptr(), ERR_CAP) };
            if raw.is_null() {
                return Err(cuda_error(ffi::TM_CUDA_ERR_NO_DEVICE, err_text(&err), "create")
                    .with_action("Ensure the machine has an sm_100 GPU and the process may use it."));
            }
            Ok(Self { inner: Arc::new(ContextInner { raw, lock: Mutex::new(()) }) })
        }
        #[cfg(not(tm_cuda_linked))]
        {
            let _ = device;
            unavailable()
        }
    }

    /// Allocate `bytes`; `shared` buffers are pinned host memory the device can
    /// address (readable through [`CudaContext::download_after`]).
    pub fn buffer(&self, bytes: usize, shared: bool) -> Result<CudaBuffer> {
        #[cfg(tm_cuda_linked)]
        {
            let _g = self.inner.lock.lock().unwrap_or_else(|e| e.into_inner());
            let mut err = [0 as c_char; ERR_CAP];
            // SAFETY: ctx is live; err is writable.
            let raw = unsafe {
                ffi::tm_cuda_buffer_new(self.inner.raw, bytes, shared as c_int, err.as_mut_ptr(), ERR_CAP)
            };
            if raw.is_null() {
                return Err(cuda_error(ffi::TM_CUDA_ERR_ALLOC, err_text(&err), "buffer"));
            }
            Ok(CudaBuffer { ctx: self.inner.clone(), raw, len: bytes, shared })
        }
        #[cfg(not(tm_cuda_linked))]
        {
            let _ = (bytes, shared);
            unavailable()
        }
    }

    /// A handle on `len` bytes of `parent` at `off` (16-byte aligned).  CUDA only.
    pub fn buffer_view(&self, parent: &CudaBuffer, off: usize, len: usize) -> Result<CudaBuffer> {
        #[cfg(tm_cuda_linked)]
        {
            let _g = self.inner.lock.lock().unwrap_or_else(|e| e.into_inner());
            let mut err = [0 as c_char; ERR_CAP];
            // SAFETY: parent belongs to this context (checked by the C layer too).
            let raw = unsafe {
                ffi::tm_cuda_buffer_view(self.inner.raw, parent.raw(), off, len, err.as_mut_ptr(), ERR_CAP)
            };
            if raw.is_null() {
                return Err(cuda_error(ffi::TM_CUDA_ERR_BOUNDS, err_text(&err), "buffer_view"));
            }
            Ok(CudaBuffer { ctx: self.inner.clone(), raw, len, shared: parent.shared })
        }
        #[cfg(not(tm_cuda_linked))]
        {
            let _ = (parent, off, len);
            unavailable()
        }
    }

    pub fn zero(&self, b: &CudaBuffer, off: usize, len: usize) -> Result<()> {
        call!(self, "buffer_zero", tm_cuda_buffer_zero(b.raw(), off, len))
    }
    pub fn upload(&self, dst: &CudaBuffer, off: usize, src: &[u8]) -> Result<()> {
        call!(self, "upload", tm_cuda_upload(dst.raw(), off, src.as_ptr() as *const c_void, src.len()))
    }
    pub fn download(&self, src: &CudaBuffer, off: usize, dst: &mut [u8]) -> Result<()> {
        call!(self, "download", tm_cuda_download(src.raw(), off, dst.as_mut_ptr() as *mut c_void, dst.len()))
    }
    /// Read a shared buffer once the first `completed_target` dispatches are done.
    pub fn download_after(&self, src: &CudaBuffer, off: usize, dst: &mut [u8], completed_target: u64) -> Result<()> {
        call!(self, "download_after",
              tm_cuda_download_after(src.raw(), off, dst.as_mut_ptr() as *mut c_void, dst.len(), completed_target))
    }

    // ---- grouped encoding -------------------------------------------------
    pub fn begin_group(&self) -> Result<()> {
        call!(self, "begin_group", tm_cuda_begin_group())
    }
    pub fn end_group(&self) -> Result<()> {
        call!(self, "end_group", tm_cuda_end_group())
    }
    pub fn abort_group(&self) -> Result<()> {
        call!(self, "abort_group", tm_cuda_abort_group())
    }
    pub fn fence(&self) -> Result<()> {
        call!(self, "fence", tm_cuda_fence())
    }
    /// End the open group without running it and keep it replayable.  CUDA only.
    pub fn end_group_retain(&self) -> Result<CudaGraph> {
        let mut raw: *mut ffi::TmCudaGraph = std::ptr::null_mut();
        call!(self, "end_group_retain", tm_cuda_end_group_retain(&mut raw as *mut _))?;
        Ok(CudaGraph { ctx: self.inner.clone(), raw })
    }
    pub fn graph_launch(&self, g: &CudaGraph) -> Result<()> {
        call!(self, "graph_launch", tm_cuda_graph_launch(g.raw))
    }

    // ---- counters -----------------------------------------------------------
    pub fn committed_dispatches(&self) -> u64 {
        #[cfg(tm_cuda_linked)]
        // SAFETY: reads an atomic of a live context.
        return unsafe { ffi::tm_cuda_committed_dispatches(self.inner.raw) };
        #[cfg(not(tm_cuda_linked))]
        0
    }
    pub fn completed_dispatches(&self) -> u64 {
        #[cfg(tm_cuda_linked)]
        // SAFETY: as above.
        return unsafe { ffi::tm_cuda_completed_dispatches(self.inner.raw) };
        #[cfg(not(tm_cuda_linked))]
        0
    }
    pub fn allocated_bytes(&self) -> u64 {
        #[cfg(tm_cuda_linked)]
        // SAFETY: as above.
        return unsafe { ffi::tm_cuda_allocated_bytes(self.inner.raw) };
        #[cfg(not(tm_cuda_linked))]
        0
    }
    /// Always 0: `tm_cuda_buffer_free` waits for committed work instead of leasing storage.
    pub fn in_flight_bytes(&self) -> u64 {
        #[cfg(tm_cuda_linked)]
        // SAFETY: as above.
        return unsafe { ffi::tm_cuda_in_flight_bytes(self.inner.raw) };
        #[cfg(not(tm_cuda_linked))]
        0
    }
    pub fn gpu_nanos_total(&self) -> u64 {
        #[cfg(tm_cuda_linked)]
        // SAFETY: as above.
        return unsafe { ffi::tm_cuda_gpu_nanos_total(self.inner.raw) };
        #[cfg(not(tm_cuda_linked))]
        0
    }
    pub fn set_profiling(&self, enabled: bool) {
        #[cfg(tm_cuda_linked)]
        {
            let _g = self.inner.lock.lock().unwrap_or_else(|e| e.into_inner());
            // SAFETY: live context.
            unsafe { ffi::tm_cuda_profile_set(self.inner.raw, enabled as c_int) };
        }
        #[cfg(not(tm_cuda_linked))]
        let _ = enabled;
    }
    /// (operator, nanoseconds, count) rows attributed since profiling was switched on.
    pub fn profile_snapshot(&self) -> Vec<(String, u64, u64)> {
        let mut rows = Vec::new();
        #[cfg(tm_cuda_linked)]
        {
            let _g = self.inner.lock.lock().unwrap_or_else(|e| e.into_inner());
            let mut name = [0 as c_char; 128];
            let (mut nanos, mut count) = (0u64, 0u64);
            let mut i = 0u32;
            // SAFETY: name is 128 writable bytes; the out pointers are valid.
            while unsafe {
                ffi::tm_cuda_profile_read(self.inner.raw, i, name.as_mut_ptr(), name.len(), &mut nanos, &mut count)
            } != 0
            {
                rows.push((err_text(&name), nanos, count));
                i += 1;
            }
        }
        rows
    }

    // ---- elementwise ----------------------------------------------------------
    pub fn f32_scale(&self, x: &CudaBuffer, y: &CudaBuffer, factor: f32, n: u32) -> Result<()> {
        call!(self, "f32_scale", tm_cuda_f32_scale(x.raw(), y.raw(), factor, n))
    }
    pub fn f32_axpy(&self, a: &CudaBuffer, y: &CudaBuffer, alpha: f32, n: u32) -> Result<()> {
        call!(self, "f32_axpy", tm_cuda_f32_axpy(a.raw(), y.raw(), alpha, n))
    }
    pub fn copy_f32(&self, src: &CudaBuffer, src_off: u32, dst: &CudaBuffer, dst_off: u32, n: u32) -> Result<()> {
        call!(self, "copy_f32", tm_cuda_copy_f32(src.raw(), src_off, dst.raw(), dst_off, n))
    }
    pub fn cast_f16_f32(&self, x: &CudaBuffer, y: &CudaBuffer, n: u32) -> Result<()> {
        call!(self, "cast_f16_f32", tm_cuda_cast_f16_f32(x.raw(), y.raw(), n))
    }
    pub fn cast_f32_f16(&self, x: &CudaBuffer, y: &CudaBuffer, n: u32) -> Result<()> {
        call!(self, "cast_f32_f16", tm_cuda_cast_f32_f16(x.raw(), y.raw(), n))
    }
    pub fn argmax_f32(&self, x: &CudaBuffer, n: u32, partial: &CudaBuffer, out: &CudaBuffer, out_index: u32) -> Result<()> {
        call!(self, "argmax_f32", tm_cuda_argmax_f32(x.raw(), n, partial.raw(), out.raw(), out_index))
    }
    pub fn rmsnorm(&self, x: &CudaBuffer, weight: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32, eps: f32) -> Result<()> {
        call!(self, "rmsnorm_f32", tm_cuda_rmsnorm_f32(x.raw(), weight.raw(), y.raw(), rows, cols, eps))
    }
    /// `x[row] += rmsnorm(p[row]) * weight` as one launch.  CUDA only.
    pub fn rmsnorm_add(&self, p: &CudaBuffer, weight: &CudaBuffer, x: &CudaBuffer, rows: u32, cols: u32, eps: f32) -> Result<()> {
        call!(self, "rmsnorm_add_f32", tm_cuda_rmsnorm_add_f32(p.raw(), weight.raw(), x.raw(), rows, cols, eps))
    }
    pub fn silu_mul(&self, gate: &CudaBuffer, up: &CudaBuffer, out: &CudaBuffer, n: u32) -> Result<()> {
        call!(self, "silu_mul_f32", tm_cuda_silu_mul_f32(gate.raw(), up.raw(), out.raw(), n))
    }
    pub fn gelu_tanh_mul(&self, gate: &CudaBuffer, up: &CudaBuffer, out: &CudaBuffer, n: u32) -> Result<()> {
        call!(self, "gelu_tanh_mul_f32", tm_cuda_gelu_tanh_mul_f32(gate.raw(), up.raw(), out.raw(), n))
    }

    // ---- Q8_0 -------------------------------------------------------------------
    /// Bytes of the packed (two-plane) form of a `rows x cols` Q8_0 matrix.  CUDA only.
    pub fn q8_0_packed_bytes(rows: u32, cols: u32) -> usize {
        #[cfg(tm_cuda_linked)]
        // SAFETY: pure function.
        return unsafe { ffi::tm_cuda_q8_0_packed_bytes(rows, cols) };
        #[cfg(not(tm_cuda_linked))]
        {
            let _ = (rows, cols);
            0
        }
    }
    /// Repack raw GGUF rows (34-byte blocks) into rows `[row0, row0 + nrows)` of `dst`.  CUDA only:
    /// the engine's `Matrix::load` calls this per staging chunk where the Metal path uploads verbatim.
    #[allow(clippy::too_many_arguments)]
    pub fn q8_0_pack(&self, dst: &CudaBuffer, rows: u32, cols: u32, raw: &CudaBuffer, raw_off: usize, row0: u32, nrows: u32) -> Result<()> {
        call!(self, "q8_0_pack", tm_cuda_q8_0_pack(dst.raw(), rows, cols, raw.raw(), raw_off, row0, nrows))
    }
    pub fn q8_0_gemv(&self, w: &CudaBuffer, x: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32) -> Result<()> {
        call!(self, "q8_0_gemv", tm_cuda_q8_0_gemv(w.raw(), x.raw(), y.raw(), rows, cols))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn q8_0_gemm(&self, w: &CudaBuffer, x: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32, batch: u32, x_off: u32, y_off: u32) -> Result<()> {
        call!(self, "q8_0_gemm", tm_cuda_q8_0_gemm(w.raw(), x.raw(), y.raw(), rows, cols, batch, x_off, y_off))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn q8_0_gemm_mma(&self, w: &CudaBuffer, x: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32, batch: u32, x_off: u32, y_off: u32) -> Result<()> {
        call!(self, "q8_0_gemm_mma", tm_cuda_q8_0_gemm_mma(w.raw(), x.raw(), y.raw(), rows, cols, batch, x_off, y_off))
    }
    /// GEMV with the neighbouring elementwise operators folded in.  CUDA only.
    #[allow(clippy::too_many_arguments)]
    pub fn q8_0_gemv_fused(&self, w: &CudaBuffer, x: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32, prologue: Prologue,
                           pro: Option<&CudaBuffer>, eps: f32, epilogue: Epilogue) -> Result<()> {
        let pro = pro.map_or(std::ptr::null_mut(), CudaBuffer::raw);
        call!(self, "q8_0_gemv_fused",
              tm_cuda_q8_0_gemv_fused(w.raw(), x.raw(), y.raw(), rows, cols, prologue as c_int, pro, eps, epilogue as c_int))
    }
    pub fn q8_0_row(&self, w: &CudaBuffer, out: &CudaBuffer, row: u32, cols: u32, out_off: u32) -> Result<()> {
        call!(self, "q8_0_row_f32", tm_cuda_q8_0_row_f32(w.raw(), out.raw(), row, cols, out_off))
    }
    // F16-weight matrices (rows * cols binary16, uploaded verbatim): crates/metal/src/lib.rs f16_gemv / f16_gemm / f16_row.
    pub fn f16_gemv(&self, w: &CudaBuffer, x: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32) -> Result<()> {
        call!(self, "f16_gemv", tm_cuda_f16_gemv(w.raw(), x.raw(), y.raw(), rows, cols))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn f16_gemm(&self, w: &CudaBuffer, x: &CudaBuffer, y: &CudaBuffer, rows: u32, cols: u32, batch: u32, x_off: u32, y_off: u32) -> Result<()> {
        call!(self, "f16_gemm", tm_cuda_f16_gemm(w.raw(), x.raw(), y.raw(), rows, cols, batch, x_off, y_off))
    }
    pub fn f16_row(&self, w: &CudaBuffer, out: &CudaBuffer, row: u32, cols: u32, out_off: u32) -> Result<()> {
        call!(self, "f16_row_f32", tm_cuda_f16_row_f32(w.raw(), out.raw(), row, cols, out_off))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn row_indirect_f32(&self, w: &CudaBuffer, type_id: u32, rows: u32, cols: u32, ids: &CudaBuffer, slot: u32, out: &CudaBuffer) -> Result<()> {
        call!(self, "row_indirect_f32", tm_cuda_row_indirect_f32(w.raw(), type_id, rows, cols, ids.raw(), slot, out.raw()))
    }

    // ---- attention ---------------------------------------------------------------
    #[allow(clippy::too_many_arguments)]
    pub fn qwen35_rope_partial(&self, q: &CudaBuffer, k: &CudaBuffer, inv_freq: &CudaBuffer, pos: u32, n_q_heads: u32,
                               n_kv_heads: u32, head_dim: u32, n_rot: u32) -> Result<()> {
        call!(self, "qwen35_rope_partial",
              tm_cuda_qwen35_rope_partial(q.raw(), k.raw(), inv_freq.raw(), pos, n_q_heads, n_kv_heads, head_dim, n_rot))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn qwen35_rope_partial_chunk(&self, q: &CudaBuffer, k: &CudaBuffer, inv_freq: &CudaBuffer, pos0: u32, n_q_heads: u32,
                                     n_kv_heads: u32, head_dim: u32, n_rot: u32, n: u32) -> Result<()> {
        call!(self, "qwen35_rope_partial_chunk",
              tm_cuda_qwen35_rope_partial_chunk(q.raw(), k.raw(), inv_freq.raw(), pos0, n_q_heads, n_kv_heads, head_dim, n_rot, n))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn qwen35_kv_store_f16(&self, k_src: &CudaBuffer, v_src: &CudaBuffer, k_cache: &CudaBuffer, v_cache: &CudaBuffer,
                               pos: u32, cap: u32, head_dim: u32, kv_heads: u32) -> Result<()> {
        call!(self, "qwen35_kv_store_f16",
              tm_cuda_qwen35_kv_store_f16(k_src.raw(), v_src.raw(), k_cache.raw(), v_cache.raw(), pos, cap, head_dim, kv_heads))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn qwen35_kv_store_chunk(&self, k_src: &CudaBuffer, v_src: &CudaBuffer, k_cache: &CudaBuffer, v_cache: &CudaBuffer,
                                 pos0: u32, cap: u32, head_dim: u32, kv_heads: u32, n: u32) -> Result<()> {
        call!(self, "qwen35_kv_store_f16_chunk",
              tm_cuda_qwen35_kv_store_f16_chunk(k_src.raw(), v_src.raw(), k_cache.raw(), v_cache.raw(), pos0, cap, head_dim, kv_heads, n))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn qwen35_attention_f16(&self, q: &CudaBuffer, k_cache: &CudaBuffer, v_cache: &CudaBuffer, out: &CudaBuffer,
                                scratch: &CudaBuffer, heads: u32, pos: u32, cap: u32, head_dim: u32, group: u32, scale: f32) -> Result<()> {
        call!(self, "qwen35_attention_f16",
              tm_cuda_qwen35_attention_f16(q.raw(), k_cache.raw(), v_cache.raw(), out.raw(), scratch.raw(), heads, pos, cap, head_dim, group, scale))
    }
    #[allow(clippy::too_many_arguments)]
    pub fn qwen35_attention_chunk(&self, q: &CudaBuffer, k_cache: &CudaBuffer, v_cache: &CudaBuffer, out: &CudaBuffer,
                                  scratch: &CudaBuffer, heads: u32, pos0: u32, cap: u32, head_dim: u32, group: u32, scale: f32,
                                  n: u32, window: u32) -> Result<()> {
        call!(self, "qwen35_attention_f16_chunk",
              tm_cuda_qwen35_attention_f16_chunk(q.raw(), k_cache.raw(), v_cache.raw(), out.raw(), scratch.raw(), heads, pos0, cap,
                                                 head_dim, group, scale, n, window))
    }
    /// The per-token attention core with the position read from device memory.  CUDA only.
    #[allow(clippy::too_many_arguments)]
    pub fn attention_decode_dev(&self, q: &CudaBuffer, k: &CudaBuffer, v: &CudaBuffer, q_norm: &CudaBuffer, k_norm: &CudaBuffer,
                                inv_freq: &CudaBuffer, k_cache: &CudaBuffer, v_cache: &CudaBuffer, out: &CudaBuffer,
                                scratch: &CudaBuffer, pos_buf: &CudaBuffer, pos_index: u32, status: &CudaBuffer, heads: u32,
                                kv_heads: u32, head_dim: u32, n_rot: u32, cap: u32, window: u32, eps: f32, scale: f32,
                                exact: bool) -> Result<()> {
        call!(self, "attention_decode_dev",
              tm_cuda_attention_decode_dev(q.raw(), k.raw(), v.raw(), q_norm.raw(), k_norm.raw(), inv_freq.raw(), k_cache.raw(),
                                           v_cache.raw(), out.raw(), scratch.raw(), pos_buf.raw(), pos_index, status.raw(), heads,
                                           kv_heads, head_dim, n_rot, cap, window, eps, scale, exact as c_int))
    }
    /// `buf[index] += delta` on the device.  CUDA only.
    pub fn u32_add(&self, buf: &CudaBuffer, index: u32, delta: u32) -> Result<()> {
        call!(self, "u32_add", tm_cuda_u32_add(buf.raw(), index, delta))
    }
}

/// The `--kernels` string this crate answers to and the implementation name the
/// worker acknowledges (`crates/supervisor/src/options.rs:274-287` compares it
/// with the request).
pub const KERNEL_IMPL: &str = "cuda";

#[cfg(test)]
mod tests {
    use super::*;

    #[test]
    fn probe_never_panics_and_names_the_state() {
        let p = probe();
        assert!(!p.info.is_empty());
        if !p.available {
            assert!(CudaContext::open(0).is_err(), "no device or no library must be a typed refusal");
        }
    }

    #[test]
    fn error_codes_map_like_the_metal_crate() {
        assert_eq!(cuda_error(ffi::TM_CUDA_ERR_NO_DEVICE, "x".into(), "t").code(), ErrorCode::Unavailable);
        assert_eq!(cuda_error(ffi::TM_CUDA_ERR_BOUNDS, "x".into(), "t").code(), ErrorCode::InvalidRequest);
        assert_eq!(cuda_error(ffi::TM_CUDA_ERR_INTERNAL, "x".into(), "t").code(), ErrorCode::Internal);
    }
}
