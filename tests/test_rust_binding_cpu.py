"""crates/cuda (the Rust side of the drop-in, source only: there is no Rust
toolchain to compile it here) must declare the C ABI exactly as
include/tm_cuda.h does: every exported function once, with the same number of
arguments, in the header's order -- the check a maintainer would otherwise get
from the linker.  Mirrors how crates/metal/src/lib.rs:34-666 restates
native/metal/tm_metal.h."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def header_prototypes():
    text = (ROOT / "include" / "tm_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = text[text.index('extern "C" {'):]
    out = []
    for m in re.finditer(r"\b(tm_cuda_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        args = m.group(2).strip()
        out.append((m.group(1), 0 if args in ("", "void") else len(args.split(","))))
    return out


def rust_prototypes():
    text = (ROOT / "crates" / "cuda" / "src" / "lib.rs").read_text()
    block = text[text.index('extern "C" {'):]
    block = block[:block.index("\n    }\n")]
    out = []
    for m in re.finditer(r"pub fn (tm_cuda_[a-z0-9_]+)\(([^)]*)\)", block):
        args = m.group(2).strip()
        out.append((m.group(1), 0 if not args else len(args.split(","))))
    return out


def test_every_header_function_is_declared_once_with_the_same_arity():
    c, r = header_prototypes(), rust_prototypes()
    assert len(c) >= 90
    assert [n for n, _ in r] == [n for n, _ in c], "the Rust extern block must follow the header, name by name"
    for (name, n_c), (_, n_r) in zip(c, r):
        assert n_c == n_r, f"{name}: {n_c} arguments in tm_cuda.h, {n_r} in crates/cuda"


def test_safe_wrapper_covers_the_reference_context_surface():
    """The method names the engine calls on the reference's MetalContext
    (crates/metal/src/lib.rs:755-2480) exist on CudaContext."""
    text = (ROOT / "crates" / "cuda" / "src" / "lib.rs").read_text()
    for method in ["buffer", "begin_group", "end_group", "abort_group", "fence", "committed_dispatches",
                   "completed_dispatches", "allocated_bytes", "in_flight_bytes", "gpu_nanos_total", "set_profiling",
                   "profile_snapshot", "q8_0_gemv", "q8_0_gemm", "q8_0_gemm_mma", "q8_0_row", "row_indirect_f32",
                   "rmsnorm", "silu_mul", "gelu_tanh_mul", "f32_axpy", "f32_scale", "copy_f32", "argmax_f32",
                   "qwen35_rope_partial", "qwen35_rope_partial_chunk", "qwen35_kv_store_f16", "qwen35_kv_store_chunk",
                   "qwen35_attention_f16", "qwen35_attention_chunk", "upload", "download", "download_after", "zero"]:
        assert re.search(rf"pub fn {method}\(", text), f"CudaContext::{method} is missing"
    for code in ("Unavailable", "InvalidRequest", "Internal"):
        assert f"ErrorCode::{code}" in text
