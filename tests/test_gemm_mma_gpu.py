"""The tensor-core prefill GEMM through the C ABI: the reference's matrix-unit
GEMM cases (crates/metal/src/tests.rs:1169-1247 -- row tails, partial token
tiles, x_off / y_off, nothing written before y_off, batch limits) under the
declared f16-operand profile: |gpu - oracle| <= 2e-2 per output, and agreement
with an f16-operand reference to accumulation error."""
import numpy as np
import pytest

from conftest import rel_err
from tuckmill_b200 import cuda, testing as T

pytestmark = pytest.mark.gpu
CASES = [(16, 1024, 16), (3584, 1024, 16), (3584, 1024, 32), (40, 64, 27), (1024, 3584, 64), (100, 96, 77),
         (40, 64, 512), (130, 1152, 129), (6144, 1024, 300), (1024, 3072, 512), (257, 2048, 640)]


def f16_profile_reference(raw, X):
    """x and d*q each rounded once to binary16, exact products, wide accumulation."""
    w16 = T.q8_0_dequant(raw).astype(np.float16).astype(np.float64)
    return X.astype(np.float16).astype(np.float64) @ w16.T


@pytest.mark.parametrize("rows,cols,batch", CASES)
def test_mma_gemm_matches_oracle_and_f16_profile(ctx, oracle, rows, cols, batch):
    x_off, y_off = 32, 8
    raw = T.q8_0_matrix(0, rows + cols, rows, cols)
    X = T.activations(0, 5, batch * cols).reshape(batch, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    xb = ctx.floats(np.concatenate([np.zeros(x_off, np.float32), X.reshape(-1)]))
    yb = ctx.floats(np.full(y_off + batch * rows, -7.0, np.float32))
    ctx.q8_0_gemm_mma(w, xb, yb, rows, cols, batch, x_off, y_off)
    out = yb.download(0, (y_off + batch * rows) * 4, np.float32)
    assert not ctx.mma_aborted()
    assert np.all(out[:y_off] == -7.0), "wrote before y_off"
    Y = out[y_off:].reshape(batch, rows)
    cpu = oracle.matmul_q8_0(raw, rows, cols, X)
    assert float(np.max(np.abs(Y - cpu))) <= 2e-2
    ref16 = f16_profile_reference(raw, X)
    assert rel_err(Y, ref16) <= 2e-5, "differs from the f16-operand profile by more than accumulation error"


def test_mma_gemm_row_view_and_larger_scales(ctx, oracle):
    """A projection stored inside a fused matrix (row view), scales up to ~1."""
    rows, cols, batch = 384, 512, 200
    nb = cols // 32
    d = (np.abs(T.normals(1, 3, 1, 0, rows * nb)) * 0.01).astype(np.float16).reshape(rows, nb)
    q = T.uniform_quants(1, 4, 0, rows * cols).reshape(rows, cols)
    raw = T.q8_0_from_parts(d, q)
    X = T.activations(1, 5, batch * cols).reshape(batch, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    part = ctx.q8_0_row_view(w, rows, cols, 128, 200)
    xb, yb = ctx.floats(X), ctx.buffer(batch * 200 * 4)
    ctx.q8_0_gemm_mma(part, xb, yb, 200, cols, batch)
    Y = yb.download(0, batch * 200 * 4, np.float32).reshape(batch, 200)
    assert not ctx.mma_aborted()
    assert rel_err(Y, f16_profile_reference(raw[128:328], X)) <= 2e-5
    assert rel_err(Y, oracle.matmul_q8_0(raw[128:328], 200, cols, X)) <= 2e-3


def test_mma_gemm_limits(ctx):
    raw = T.q8_0_matrix(0, 1, 40, 64)
    w = ctx.q8_0_matrix(raw, 40, 64)
    x, y = ctx.buffer(8193 * 64 * 4), ctx.buffer(8193 * 40 * 4)
    with pytest.raises(cuda.CudaError) as e:
        ctx.q8_0_gemm_mma(w, x, y, 40, 64, 8193)
    assert e.value.code == -4
    with pytest.raises(cuda.CudaError):
        ctx.q8_0_gemm_mma(w, ctx.buffer(16), y, 40, 64, 64)
    wide = ctx.q8_0_matrix(T.q8_0_matrix(0, 2, 8, 8192), 8, 8192)
    xw, yw = ctx.buffer(4096 * 8192 * 4), ctx.buffer(4096 * 8 * 4)
    ctx.begin_group()
    try:
        with pytest.raises(cuda.CudaError) as e:
            ctx.q8_0_gemm_mma(wide, xw, yw, 8, 8192, 4096)  # the 64 MiB workspace would have to grow inside a group
        assert e.value.code == -5
    finally:
        ctx.abort_group()
