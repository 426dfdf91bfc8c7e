"""Q8_0 GEMV / exact GEMM / repack parity through the C ABI, mirroring the
reference's device tests (crates/metal/src/tests.rs:310-406, 835-921)."""
import numpy as np
import pytest

from conftest import rel_err
from tuckmill_b200 import cuda, testing as T

pytestmark = pytest.mark.gpu
TOL = 1e-4  # |gpu - cpu| <= 1e-4 * max(1, max|cpu|), the reference's GEMV rule


def run_gemv(ctx, raw, rows, cols, x):
    w = ctx.q8_0_matrix(raw, rows, cols)
    xb, yb = ctx.floats(x), ctx.buffer(rows * 4)
    ctx.q8_0_gemv(w, xb, yb, rows, cols)
    return yb.download(0, rows * 4, np.float32)


def test_one_block_of_ones_is_exactly_64(ctx):
    raw = T.q8_0_from_parts(np.ones((1, 1), np.float16), np.ones((1, 32), np.int8))
    y = run_gemv(ctx, raw, 1, 32, np.full(32, 2.0, np.float32))
    assert y[0] == 64.0


def test_zero_row_and_zero_x(ctx):
    raw = T.q8_0_from_parts(np.ones((2, 2), np.float16), np.zeros((2, 64), np.int8))
    assert np.all(run_gemv(ctx, raw, 2, 64, np.ones(64, np.float32)) == 0.0)
    raw = T.q8_0_matrix(3, 1, 5, 64)
    assert np.all(run_gemv(ctx, raw, 5, 64, np.zeros(64, np.float32)) == 0.0)


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 32), (17, 64), (5, 96), (33, 544), (1024, 1024),
                                       (2048, 1024), (3072, 1024), (1024, 3072), (1152, 6912),
                                       (256, 1152), (4096, 12288), (151936, 1024)])
def test_gemv_matches_oracle_seeded(ctx, oracle, rows, cols):
    raw = T.q8_0_matrix(0, rows * 7 + cols, rows, cols)
    x = T.activations(0, 77, cols)
    cpu = oracle.matmul_q8_0(raw, rows, cols, x)
    gpu = run_gemv(ctx, raw, rows, cols, x)
    assert rel_err(gpu, cpu) <= TOL


# The projection and head shapes of the 8B-scale and Gemma configurations: long column ranges and
# tall matrices, which take the shared-memory ring forms (8, 16 and 24 chunks deep) and the row cut
# that the small shapes above never reach.  Weights repeat with a period of 4096 rows (generating
# 600 M seeded elements would dominate the test); the activations do not.
@pytest.mark.parametrize("rows,cols", [(4096, 4096), (12288, 4096), (24576, 4096), (151936, 4096), (262144, 1152)])
def test_gemv_large_shapes_match_oracle(ctx, oracle, rows, cols):
    base = T.q8_0_matrix(4, rows + cols, 4096, cols)
    raw = np.ascontiguousarray(np.tile(base, ((rows + 4095) // 4096, 1, 1))[:rows])
    x = T.activations(4, 78, cols)
    cpu = oracle.matmul_q8_0(raw, rows, cols, x)
    gpu = run_gemv(ctx, raw, rows, cols, x)
    assert rel_err(gpu, cpu) <= TOL
    period = gpu[:rows // 4096 * 4096].reshape(-1, 4096)
    assert np.all(period == period[0]), "equal weight rows gave different results: a row-dependent path"


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 32), (17, 64), (1024, 1024), (2048, 1024)])
def test_gemv_boundary_weights(ctx, oracle, rows, cols):
    """Adversarial scales (+-65504, subnormal, +-0) and quants (-128, 127, 0)."""
    raw = T.boundary_weights(1, rows, cols)
    x = T.boundary_input(2, cols)
    cpu = oracle.matmul_q8_0(raw, rows, cols, x)
    gpu = run_gemv(ctx, raw, rows, cols, x)
    assert np.all(np.isfinite(cpu)) and rel_err(gpu, cpu) <= TOL


def test_repack_round_trip_is_bit_exact(ctx):
    for rows, cols in [(1, 32), (7, 96), (300, 1024), (129, 1152)]:
        raw = T.boundary_weights(5, rows, cols)
        w = ctx.q8_0_matrix(raw, rows, cols, chunk_rows=64)
        back = ctx.q8_0_unpack(w, rows, cols)
        assert np.array_equal(back, raw.reshape(-1))


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 7, 8, 16, 31, 32])
def test_exact_gemm_all_rows_and_bit_identity(ctx, oracle, batch):
    """Every batch equals `batch` GEMV calls bit for bit (tests.rs:895-921) and
    the oracle within tolerance; x_off / y_off respected, nothing before y_off."""
    rows, cols, x_off, y_off = 203, 1024, 32, 8
    raw = T.q8_0_matrix(0, 11, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    X = T.activations(0, 12, batch * cols).reshape(batch, cols)
    xb = ctx.floats(np.concatenate([np.zeros(x_off, np.float32), X.reshape(-1)]))
    yb = ctx.floats(np.full(y_off + batch * rows, -7.0, np.float32))
    ctx.q8_0_gemm(w, xb, yb, rows, cols, batch, x_off, y_off)
    out = yb.download(0, (y_off + batch * rows) * 4, np.float32)
    assert np.all(out[:y_off] == -7.0)
    Y = out[y_off:].reshape(batch, rows)
    assert rel_err(Y, oracle.matmul_q8_0(raw, rows, cols, X)) <= TOL
    for b in {0, batch // 2, batch - 1}:
        single = run_gemv(ctx, raw, rows, cols, X[b])
        assert np.array_equal(single, Y[b]), f"token {b} differs from the one-token GEMV"


def test_fused_prologues_and_epilogue(ctx, oracle):
    rows, cols = 515, 1024
    raw = T.q8_0_matrix(0, 21, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    x = T.activations(0, 22, cols)
    up = T.activations(0, 23, cols)
    nw = (1.0 + 0.1 * T.activations(0, 24, cols)).astype(np.float32)
    base = T.activations(0, 25, rows)
    xb, ub, nb_ = ctx.floats(x), ctx.floats(up), ctx.floats(nw)
    # rmsnorm prologue == rmsnorm kernel + gemv, bit for bit
    h = ctx.buffer(cols * 4)
    ctx.rmsnorm(xb, nb_, h, 1, cols, 1e-6)
    y0, y1 = ctx.buffer(rows * 4), ctx.buffer(rows * 4)
    ctx.q8_0_gemv(w, h, y0, rows, cols)
    ctx.q8_0_gemv_fused(w, xb, y1, rows, cols, cuda.PRO_RMSNORM, nb_, 1e-6, cuda.EPI_STORE)
    a, b = y0.download(0, rows * 4, np.float32), y1.download(0, rows * 4, np.float32)
    assert np.array_equal(a, b)
    assert rel_err(b, oracle.matmul_q8_0(raw, rows, cols, oracle.rmsnorm(x, nw, 1e-6))) <= TOL
    # silu / gelu gate prologue + accumulate epilogue
    for pro, fn in ((cuda.PRO_SILU_MUL, oracle.silu), (cuda.PRO_GELU_MUL, oracle.gelu_tanh)):
        act = np.array([fn(v) for v in x], np.float32) * up
        yb = ctx.floats(base)
        ctx.q8_0_gemv_fused(w, xb, yb, rows, cols, pro, ub, 0.0, cuda.EPI_ADD)
        got = yb.download(0, rows * 4, np.float32)
        assert rel_err(got, base + oracle.matmul_q8_0(raw, rows, cols, act)) <= TOL


def test_argument_rejection(ctx):
    """Malformed shapes are refused before any launch (tests.rs:386-406,
    kernels.rs:560-587)."""
    raw = T.q8_0_matrix(0, 1, 4, 64)
    w = ctx.q8_0_matrix(raw, 4, 64)
    x, y = ctx.buffer(64 * 4), ctx.buffer(4 * 4)
    with pytest.raises(cuda.CudaError) as e:
        ctx.q8_0_gemv(w, x, y, 4, 48)  # cols not a multiple of 32
    assert e.value.code == -4
    with pytest.raises(cuda.CudaError):
        ctx.q8_0_gemv(w, x, y, 0, 64)
    with pytest.raises(cuda.CudaError) as e:
        ctx.q8_0_gemv(w, x, y, 8, 64)  # weight buffer too small
    assert e.value.code == -4
    with pytest.raises(cuda.CudaError) as e:
        ctx.q8_0_gemv(w, ctx.buffer(32 * 4), y, 4, 64)  # x too short
    assert e.value.code == -4
    with pytest.raises(cuda.CudaError) as e:
        ctx.q8_0_gemv(x, x, y, 4, 32)  # not a packed matrix
    assert e.value.code in (-4, -5)
    with pytest.raises(cuda.CudaError):
        ctx.q8_0_gemm(w, x, y, 4, 64, 33)  # batch beyond the exact kernel's limit
    other = cuda.CudaContext(0)
    try:
        foreign = other.buffer(64 * 4)
        with pytest.raises(cuda.CudaError) as e:
            ctx.q8_0_gemv(w, foreign, y, 4, 64)  # buffer of another context
        assert e.value.code == -5
        foreign.free()
    finally:
        other.close()


def test_row_dequant_exact(ctx):
    rows, cols = 9, 96
    raw = T.boundary_weights(3, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    ref = T.q8_0_dequant(raw)
    out = ctx.floats(np.full(8 + cols, 5.0, np.float32))
    for r in (0, 4, 8):
        ctx.q8_0_row(w, out, r, cols, 8)
        got = out.download(0, (8 + cols) * 4, np.float32)
        assert np.all(got[:8] == 5.0)
        np.testing.assert_array_equal(got[8:], ref[r])
    ids = ctx.from_array(np.array([3, 100, 0xFFFFFFFF, 7], np.uint32))
    o2 = ctx.buffer(cols * 4)
    ctx.row_indirect_f32(w, 8, rows, cols, ids, 0, o2)
    np.testing.assert_array_equal(o2.download(0, cols * 4, np.float32), ref[3])
    for slot in (1, 2):  # out-of-table ids (incl. the all-NaN marker) write zeros
        ctx.row_indirect_f32(w, 8, rows, cols, ids, slot, o2)
        assert np.all(o2.download(0, cols * 4, np.float32) == 0.0)


@pytest.mark.parametrize("rows,cols", [(1536, 1152), (13824, 1152), (40, 64), (4096, 1024), (6144, 4096), (262144, 1152)])
def test_output_norm_and_residual_folded_into_the_next_projection(ctx, rows, cols):
    """tm_cuda_q8_0_gemv_addnorm is tm_cuda_rmsnorm_add_f32 followed by the norm-prologue GEMV, bit for
    bit, in one launch (every launch form the shapes select, incl. the row cut of a tall matrix)."""
    base = T.q8_0_matrix(11, rows + cols, min(rows, 4096), cols)
    raw = np.tile(base, ((rows + base.shape[0] - 1) // base.shape[0], 1, 1))[:rows]
    w = ctx.q8_0_matrix(raw, rows, cols)
    x = T.activations(11, 1, cols)
    p = (T.activations(11, 2, cols) * np.float32(5.0)).astype(np.float32)
    aw = (1 + 0.1 * T.activations(11, 3, cols)).astype(np.float32)
    nw = (1 + 0.1 * T.activations(11, 4, cols)).astype(np.float32)
    xb, pb, awb, nwb = ctx.floats(x), ctx.floats(p), ctx.floats(aw), ctx.floats(nw)
    want_x, want_y = ctx.floats(x), ctx.buffer(rows * 4)
    ctx.rmsnorm_add(pb, awb, want_x, 1, cols, 1e-6)
    ctx.q8_0_gemv_fused(w, want_x, want_y, rows, cols, cuda.PRO_RMSNORM, nwb, 1e-6)
    x_out, y = ctx.floats(np.zeros(cols, np.float32)), ctx.buffer(rows * 4)
    ctx.q8_0_gemv_addnorm(w, xb, pb, awb, x_out, nwb, y, rows, cols, 1e-6)
    np.testing.assert_array_equal(x_out.download(0, cols * 4, np.float32), want_x.download(0, cols * 4, np.float32))
    np.testing.assert_array_equal(y.download(0, rows * 4, np.float32), want_y.download(0, rows * 4, np.float32))
    np.testing.assert_array_equal(xb.download(0, cols * 4, np.float32), x)  # the input stream is left alone
    with pytest.raises(cuda.CudaError):
        ctx.q8_0_gemv_addnorm(w, xb, pb, awb, xb, nwb, y, rows, cols, 1e-6)
    for b in (w, want_y, y):
        b.free()


def test_output_norm_fold_refuses_wide_rows(ctx):
    rows, cols = 32, 8192
    w = ctx.q8_0_matrix(T.q8_0_matrix(1, 2, rows, cols), rows, cols)
    v = ctx.floats(np.zeros(cols, np.float32))
    with pytest.raises(cuda.CudaError):
        ctx.q8_0_gemv_addnorm(w, v, v, v, ctx.floats(np.zeros(cols, np.float32)), v, ctx.buffer(rows * 4), rows, cols, 1e-6)
