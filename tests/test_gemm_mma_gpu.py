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
         (40, 64, 512), (130, 1152, 129), (6144, 1024, 300), (1024, 3072, 512), (257, 2048, 640),
         (1024, 3584, 7), (384, 4096, 3), (40, 64, 3)]  # a handful of tokens: tensor cores on wide matrices only


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
    if batch < 3 or (batch < 9 and cols < 2048):
        # handed to the exact batched GEMV (one or two tokens; up to eight on a narrow matrix)
        assert rel_err(Y, cpu) <= 1e-4
    else:
        ref16 = f16_profile_reference(raw, X)
        assert rel_err(Y, ref16) <= 2e-5, "differs from the f16-operand profile by more than accumulation error"


# Shapes the launcher serves with its wider instantiations (token sub-tile 128 and 192: a different
# shared-memory ring and tensor-memory split each) and batches up to the limit of one launch.  The
# whole GEMM runs on the device; the first, middle and last 256 weight rows of Y (every token) are
# compared with the oracle and with the f16-operand profile.  The expected instantiation is asserted,
# so a change of the launcher's choice cannot silently drop the coverage.
BIG_CASES = [(3072, 1024, 512, 64),        # the single-operator configuration at its batch
             (12288, 4096, 512, 128), (4096, 4096, 2048, 128),
             (12288, 4096, 2048, 192), (4096, 4096, 8192, 192), (151936, 4096, 2048, 192)]


@pytest.mark.parametrize("rows,cols,batch,tile", BIG_CASES)
def test_mma_gemm_large_shapes_every_instantiation(ctx, oracle, rows, cols, batch, tile):
    base_rows = min(rows, 4096)
    base = T.q8_0_matrix(3, rows + cols, base_rows, cols)
    raw = np.tile(base, ((rows + base_rows - 1) // base_rows, 1, 1))[:rows]
    X = T.activations(3, 5, min(batch, 2048) * cols).reshape(-1, cols)
    X = np.tile(X, ((batch + X.shape[0] - 1) // X.shape[0], 1))[:batch]
    X = (X * (1 + 0.25 * np.arange(batch, dtype=np.float32)[:, None] / batch)).astype(np.float32)  # rows differ
    w = ctx.q8_0_matrix(raw, rows, cols)
    xb, yb = ctx.floats(X), ctx.buffer(batch * rows * 4)
    ctx.q8_0_gemm_mma(w, xb, yb, rows, cols, batch)
    Y = yb.download(0, batch * rows * 4, np.float32).reshape(batch, rows)
    assert not ctx.mma_aborted()
    assert ctx.mma_last_tile() == tile, f"launcher picked sub-tile {ctx.mma_last_tile()}, the case is meant for {tile}"
    mid = (rows // 2) // 128 * 128 + 64  # straddles a 128-row tile boundary
    for r0 in sorted({0, mid, rows - 256}):
        sub = np.ascontiguousarray(raw[r0:r0 + 256])
        got = Y[:, r0:r0 + 256]
        cpu = oracle.matmul_q8_0(sub, 256, cols, X)
        assert float(np.max(np.abs(got - cpu))) <= 2e-2, f"rows {r0}..{r0 + 256}"
        assert rel_err(got, f16_profile_reference(sub, X)) <= 2e-5, f"rows {r0}..{r0 + 256}: not the f16-operand profile"
    for b in (w, xb, yb):
        b.free()


# Few output tiles (decode batches, narrow projections): the K range is cut into parts whose sums meet
# in a workspace and are added in part order.  (rows, cols, batch, expected parts)
SPLIT_CASES = [(4096, 12288, 32, 4), (6144, 4096, 32, 2), (1024, 3072, 64, 8), (1024, 2048, 17, 8),
               (4096, 1024, 32, 4), (2048, 4096, 300, 2), (12288, 4096, 32, 1), (24576, 4096, 32, 2)]


@pytest.mark.parametrize("rows,cols,batch,parts", SPLIT_CASES)
def test_mma_gemm_split_k_is_deterministic_and_within_the_profile(ctx, oracle, rows, cols, batch, parts):
    raw = T.q8_0_matrix(5, rows + cols, rows, cols)
    X = T.activations(5, 7, batch * cols).reshape(batch, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    xb, yb = ctx.floats(X), ctx.buffer(batch * rows * 4)
    runs = []
    for _ in range(3):
        yb.zero()
        ctx.q8_0_gemm_mma(w, xb, yb, rows, cols, batch)
        runs.append(yb.download(0, batch * rows * 4, np.float32).reshape(batch, rows).copy())
    assert not ctx.mma_aborted()
    assert ctx.mma_last_split() == parts
    np.testing.assert_array_equal(runs[1], runs[0])
    np.testing.assert_array_equal(runs[2], runs[0])
    for r0 in sorted({0, rows // 2 - 64, rows - 256}):
        sub = np.ascontiguousarray(raw[r0:r0 + 256])
        got = runs[0][:, r0:r0 + 256]
        assert rel_err(got, f16_profile_reference(sub, X)) <= 2e-5, f"rows {r0}..{r0 + 256}"
        assert float(np.max(np.abs(got - oracle.matmul_q8_0(sub, 256, cols, X)))) <= 2e-2
    # the residual-adding epilogue runs after the parts are summed
    base = T.activations(5, 9, batch * rows).reshape(batch, rows)
    acc = ctx.floats(base)
    ctx.q8_0_gemm_mma_fused(w, xb, rows, cols, batch, [acc], [rows], cuda.PRO_NONE, None, 0.0, cuda.EPI_ADD)
    got = acc.download(0, batch * rows * 4, np.float32).reshape(batch, rows)
    assert ctx.mma_last_split() == parts
    np.testing.assert_array_equal(got, base + runs[0])
    for b in (w, xb, yb, acc):
        b.free()


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
    wide = ctx.q8_0_matrix(T.q8_0_matrix(0, 2, 8, 16384), 8, 16384)
    xw, yw = ctx.buffer(8192 * 16384 * 4), ctx.buffer(8192 * 8 * 4)
    ctx.begin_group()
    try:
        with pytest.raises(cuda.CudaError) as e:
            # a 256 MiB workspace, larger than any earlier test needed: it would have to grow inside a group
            ctx.q8_0_gemm_mma(wide, xw, yw, 8, 16384, 8192)
        assert e.value.code == -5
    finally:
        ctx.abort_group()


@pytest.mark.parametrize("parts,cols,batch,prologue,add", [
    ((2048, 1024, 1024), 1024, 512, cuda.PRO_RMSNORM, False),   # Qwen3-0.6B q | k | v with the input norm folded in
    ((3072, 3072), 1024, 300, cuda.PRO_RMSNORM, False),         # gate | up
    ((1024,), 3072, 200, cuda.PRO_SILU_MUL, True),              # down: silu(gate) * up in, residual add out
    ((1152,), 640, 77, cuda.PRO_GELU_MUL, True),                # Gemma-style activation, ragged sizes
    ((256, 100), 256, 40, cuda.PRO_NONE, False),                # a last part that is not a multiple of 128
])
def test_fused_prefill_gemm_equals_operator_sequence(ctx, oracle, parts, cols, batch, prologue, add):
    """One prologue-fused f16 copy + one multi-part launch against the launches it
    replaces (rmsnorm / silu_mul, one GEMM per part, axpy) and against the oracle."""
    rows = sum(parts)
    raw = T.q8_0_matrix(2, rows + cols, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    X = T.activations(2, 5, batch * cols).reshape(batch, cols)
    eps = 1e-6
    if prologue == cuda.PRO_RMSNORM:
        pro = (1 + 0.1 * T.activations(2, 6, cols)).astype(np.float32)
        xin = (X / np.sqrt((X.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + eps) * pro).astype(np.float32)
    elif prologue == cuda.PRO_NONE:
        pro, xin = None, X
    else:
        pro = T.activations(2, 7, batch * cols).reshape(batch, cols)
        x64 = X.astype(np.float64)
        act = x64 / (1 + np.exp(-x64)) if prologue == cuda.PRO_SILU_MUL else \
            0.5 * x64 * (1 + np.tanh(0.7978845608028654 * (x64 + 0.044715 * x64 ** 3)))
        xin = (act * pro).astype(np.float32)
    ref = oracle.matmul_q8_0(raw, rows, cols, xin)
    before = [T.activations(2, 20 + i, batch * p).reshape(batch, p) for i, p in enumerate(parts)]
    ys = [ctx.floats(b) for b in before]
    ctx.q8_0_gemm_mma_fused(w, ctx.floats(X), rows, cols, batch, ys, list(parts), prologue,
                            ctx.floats(pro) if pro is not None else None, eps, cuda.EPI_ADD if add else cuda.EPI_STORE)
    assert not ctx.mma_aborted()
    r0 = 0
    for y, p, b in zip(ys, parts, before):
        got = y.download(0, batch * p * 4, np.float32).reshape(batch, p)
        want = ref[:, r0:r0 + p] + (b if add else 0)
        scale = max(1.0, float(np.max(np.abs(want))))
        assert float(np.max(np.abs(got - want))) <= 2e-2 * scale, f"part at row {r0}"
        r0 += p
    with pytest.raises(cuda.CudaError):  # a middle part that would let a tile straddle two outputs
        ctx.q8_0_gemm_mma_fused(w, ctx.floats(X), rows, cols, batch, [ys[0], ys[0]], [100, rows - 100])


@pytest.mark.parametrize("heads,kvh,hd,n_rot,pos0,n,cap", [(16, 8, 128, 128, 0, 70, 100), (4, 1, 256, 256, 33, 50, 90),
                                                         (4, 2, 32, 32, 5, 9, 40), (12, 2, 64, 32, 7, 21, 64)])
def test_qk_prep_chunk_equals_operator_sequence(ctx, heads, kvh, hd, n_rot, pos0, n, cap):
    """rmsnorm (q heads), rmsnorm (k heads), rope, kv_store as one launch: same values to a few ulp."""
    eps = 1e-6
    q = T.activations(3, 1, n * heads * hd)
    k = T.activations(3, 2, n * kvh * hd)
    v = T.activations(3, 3, n * kvh * hd)
    qn = (1 + 0.1 * T.activations(3, 4, hd)).astype(np.float32)
    kn = (1 + 0.1 * T.activations(3, 5, hd)).astype(np.float32)
    inv = (1e4 ** (-np.arange(n_rot // 2, dtype=np.float64) * 2 / n_rot)).astype(np.float32)
    qnb, knb, ib = ctx.floats(qn), ctx.floats(kn), ctx.floats(inv)
    plane = kvh * cap * hd * 2
    caches = [[ctx.buffer(plane), ctx.buffer(plane)] for _ in range(2)]
    for pair in caches:
        for c in pair:
            c.zero()
    qa, ka, va = ctx.floats(q), ctx.floats(k), ctx.floats(v)
    ctx.rmsnorm(qa, qnb, qa, n * heads, hd, eps)
    ctx.rmsnorm(ka, knb, ka, n * kvh, hd, eps)
    ctx.qwen35_rope_partial_chunk(qa, ka, ib, pos0, heads, kvh, hd, n_rot, n)
    ctx.qwen35_kv_store_chunk(ka, va, caches[0][0], caches[0][1], pos0, cap, hd, kvh, n)
    qb, kb, vb = ctx.floats(q), ctx.floats(k), ctx.floats(v)
    ctx.qk_prep_chunk(qb, kb, vb, qnb, knb, ib, caches[1][0], caches[1][1], heads, kvh, hd, n_rot, pos0, cap, n, eps)
    qa_h, qb_h = qa.download(0, q.size * 4, np.float32), qb.download(0, q.size * 4, np.float32)
    assert rel_err(qb_h, qa_h) <= 2e-6
    np.testing.assert_array_equal(kb.download(0, k.size * 4, np.float32), k)  # k itself is left alone
    for a_, b_ in zip(caches[0], caches[1]):
        ca = a_.download(0, plane, np.float16).astype(np.float32)
        cb = b_.download(0, plane, np.float16).astype(np.float32)
        assert np.max(np.abs(ca - cb)) <= 2e-3 * max(1.0, float(np.max(np.abs(ca))))  # one f16 ulp at most
