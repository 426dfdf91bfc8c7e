"""F16-weight matrices: the tm_cuda_f16_* operators against the oracle's F16 dot
(crates/tuckcore/src/kernels.rs:223-232) and the engine on F16 artifacts -- the
reference's own `tiny_qwen3` fixture tensors (crates/manifest/src/testing.rs:64-81,
236-396, 611-690) and a seeded F16 twin whose rows differ -- under the invariants of
crates/tuckcore/src/engine/metal.rs:3682-3774 (prefill == decode bit for bit, ledger ==
plan) and the model-parity policy of crates/tuckcore/src/executor.rs:2143-2321."""
import numpy as np
import pytest

from tuckmill_b200 import cuda as tc, engine as E, testing as T

pytestmark = pytest.mark.gpu


def f16_matrix(seed, rows, cols):
    return (T.normals(seed, 77, 1, 0, rows * cols).reshape(rows, cols) * 0.25).astype(np.float16)


@pytest.mark.parametrize("rows,cols", [(1, 32), (7, 64), (512, 128), (300, 1024), (64, 2080), (1024, 4096), (33, 96), (5, 63)])
def test_gemv_against_the_oracle(ctx, oracle, rows, cols):
    w = f16_matrix(rows + cols, rows, cols)
    x = T.activations(3, 5, cols)
    wb, xb, yb = ctx.from_array(w), ctx.from_array(x), ctx.floats(np.zeros(rows, np.float32))
    ctx.f16_gemv(wb, xb, yb, rows, cols)
    got = yb.download(0, (rows) * 4, np.float32)
    want = oracle.matmul_f16(w, rows, cols, x)
    scale = max(1.0, float(np.max(np.abs(want))))
    # different summation order (32 lanes, stride 64) from the oracle's sequential dot
    assert np.max(np.abs(got - want)) <= 2e-5 * scale
    # exact integers: small-integer weights and activations sum exactly in any order
    wi = (np.arange(rows * cols).reshape(rows, cols) % 7 - 3).astype(np.float16)
    xi = (np.arange(cols) % 5 - 2).astype(np.float32)
    wb2, xb2 = ctx.from_array(wi), ctx.from_array(xi)
    ctx.f16_gemv(wb2, xb2, yb, rows, cols)
    np.testing.assert_array_equal(yb.download(0, (rows) * 4, np.float32), oracle.matmul_f16(wi, rows, cols, xi))


@pytest.mark.parametrize("batch", [1, 2, 3, 5, 8, 9, 31, 32])
def test_gemm_rows_are_the_gemv_bit_for_bit(ctx, batch):
    rows, cols = 96, 320
    w = f16_matrix(9, rows, cols)
    x = T.activations(4, 6, batch * cols).reshape(batch, cols)
    wb, xb = ctx.from_array(w), ctx.from_array(x)
    yb, y1 = ctx.floats(np.zeros(batch * rows, np.float32)), ctx.floats(np.zeros(rows, np.float32))
    ctx.f16_gemm(wb, xb, yb, rows, cols, batch)
    got = yb.download(0, (batch * rows) * 4, np.float32).reshape(batch, rows)
    for b in range(batch):
        xv = ctx.from_array(x[b])
        ctx.f16_gemv(wb, xv, y1, rows, cols)
        np.testing.assert_array_equal(got[b], y1.download(0, (rows) * 4, np.float32))


def test_gemm_offsets_and_limits(ctx):
    rows, cols = 40, 64
    w = f16_matrix(1, rows, cols)
    x = T.activations(2, 1, 6 * cols).reshape(6, cols)
    wb, xb, yb = ctx.from_array(w), ctx.from_array(x), ctx.floats(np.zeros(6 * rows, np.float32))
    ctx.f16_gemm(wb, xb, yb, rows, cols, 2, x_off=3 * cols, y_off=4 * rows)
    out = yb.download(0, (6 * rows) * 4, np.float32).reshape(6, rows)
    assert not out[:4].any()
    ref = ctx.floats(np.zeros(2 * rows, np.float32))
    ctx.f16_gemm(wb, ctx.from_array(x[3:5]), ref, rows, cols, 2)
    np.testing.assert_array_equal(out[4:], ref.download(0, (2 * rows) * 4, np.float32).reshape(2, rows))
    for bad in (dict(batch=0), dict(batch=33), dict(batch=2, x_off=5 * cols), dict(batch=2, y_off=5 * rows)):
        with pytest.raises(tc.CudaError):
            ctx.f16_gemm(wb, xb, yb, rows, cols, **bad)
    with pytest.raises(tc.CudaError):  # matrix smaller than rows * cols
        ctx.f16_gemv(wb, xb, yb, rows + 1, cols)


def test_rows_and_gathers(ctx):
    rows, cols = 50, 96
    w = f16_matrix(5, rows, cols)
    wb = ctx.from_array(w)
    out = ctx.floats(np.zeros(3 * cols, np.float32))
    ctx.f16_row(wb, out, 17, cols, out_off=cols)
    got = out.download(0, (3 * cols) * 4, np.float32).reshape(3, cols)
    np.testing.assert_array_equal(got[1], w[17].astype(np.float32))
    assert not got[0].any() and not got[2].any()
    ids = np.array([4, 49, 50, 0, 1000, 17], np.uint32)  # 50 and 1000 are outside: zeros
    idb = ctx.from_array(ids)
    many = ctx.floats(np.zeros(4 * cols, np.float32))
    ctx.f16_rows_indirect(wb, rows, cols, idb, 1, 4, 2.0, many)
    got = many.download(0, (4 * cols) * 4, np.float32).reshape(4, cols)
    np.testing.assert_array_equal(got[0], w[49].astype(np.float32) * 2.0)
    assert not got[1].any() and not got[3].any()
    np.testing.assert_array_equal(got[2], w[0].astype(np.float32) * 2.0)
    pos = ctx.from_array(np.array([0, 3], np.uint32))
    one = ctx.floats(np.zeros(cols, np.float32))
    ctx.f16_row_indirect_dev(wb, rows, cols, idb, 2, pos, 1, 0, 0.0, one)  # slot 2 + pos[1] = 5
    np.testing.assert_array_equal(one.download(0, (cols) * 4, np.float32), w[17].astype(np.float32))
    ctx.f16_row_indirect_dev(wb, rows, cols, idb, 0, None, 0, 0, 0.0, one)  # no position buffer: slot = base
    np.testing.assert_array_equal(one.download(0, (cols) * 4, np.float32), w[4].astype(np.float32))


def test_fused_forms_equal_their_unfused_sequences(ctx, oracle):
    rows, cols = 72, 256
    w = f16_matrix(2, rows, cols)
    x = T.activations(8, 2, cols)
    g = (1.0 + 0.1 * T.normals(8, 3, 1, 0, cols)).astype(np.float32)
    wb, xb, gb = ctx.from_array(w), ctx.from_array(x), ctx.from_array(g)
    yb, hb, ref = ctx.floats(np.zeros(rows, np.float32)), ctx.floats(np.zeros(cols, np.float32)), ctx.floats(np.zeros(rows, np.float32))
    ctx.rmsnorm(xb, gb, hb, 1, cols, 1e-6)
    ctx.f16_gemv(wb, hb, ref, rows, cols)
    ctx.f16_gemv_fused(wb, xb, yb, rows, cols, tc.PRO_RMSNORM, gb, 1e-6)
    np.testing.assert_array_equal(yb.download(0, (rows) * 4, np.float32), ref.download(0, (rows) * 4, np.float32))
    for pro, act in ((tc.PRO_SILU_MUL, ctx.silu_mul), (tc.PRO_GELU_MUL, ctx.gelu_tanh_mul)):
        u = ctx.from_array(T.activations(8, 4, cols))
        a = ctx.from_array(x)
        base = ctx.from_array(np.arange(rows, dtype=np.float32))
        ctx.f16_gemv_fused(wb, a, base, rows, cols, pro, u, 0.0, tc.EPI_ADD)
        act(a, u, a, cols)
        ctx.f16_gemv(wb, a, ref, rows, cols)
        np.testing.assert_array_equal(base.download(0, (rows) * 4, np.float32),
                                      ref.download(0, (rows) * 4, np.float32) + np.arange(rows, dtype=np.float32))


@pytest.fixture(scope="module", params=["fixture-f16", "seeded-f16"])
def artifact(request, tmp_path_factory):
    path = tmp_path_factory.mktemp("f16") / f"tiny_qwen3_{request.param}.gguf"
    T.write_gguf(path, T.TINY_QWEN3, seed=3, norm_jitter=0.1, fill=request.param)
    return path, T.TINY_QWEN3, request.param


def scale_of(v):
    return max(1.0, float(np.max(np.abs(v))))


@pytest.mark.parametrize("n_prompt,batch", [(1, 16), (3, 16), (16, 16), (20, 16), (128, 128), (132, 128)])
def test_engine_prefill_equals_decode_on_f16_weights(ctx, artifact, n_prompt, batch):
    path, shape, _ = artifact
    toks = T.token_ids(9, n_prompt, shape.vocab)
    eng = E.Engine(path, context=160, exact=True, prefill_batch=batch)
    eng.reset()
    for t in toks[:-1]:
        eng.step(int(t), want_logits=False)
    by_token = eng.step(int(toks[-1]))
    eng.reset()
    eng.prefill(toks, want_token=True)
    np.testing.assert_array_equal(eng.logits(), by_token)
    assert eng.prefill_token() == int(np.argmax(by_token))
    eng.close()


@pytest.mark.parametrize("exact", [True, False])
def test_engine_on_f16_weights_matches_the_oracle(ctx, oracle, artifact, exact):
    path, shape, fill = artifact
    cpu = oracle.Model(path)
    assert cpu.weight_type == 1
    toks = T.token_ids(5, 24, shape.vocab)
    cpu.reset(64)
    ref = np.stack([cpu.forward([t]) for t in toks])
    eng = E.Engine(path, context=64, exact=exact, prefill_batch=16)
    got = eng.score(toks)
    for i in range(len(toks)):
        assert np.max(np.abs(got[i] - ref[i])) <= 1e-2 * scale_of(ref[i]), f"position {i}"
        if fill == "seeded-f16":  # the fixture's head rows are all equal: every logit ties
            assert int(np.argmax(got[i])) == oracle.argmax(ref[i])
    prompt = T.token_ids(11, 20, shape.vocab)
    cpu.reset(64)
    want, margins = cpu.generate_greedy(prompt, 24, chunk=16)
    tokens, stats = eng.generate(prompt, 24)
    assert stats.generated == 24
    if fill == "seeded-f16":
        bad = np.nonzero(tokens != want)[0]
        assert bad.size == 0, f"first divergence at step {bad[0]} (oracle top-1 margin {margins[bad[0]]:.3g})"
    i = eng.info
    assert i.allocated_bytes == i.plan_weights + i.plan_state + i.plan_scratch
    eng.close()


def test_f16_models_take_the_graph_even_when_the_program_is_asked_for(ctx, artifact):
    path, shape, _ = artifact
    eng = E.Engine(path, context=32, persistent_step=True)
    assert eng.decode_program() == 0
    toks, _ = eng.generate(T.token_ids(1, 4, shape.vocab), 4)
    assert len(toks) == 4
    eng.close()
