"""Decode steps of several sequences at once (no counterpart in the reference, which serves one
request at a time: crates/supervisor/src/queue.rs:1-4).  The bar: a sequence decoded in a batch is
the sequence decoded alone -- bit for bit wherever the same kernels run (`exact` mode; small batches
of models whose attention has no tensor-core form), within the tolerance-qualified kernels' bars
otherwise -- so every parity statement about the one-sequence engine carries over."""
import numpy as np
import pytest

from tuckmill_b200 import cuda, engine as E, testing as T

pytestmark = pytest.mark.gpu


def f32(buf, n, off=0):
    return buf.download(off * 4, n * 4, np.float32)


# ---------------------------------------------------------------- operators

@pytest.mark.parametrize("exact", [True, False])
@pytest.mark.parametrize("heads,kvh,hd,window", [(16, 8, 128, 0), (4, 1, 256, 40), (4, 2, 32, 0)])
def test_batched_decode_attention_is_the_single_call_per_sequence(ctx, exact, heads, kvh, hd, window):
    cap, eps, S = 150, 1e-6, 5
    scale = 1.0 / np.sqrt(np.float32(hd))
    positions = np.array([0, 63, 64, 149, 17], np.uint32)  # empty cache, split edges, the last row
    qn = ctx.floats((1 + 0.1 * T.activations(0, 20, hd)).astype(np.float32))
    kn = ctx.floats((1 + 0.1 * T.activations(0, 21, hd)).astype(np.float32))
    inv = ctx.floats((1e4 ** (-np.arange(hd // 2, dtype=np.float64) * 2 / hd)).astype(np.float32))
    plane = kvh * cap * hd
    kfill = T.activations(1, 1, S * plane).astype(np.float16)
    vfill = T.activations(1, 2, S * plane).astype(np.float16)
    width = (heads + 2 * kvh) * hd  # one [S][q|k|v] projection output: the strided form
    qkv = T.activations(2, 3, S * width).reshape(S, width)
    status = ctx.buffer(4, shared=True)
    status.zero()
    per_seq = cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap)

    # one call per sequence on its own planes
    want, want_k, want_v = [], [], []
    for s in range(S):
        kc = ctx.from_array(kfill[s * plane:(s + 1) * plane])
        vc = ctx.from_array(vfill[s * plane:(s + 1) * plane])
        q = ctx.floats(qkv[s, :heads * hd])
        k = ctx.floats(qkv[s, heads * hd:(heads + kvh) * hd])
        v = ctx.floats(qkv[s, (heads + kvh) * hd:])
        out, sb = ctx.buffer(heads * hd * 4), ctx.buffer(per_seq)
        sb.zero()
        pos = ctx.from_array(positions[s:s + 1])
        ctx.attention_decode_dev(q, k, v, qn, kn, inv, kc, vc, out, sb, pos, 0, status, heads, kvh, hd, hd, cap, window,
                                 eps, scale, exact=exact)
        ctx.fence()
        want.append(f32(out, heads * hd))
        want_k.append(kc.download(0, plane * 2, np.float16))
        want_v.append(vc.download(0, plane * 2, np.float16))

    for strided in (False, True):
        kc, vc = ctx.from_array(kfill), ctx.from_array(vfill)
        out, sb = ctx.buffer(S * heads * hd * 4), ctx.buffer(S * per_seq)
        sb.zero()
        pos = ctx.from_array(positions)
        if strided:
            whole = ctx.floats(qkv)
            n = S * width * 4
            q, k, v = whole.view(0, n), whole.view(heads * hd * 4, n - heads * hd * 4), \
                whole.view((heads + kvh) * hd * 4, n - (heads + kvh) * hd * 4)
            strides = dict(q_stride=width, kv_stride=width)
        else:
            q = ctx.floats(qkv[:, :heads * hd])
            k = ctx.floats(qkv[:, heads * hd:(heads + kvh) * hd])
            v = ctx.floats(qkv[:, (heads + kvh) * hd:])
            strides = {}
        for _ in range(2):  # the second launch finds the counters the first one left
            ctx.attention_decode_batch(q, k, v, qn, kn, inv, kc, vc, out, sb, pos, status, S, heads, kvh, hd, hd, cap,
                                       window, eps, scale, exact, **strides)
        ctx.fence()
        got = f32(out, S * heads * hd).reshape(S, heads * hd)
        # Head size 128 outside `exact` mode: batches run the tensor-core form (f16 Q and weights,
        # base-2 exponentials), qualified at 2e-3 of the output scale like the prefill form;
        # everywhere else the batch is the single call's kernel with one more grid dimension.
        tensor_core = not exact and hd == 128
        for s in range(S):
            gk = kc.download(s * plane * 2, plane * 2, np.float16)
            gv = vc.download(s * plane * 2, plane * 2, np.float16)
            if tensor_core:
                tol = 2e-3 * max(1.0, float(np.max(np.abs(want[s]))))
                assert np.max(np.abs(got[s] - want[s])) <= tol, f"sequence {s} (strided={strided})"
                assert np.max(np.abs(gk.astype(np.float32) - want_k[s].astype(np.float32))) <= 4e-3
                np.testing.assert_array_equal(gv, want_v[s])
            else:
                np.testing.assert_array_equal(got[s], want[s], err_msg=f"sequence {s} (strided={strided})")
                np.testing.assert_array_equal(gk, want_k[s])
                np.testing.assert_array_equal(gv, want_v[s])
    assert int(status.download(0, 4, np.uint32)[0]) == 0
    # a sequence past its capacity writes nothing and raises the status bit; the others are served
    pos = ctx.from_array(np.array([3, cap, 5, 6, 7], np.uint32))
    before = kc.download(plane * 2, plane * 2, np.float16).copy()
    ctx.attention_decode_batch(q, k, v, qn, kn, inv, kc, vc, out, sb, pos, status, S, heads, kvh, hd, hd, cap, window,
                               eps, scale, exact, **strides)
    ctx.fence()
    assert int(status.download(0, 4, np.uint32)[0]) & 1
    np.testing.assert_array_equal(kc.download(plane * 2, plane * 2, np.float16), before)
    with pytest.raises(cuda.CudaError):
        ctx.attention_decode_batch(q, k, v, qn, kn, inv, kc, vc, out, sb, pos, status, S + 1, heads, kvh, hd, hd, cap,
                                   window, eps, scale, exact, **strides)


@pytest.mark.parametrize("heads,kvh,window", [(16, 8, 0), (32, 8, 0), (8, 8, 0), (8, 2, 300)])
def test_tensor_core_decode_attention_against_the_oracle(ctx, oracle, heads, kvh, window):
    """The throughput form over long caches (several tiles per CTA, several splits per sequence, ragged
    positions, a sliding window) against oracle.attend_head on the same f16 cache: 2e-3 of the scale."""
    hd, cap, eps, S = 128, 1400, 1e-6, 6
    scale = 1.0 / np.sqrt(np.float32(hd))
    positions = np.array([1399, 0, 511, 512, 1023, 77], np.uint32)
    qn = ctx.floats(np.ones(hd, np.float32))
    kn = ctx.floats(np.ones(hd, np.float32))
    inv = np.zeros(hd // 2, np.float32)  # no rotation: the oracle attends the cache as stored
    plane = kvh * cap * hd
    kfill = (T.activations(1, 1, S * plane) * 0.3).astype(np.float16)
    vfill = T.activations(1, 2, S * plane).astype(np.float16)
    q = T.activations(2, 3, S * heads * hd).reshape(S, heads, hd)
    k = T.activations(2, 4, S * kvh * hd).reshape(S, kvh, hd)
    v = T.activations(2, 5, S * kvh * hd).reshape(S, kvh, hd)
    kc, vc = ctx.from_array(kfill), ctx.from_array(vfill)
    out = ctx.buffer(S * heads * hd * 4)
    sb = ctx.buffer(S * cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
    sb.zero()
    status = ctx.buffer(4, shared=True)
    status.zero()
    ctx.attention_decode_batch(ctx.floats(q), ctx.floats(k), ctx.floats(v), qn, kn, ctx.floats(inv), kc, vc, out, sb,
                               ctx.from_array(positions), status, S, heads, kvh, hd, hd, cap, window, eps, scale, False)
    ctx.fence()
    got = f32(out, S * heads * hd).reshape(S, heads, hd)
    assert int(status.download(0, 4, np.uint32)[0]) == 0

    def unit_norm(x):  # the kernel's RMS norm with weight 1
        return (x / np.sqrt(np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True) + eps)).astype(np.float32)

    group = heads // kvh
    for s in range(S):
        pos = int(positions[s])
        kcache = kfill[s * plane:(s + 1) * plane].reshape(kvh, cap, hd).copy()
        vcache = vfill[s * plane:(s + 1) * plane].reshape(kvh, cap, hd).copy()
        kcache[:, pos] = unit_norm(k[s]).astype(np.float16)
        vcache[:, pos] = v[s].astype(np.float16)
        np.testing.assert_array_equal(vc.download((s * plane + pos * hd) * 2, hd * 2, np.float16), vcache[0, pos])
        qs = unit_norm(q[s])
        for h in (0, heads // 2, heads - 1):
            seq = pos + 1
            start = seq - window if window and seq > window else 0
            want = oracle.attend_head(qs[h], kcache[h // group], vcache[h // group], start, seq, float(scale))
            err = np.max(np.abs(got[s, h] - want)) / max(1.0, float(np.max(np.abs(want))))
            assert err <= 2e-3, f"sequence {s} head {h}: {err:.3g}"


def test_row_gather_argmax_and_positions_per_sequence(ctx):
    rows, cols, S, stride, cap1 = 300, 96, 4, 12, 10
    raw = T.q8_0_matrix(3, 9, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    dense = T.q8_0_dequant(raw)
    logs = np.zeros((S, stride), np.uint32)
    logs[0, 2], logs[1, 0], logs[2, 9], logs[3, 5] = 7, 299, 300, 150  # id 300 is outside: zeros
    pos = np.array([2, 0, 9, 5], np.uint32)
    lb, pb = ctx.from_array(logs), ctx.from_array(pos)
    out = ctx.buffer(S * cols * 4)
    ctx.rows_indirect_seq(w, rows, cols, lb, stride, pb, S, 0, 2.0, out)
    got = f32(out, S * cols).reshape(S, cols)
    np.testing.assert_array_equal(got[0], dense[7] * 2.0)
    np.testing.assert_array_equal(got[1], dense[299] * 2.0)
    assert not got[2].any()
    np.testing.assert_array_equal(got[3], dense[150] * 2.0)
    ctx.rows_indirect_seq(w, rows, cols, lb, stride, pb, S, 5, 0.0, out)  # slots pos + 5: sequence 2's is outside its log
    got = f32(out, S * cols).reshape(S, cols)
    np.testing.assert_array_equal(got[0], dense[0])
    assert not got[2].any()

    n = 1000
    x = T.activations(5, 1, S * n).reshape(S, n)
    x[0, 123] = 60.0
    x[1, 17] = x[1, 900] = 50.0  # tie: the lower index
    x[2, :] = np.nan             # every logit NaN: the "none" id
    xb, partial = ctx.floats(x), ctx.buffer(S * 512)
    tok, mirror = ctx.from_array(np.zeros((S, stride), np.uint32)), ctx.buffer(S * stride * 4, shared=True)
    mirror.zero()
    pb = ctx.from_array(np.array([0, 3, 8, 9], np.uint32))  # 1 + 9 = slot 10 is outside a log of 10 slots
    ctx.argmax_rows_dev(xb, S, n, partial, tok, stride, 1, pb, cap1, mirror)
    got = tok.download(0, S * stride * 4, np.uint32).reshape(S, stride)
    assert got[0, 1] == 123 and got[1, 4] == 17 and got[2, 9] == 0xFFFFFFFF
    assert not got[3].any() and np.count_nonzero(got) == 3
    np.testing.assert_array_equal(mirror.download(0, S * stride * 4, np.uint32).reshape(S, stride), got)
    with pytest.raises(cuda.CudaError):
        ctx.argmax_rows_dev(xb, S, n, partial, tok, stride, 1, pb, stride + 1, mirror)

    c = ctx.from_array(np.array([5, 0, 98, 99, 7], np.uint32))
    ctx.u32_add_sat(c, 1, 3, 1, 99)
    np.testing.assert_array_equal(c.download(0, 20, np.uint32), [5, 1, 99, 99, 7])
    ctx.u32_add_sat(c, 0, 5, 0xFFFFFFF0, 99)  # no wrap-around
    np.testing.assert_array_equal(c.download(0, 20, np.uint32), [99] * 5)


@pytest.mark.parametrize("batch", [2, 5, 8, 13, 32])
def test_batched_fused_multiply_rows_are_the_one_token_call(ctx, batch):
    rows, cols = 200, 320
    raw = T.q8_0_matrix(4, 2, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    x = T.activations(6, 1, batch * cols).reshape(batch, cols)
    u = T.activations(6, 2, batch * cols).reshape(batch, cols)
    g = (1 + 0.1 * T.activations(6, 3, cols)).astype(np.float32)
    base = T.activations(6, 4, batch * rows).reshape(batch, rows)
    gb, one = ctx.floats(g), ctx.buffer(rows * 4)
    for pro, pbuf, rowwise in ((cuda.PRO_NONE, None, None), (cuda.PRO_RMSNORM, gb, None),
                               (cuda.PRO_SILU_MUL, ctx.floats(u), u), (cuda.PRO_GELU_MUL, ctx.floats(u), u)):
        for epi in (cuda.EPI_STORE, cuda.EPI_ADD):
            y = ctx.floats(base)
            ctx.q8_0_gemm_fused(w, ctx.floats(x), y, rows, cols, batch, pro, pbuf, 1e-6, epi)
            got = f32(y, batch * rows).reshape(batch, rows)
            for t in (0, batch // 2, batch - 1):
                one.upload(0, base[t])
                p1 = ctx.floats(rowwise[t]) if rowwise is not None else pbuf
                ctx.q8_0_gemv_fused(w, ctx.floats(x[t]), one, rows, cols, pro, p1, 1e-6, epi)
                np.testing.assert_array_equal(got[t], f32(one, rows), err_msg=f"prologue {pro} epilogue {epi} row {t}")
    with pytest.raises(cuda.CudaError):
        ctx.q8_0_gemm_fused(w, ctx.floats(x), ctx.floats(base), rows, cols, 33)


def test_a_row_view_multiplies_with_its_parents_column_split(ctx):
    """A part of a fused projection (a row view) must add a row's partial sums in the order the whole
    matrix does, whatever the part's own size would have suggested."""
    rows, cols = 24576, 1024  # 1536 row tiles: split 2 on this part; a quarter of it alone would take 8
    raw = T.q8_0_matrix(8, 1, rows, cols)
    w = ctx.q8_0_matrix(raw, rows, cols)
    x = ctx.floats(T.activations(8, 2, cols))
    y, part = ctx.buffer(rows * 4), ctx.buffer(6144 * 4)
    ctx.q8_0_gemv(w, x, y, rows, cols)
    view = ctx.q8_0_row_view(w, rows, cols, 12288, 6144)
    ctx.q8_0_gemv(view, x, part, 6144, cols)
    np.testing.assert_array_equal(f32(part, 6144), f32(y, 6144, off=12288))


# ---------------------------------------------------------------- engine

@pytest.fixture(scope="module", params=["qwen3", "gemma3", "small_qwen3"])
def artifact(request, tmp_path_factory):
    shape = {"qwen3": T.TINY_QWEN3, "gemma3": T.TINY_GEMMA3, "small_qwen3": T.SMALL_QWEN3}[request.param]
    path = tmp_path_factory.mktemp("gguf") / f"{request.param}.gguf"
    T.write_gguf(path, shape, seed=3, norm_jitter=0.1)
    return path, shape


def prompts_for(shape, n, base_len=5):
    return [T.token_ids(20 + i, base_len + 3 * i, shape.vocab) for i in range(n)]


@pytest.mark.parametrize("S,exact", [(3, True), (12, True), (40, True), (3, False), (8, False)])
def test_batched_steps_equal_single_sequence_steps_bit_for_bit(ctx, artifact, S, exact):
    path, shape = artifact
    prompts = prompts_for(shape, S, base_len=2)
    feed = [T.token_ids(50 + i, 6, shape.vocab) for i in range(S)]
    cap = 160
    one = E.Engine(path, context=cap, exact=exact, prefill_batch=16)
    want = []
    for s in range(S):
        one.reset()
        one.prefill(prompts[s], want_token=True)
        rows = [one.logits()] + [one.step(int(t)) for t in feed[s]]
        want.append(np.stack(rows))
    one.close()
    eng = E.Engine(path, context=cap, exact=exact, prefill_batch=16, sequences=S)
    i = eng.info
    assert i.allocated_bytes == i.plan_weights + i.plan_state + i.plan_scratch
    assert i.plan_state == S * shape.layers * 2 * shape.kv_heads * cap * shape.head_dim * 2
    # outside `exact` mode head size 128 decodes batches with the tensor-core attention: tolerance there
    identical = exact or shape.head_dim != 128
    for rounds in range(2):  # reset() brings every sequence back
        eng.reset()
        for s in range(S):
            eng.prefill_seq(s, prompts[s], want_token=True)
            np.testing.assert_array_equal(eng.logits(), want[s][0])
            assert eng.prefill_token_of(s) == int(np.argmax(want[s][0]))
        for j in range(6):
            got = eng.step_batch([int(feed[s][j]) for s in range(S)])
            for s in range(S):
                if identical:
                    np.testing.assert_array_equal(got[s], want[s][j + 1], err_msg=f"sequence {s} step {j}")
                else:
                    scale = max(1.0, float(np.max(np.abs(want[s][j + 1]))))
                    assert np.max(np.abs(got[s] - want[s][j + 1])) <= 2e-2 * scale, f"sequence {s} step {j}"
    eng.close()


@pytest.mark.parametrize("S", [12, 33])
def test_larger_batches_on_the_tensor_core_path_match_the_oracle(ctx, oracle, artifact, S):
    """More than 8 sequences outside `exact` mode go through the batched tensor-core projections
    (f16-operand profile): the model-parity policy of crates/tuckcore/src/executor.rs:2143-2321."""
    path, shape = artifact
    prompts = prompts_for(shape, S, base_len=3)
    feed = [T.token_ids(70 + i, 4, shape.vocab) for i in range(S)]
    eng = E.Engine(path, context=160, prefill_batch=16, sequences=S)
    for s in range(S):
        eng.prefill_seq(s, prompts[s], want_token=False)
    rows = [eng.step_batch([int(feed[s][j]) for s in range(S)]) for j in range(4)]
    eng.close()
    cpu = oracle.Model(path)
    for s in (0, S // 2, S - 1):
        cpu.reset(160)
        cpu.forward(prompts[s], want_logits=False)
        for j in range(4):
            ref = cpu.forward([int(feed[s][j])])
            scale = max(1.0, float(np.max(np.abs(ref))))
            assert np.max(np.abs(rows[j][s] - ref)) <= 2e-2 * scale, f"sequence {s} step {j}"
            top2 = np.partition(ref, -2)[-2:]
            if top2[1] - top2[0] > 1e-3 * scale:
                assert int(np.argmax(rows[j][s])) == oracle.argmax(ref)


@pytest.mark.parametrize("exact", [True, False])
def test_generate_batch_equals_one_request_at_a_time(ctx, artifact, exact):
    path, shape = artifact
    S, cap, max_new = 6, 48, 20
    prompts = prompts_for(shape, 5, base_len=4)          # 5 requests on 6 sequences, ragged lengths
    prompts[3] = T.token_ids(99, cap - 6, shape.vocab)   # this one reaches the capacity after 7 tokens
    one = E.Engine(path, context=cap, exact=exact, prefill_batch=16)
    want = [one.generate(p, max_new)[0] for p in prompts]
    one.close()
    assert len(want[3]) == 7 and len(want[0]) == max_new
    eng = E.Engine(path, context=cap, exact=exact, prefill_batch=16, sequences=S)
    for _ in range(2):
        got, stats = eng.generate_batch(prompts, max_new)
        assert stats.generated == sum(len(w) for w in want) and stats.prompt_tokens == sum(len(p) for p in prompts)
        for r in range(len(prompts)):
            np.testing.assert_array_equal(got[r], want[r], err_msg=f"request {r}")
    with pytest.raises(E.EngineError) as e:
        eng.generate_batch(prompts + prompts, max_new)
    assert e.value.code == "INVALID_REQUEST"
    with pytest.raises(E.EngineError) as e:
        eng.step_batch([0] * S)  # the state is spent after a generation: reset first
    assert e.value.code == "CONTEXT_EXCEEDS_BUDGET"
    eng.reset()
    with pytest.raises(E.EngineError) as e:
        eng.step_batch([0] * (S - 1) + [shape.vocab])
    assert e.value.code == "INVALID_REQUEST"
    eng.close()
    with pytest.raises(E.EngineError):
        E.Engine(path, context=cap, sequences=100000)
    single = E.Engine(path, context=cap)
    with pytest.raises(E.EngineError) as e:
        single.step_batch([0])
    assert e.value.code == "INVALID_REQUEST"
    single.close()
