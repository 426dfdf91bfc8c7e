"""Support operators and the context contract through the C ABI (the
reference's crates/metal/src/tests.rs:257-306 casts, :409-574 ownership /
ledger / grouping, :1250-1355 argmax, and the attention kernels against the
scalar executor's arithmetic)."""
import numpy as np
import pytest

from conftest import rel_err
from tuckmill_b200 import cuda, testing as T

pytestmark = pytest.mark.gpu


def f32(buf, n):
    return buf.download(0, n * 4, np.float32)


def test_elementwise(ctx, oracle):
    n = 1000
    x, a = T.activations(0, 1, n), T.activations(0, 2, n)
    xb, ab, yb = ctx.floats(x), ctx.floats(a), ctx.buffer(n * 4)
    ctx.f32_scale(xb, yb, 3.5, n)
    np.testing.assert_array_equal(f32(yb, n), x * np.float32(3.5))
    ctx.f32_axpy(ab, yb, 1.0, n)
    np.testing.assert_array_equal(f32(yb, n), x * np.float32(3.5) + a)
    dst = ctx.floats(np.zeros(n + 10, np.float32))
    ctx.copy_f32(xb, 5, dst, 7, 100)
    got = f32(dst, n + 10)
    np.testing.assert_array_equal(got[7:107], x[5:105])
    assert np.all(got[:7] == 0) and np.all(got[107:] == 0)
    ctx.silu_mul(xb, ab, yb, n)
    ref = np.array([oracle.silu(v) for v in x], np.float32) * a
    assert rel_err(f32(yb, n), ref) <= 1e-6
    ctx.gelu_tanh_mul(xb, ab, yb, n)
    ref = np.array([oracle.gelu_tanh(v) for v in x], np.float32) * a
    assert rel_err(f32(yb, n), ref) <= 1e-6
    with pytest.raises(cuda.CudaError):
        ctx.f32_scale(xb, yb, 1.0, n + 1)
    with pytest.raises(cuda.CudaError):
        ctx.copy_f32(xb, n - 5, dst, 0, 10)


def test_casts_match_reference_tables(ctx, oracle):
    """f16 encode/decode lists of tensor.rs:358-370 and tests.rs:257-306."""
    vals = np.array([0.0, 1.0, -2.0, 65504.0, 100000.0, 5.96e-8, 1 + 2.0**-11, 1 + 2.0**-11 + 2.0**-13,
                     65520.0, np.inf, -np.inf, 2.0**-25, 6e-5, -0.0, 448.0], np.float32)
    xb, hb = ctx.floats(vals), ctx.buffer(vals.size * 2)
    ctx.cast_f32_f16(xb, hb, vals.size)
    bits = hb.download(0, vals.size * 2, np.uint16)
    want = np.array([oracle.f32_to_f16_bits(v) for v in vals], np.uint16)
    np.testing.assert_array_equal(bits, want)
    assert list(bits[:8]) == [0x0000, 0x3C00, 0xC000, 0x7BFF, 0x7C00, 0x0001, 0x3C00, 0x3C01]
    back = ctx.buffer(vals.size * 4)
    ctx.cast_f16_f32(hb, back, vals.size)
    np.testing.assert_array_equal(f32(back, vals.size), np.array([oracle.f16_to_f32(int(b)) for b in bits], np.float32))
    rnd = T.activations(3, 9, 4096) * np.float32(100.0)
    rb, hb2 = ctx.floats(rnd), ctx.buffer(rnd.size * 2)
    ctx.cast_f32_f16(rb, hb2, rnd.size)
    np.testing.assert_array_equal(hb2.download(0, rnd.size * 2, np.uint16),
                                  np.array([oracle.f32_to_f16_bits(v) for v in rnd], np.uint16))


def test_rmsnorm(ctx, oracle):
    xb, wb, yb = ctx.floats([3.0, 4.0]), ctx.floats([1.0, 1.0]), ctx.buffer(8)
    ctx.rmsnorm(xb, wb, yb, 1, 2, 0.0)
    np.testing.assert_allclose(f32(yb, 2), np.array([3.0, 4.0]) / np.sqrt(12.5), rtol=1e-6)
    rows, cols = 5, 1152
    x = T.activations(0, 3, rows * cols).reshape(rows, cols)
    w = (1 + 0.1 * T.activations(0, 4, cols)).astype(np.float32)
    xb, wb = ctx.floats(x), ctx.floats(w)
    ctx.rmsnorm(xb, wb, xb, rows, cols, 1e-6)  # in place
    ref = np.stack([oracle.rmsnorm(x[r], w, 1e-6) for r in range(rows)])
    assert rel_err(f32(xb, rows * cols).reshape(rows, cols), ref) <= 1e-5


def test_argmax_rule(ctx, oracle):
    nan, inf = np.nan, np.inf
    cases = [[3.0, 3.0], [nan, 1.0], [nan, inf], [nan, nan, nan], [-0.0, 0.0], [1.0, 5.0, 5.0, 2.0],
             [-inf, -inf], [nan, -inf]]
    part, out = ctx.buffer(512), ctx.buffer(16, shared=True)
    for c in cases:
        xb = ctx.floats(c)
        ctx.argmax_f32(xb, len(c), part, out, 1)
        got = int(out.download(4, 4, np.uint32)[0])
        assert got == oracle.argmax(np.array(c, np.float32)), c
    assert oracle.argmax(np.array([nan, nan], np.float32)) == cuda.ARGMAX_NONE
    big = T.activations(1, 5, 248320)
    big[[777, 200000, 248319]] = big.max() + 1.0  # planted ties: lowest index wins
    xb = ctx.floats(big)
    ctx.argmax_f32(xb, big.size, part, out, 0)
    assert int(out.download(0, 4, np.uint32)[0]) == 777 == oracle.argmax(big)


def test_rope_and_kv_store(ctx, oracle):
    n, nq, nkv, hd, cap, pos0 = 3, 4, 2, 64, 16, 5
    q = T.activations(0, 6, n * nq * hd).reshape(n, nq, hd)
    k = T.activations(0, 7, n * nkv * hd).reshape(n, nkv, hd)
    v = T.activations(0, 8, n * nkv * hd).reshape(n, nkv, hd)
    inv = oracle.rope_inv_freq(hd, 1e6)
    qb, kb, vb, ib = ctx.floats(q), ctx.floats(k), ctx.floats(v), ctx.floats(inv)
    ctx.qwen35_rope_partial_chunk(qb, kb, ib, pos0, nq, nkv, hd, hd, n)
    qr = np.stack([[oracle.rope_apply(q[t, h], pos0 + t, inv) for h in range(nq)] for t in range(n)])
    kr = np.stack([[oracle.rope_apply(k[t, h], pos0 + t, inv) for h in range(nkv)] for t in range(n)])
    assert rel_err(f32(qb, q.size).reshape(q.shape), qr) <= 2e-6
    assert rel_err(f32(kb, k.size).reshape(k.shape), kr) <= 2e-6
    # reference rope KAT (forward.rs:1026-1041)
    xb, fb, kd = ctx.floats([1.0, 0.0, 0.5, 1.5]), ctx.floats([1.0, 0.5]), ctx.floats(np.zeros(4))
    ctx.qwen35_rope_partial(xb, kd, fb, 3, 1, 1, 4, 4)
    s3, c3, s15, c15 = np.sin(np.float32(3)), np.cos(np.float32(3)), np.sin(np.float32(1.5)), np.cos(np.float32(1.5))
    np.testing.assert_allclose(f32(xb, 4), [c3 - 0.5 * s3, -1.5 * s15, s3 + 0.5 * c3, 1.5 * c15], atol=1e-6)
    plane = nkv * cap * hd
    kc, vc = ctx.buffer(plane * 2), ctx.buffer(plane * 2)
    kc.zero(); vc.zero()
    ctx.qwen35_kv_store_chunk(kb, vb, kc, vc, pos0, cap, hd, nkv, n)
    kcache = kc.download(0, plane * 2, np.float16).reshape(nkv, cap, hd)
    vcache = vc.download(0, plane * 2, np.float16).reshape(nkv, cap, hd)
    kgpu = f32(kb, k.size).reshape(k.shape)
    for t in range(n):
        np.testing.assert_array_equal(kcache[:, pos0 + t], kgpu[t].astype(np.float16))
        np.testing.assert_array_equal(vcache[:, pos0 + t], v[t].astype(np.float16))
    assert np.all(kcache[:, :pos0] == 0) and np.all(kcache[:, pos0 + n:] == 0)
    with pytest.raises(cuda.CudaError):
        ctx.qwen35_kv_store_chunk(kb, vb, kc, vc, cap - 1, cap, hd, nkv, n)


@pytest.mark.parametrize("heads,kvh,hd,window", [(4, 2, 32, 0), (16, 8, 128, 0), (4, 1, 256, 8), (4, 1, 256, 0), (6, 2, 96, 5), (12, 2, 64, 0)])
def test_attention_chunk_matches_scalar_executor(ctx, oracle, heads, kvh, hd, window):
    cap, pos0, n = 90, 57, 6
    group = heads // kvh
    kf = T.activations(0, 10, kvh * cap * hd).astype(np.float16).reshape(kvh, cap, hd)
    vf = T.activations(0, 11, kvh * cap * hd).astype(np.float16).reshape(kvh, cap, hd)
    q = T.activations(0, 12, n * heads * hd).reshape(n, heads, hd)
    kc, vc, qb = ctx.from_array(kf), ctx.from_array(vf), ctx.floats(q)
    ob, sb = ctx.buffer(q.size * 4), ctx.buffer(n * heads * cap * 4)
    scale = 1.0 / np.sqrt(np.float32(hd))
    ctx.qwen35_attention_chunk(qb, kc, vc, ob, sb, heads, pos0, cap, hd, group, scale, n, window)
    got = f32(ob, q.size).reshape(n, heads, hd)
    k32, v32 = kf.astype(np.float32), vf.astype(np.float32)
    for t in range(n):
        seq = pos0 + t + 1
        start = seq - window if (window and seq > window) else 0
        for h in range(heads):
            ref = oracle.attend_head(q[t, h], k32[h // group], v32[h // group], start, seq, scale)
            assert rel_err(got[t, h], ref) <= 1e-5
    if window == 0:  # the one-row entry point is the chunk kernel at n = 1
        o1 = ctx.buffer(heads * hd * 4)
        ctx.qwen35_attention_f16(qb, kc, vc, o1, sb, heads, pos0, cap, hd, group, scale)
        np.testing.assert_array_equal(f32(o1, heads * hd).reshape(heads, hd), got[0])


@pytest.mark.parametrize("heads,kvh,hd,window,cap,steps", [(16, 8, 128, 0, 24, 10), (4, 1, 256, 6, 24, 10),
                                                            (4, 2, 32, 0, 100, 70), (12, 2, 64, 40, 100, 90), (16, 8, 128, 0, 200, 150),
                                                            (4, 1, 256, 70, 200, 150)])
def test_decode_attention_core_equals_operator_sequence(ctx, oracle, heads, kvh, hd, window, cap, steps):
    """The fused device-position core is bit-identical to rmsnorm x2 + rope +
    kv_store + attention_chunk(n=1) (the prefill == decode invariant of
    crates/tuckcore/src/engine/metal.rs:3682-3774)."""
    eps = 1e-6
    group, scale = heads // kvh, 1.0 / np.sqrt(np.float32(hd))
    qn = (1 + 0.1 * T.activations(0, 20, hd)).astype(np.float32)
    kn = (1 + 0.1 * T.activations(0, 21, hd)).astype(np.float32)
    inv = oracle.rope_inv_freq(hd, 1e4)
    qnb, knb, ib = ctx.floats(qn), ctx.floats(kn), ctx.floats(inv)
    plane = kvh * cap * hd * 2
    caches = [[ctx.buffer(plane), ctx.buffer(plane)] for _ in range(3)]
    for pair in caches:
        for c in pair:
            c.zero()
    pos_buf, status = ctx.from_array(np.zeros(2, np.uint32)), ctx.buffer(4, shared=True)
    status.zero()
    sb = ctx.buffer(cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
    sb.zero()
    sb2 = ctx.buffer(cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
    sb2.zero()
    for pos in range(steps):
        q = T.activations(pos, 30, heads * hd)
        k = T.activations(pos, 31, kvh * hd)
        v = T.activations(pos, 32, kvh * hd)
        # (a) operator sequence
        qa, ka, va, oa = ctx.floats(q), ctx.floats(k), ctx.floats(v), ctx.buffer(heads * hd * 4)
        ctx.rmsnorm(qa, qnb, qa, heads, hd, eps)
        ctx.rmsnorm(ka, knb, ka, kvh, hd, eps)
        ctx.qwen35_rope_partial(qa, ka, ib, pos, heads, kvh, hd, hd)
        ctx.qwen35_kv_store_chunk(ka, va, caches[0][0], caches[0][1], pos, cap, hd, kvh, 1)
        ctx.qwen35_attention_chunk(qa, caches[0][0], caches[0][1], oa, sb, heads, pos, cap, hd, group, scale, 1, window)
        # (b) fused core with the position on the device
        qf, kf, vf, of = ctx.floats(q), ctx.floats(k), ctx.floats(v), ctx.buffer(heads * hd * 4)
        ctx.attention_decode_dev(qf, kf, vf, qnb, knb, ib, caches[1][0], caches[1][1], of, sb, pos_buf, 1,
                                 status, heads, kvh, hd, hd, cap, window, eps, scale)
        ctx.u32_add(pos_buf, 1, 1)
        np.testing.assert_array_equal(f32(of, heads * hd), f32(oa, heads * hd))
        # (c) the latency-optimised kernel: same mathematics, tolerance-qualified
        og = ctx.buffer(heads * hd * 4)
        ctx.attention_decode_dev(ctx.floats(q), ctx.floats(k), ctx.floats(v), qnb, knb, ib, caches[2][0], caches[2][1],
                                 og, sb2, pos_buf, 0, status, heads, kvh, hd, hd, cap, window, eps, scale, exact=False)
        ctx.u32_add(pos_buf, 0, 1)
        assert rel_err(f32(og, heads * hd), f32(oa, heads * hd)) <= 1e-4
    # its stored K rows agree to f16 rounding (different norm / sincos summation order)
    ka = caches[0][0].download(0, plane, np.float16).astype(np.float32)
    kb = caches[2][0].download(0, plane, np.float16).astype(np.float32)
    assert rel_err(kb, ka) <= 2e-3
    np.testing.assert_array_equal(caches[0][1].download(0, plane), caches[2][1].download(0, plane))
    for i in range(2):
        np.testing.assert_array_equal(caches[0][i].download(0, plane), caches[1][i].download(0, plane))
    assert int(status.download(0, 4, np.uint32)[0]) == 0
    # a position at capacity writes nothing and raises the status bit
    pos_buf.upload(0, np.array([0, cap], np.uint32))
    before = caches[1][0].download(0, plane).copy()
    ctx.attention_decode_dev(qf, kf, vf, qnb, knb, ib, caches[1][0], caches[1][1], of, sb, pos_buf, 1,
                             status, heads, kvh, hd, hd, cap, window, eps, scale)
    ctx.fence()
    assert int(status.download(0, 4, np.uint32)[0]) & 1
    np.testing.assert_array_equal(caches[1][0].download(0, plane), before)


@pytest.mark.parametrize("exact", [True, False])
def test_consecutive_decode_calls_inside_one_group(ctx, exact):
    """attention(pos) -> advance -> attention(pos + 1) -> ... on ONE cache inside ONE dispatch group:
    kernels of a group start while their predecessors still run, so a call must not pick up the row
    its predecessor-but-one is still storing.  Compared with the same calls issued one by one."""
    heads, kvh, hd, cap, eps, filled, n = 16, 8, 128, 200, 1e-6, 60, 6
    scale = 1.0 / np.sqrt(np.float32(hd))
    qnb = ctx.floats((1 + 0.1 * T.activations(0, 20, hd)).astype(np.float32))
    knb = ctx.floats((1 + 0.1 * T.activations(0, 21, hd)).astype(np.float32))
    ib = ctx.floats((1e4 ** (-np.arange(hd // 2, dtype=np.float64) * 2 / hd)).astype(np.float32))
    kfill = T.activations(1, 1, kvh * cap * hd).astype(np.float16)
    vfill = T.activations(1, 2, kvh * cap * hd).astype(np.float16)
    qs = [ctx.floats(T.activations(40 + i, 30, heads * hd)) for i in range(n)]
    ks = [ctx.floats(T.activations(40 + i, 31, kvh * hd)) for i in range(n)]
    vs = [ctx.floats(T.activations(40 + i, 32, kvh * hd)) for i in range(n)]
    status = ctx.buffer(4, shared=True)
    status.zero()
    results = []
    for grouped in (False, True):
        kc, vc = ctx.from_array(kfill), ctx.from_array(vfill)
        pos_buf = ctx.from_array(np.array([filled], np.uint32))
        sb = ctx.buffer(cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
        sb.zero()
        outs = [ctx.buffer(heads * hd * 4) for _ in range(n)]
        if grouped:
            ctx.begin_group()
        for i in range(n):
            ctx.attention_decode_dev(qs[i], ks[i], vs[i], qnb, knb, ib, kc, vc, outs[i], sb, pos_buf, 0, status,
                                     heads, kvh, hd, hd, cap, 0, eps, scale, exact=exact)
            ctx.u32_add(pos_buf, 0, 1)
            if not grouped:
                ctx.fence()
        if grouped:
            ctx.end_group()
        ctx.fence()
        results.append([f32(o, heads * hd) for o in outs])
    for i in range(n):
        np.testing.assert_array_equal(results[1][i], results[0][i], err_msg=f"call {i} of the group")
    assert int(status.download(0, 4, np.uint32)[0]) == 0


def test_buffers_ledger_and_ownership(ctx):
    base = ctx.allocated_bytes()
    a, b = ctx.buffer(1000), ctx.buffer(24, shared=True)
    assert ctx.allocated_bytes() == base + 1024 and len(a) == 1000 and ctx.in_flight_bytes() == 0
    v = a.view(256, 512)
    assert ctx.allocated_bytes() == base + 1024 and len(v) == 512
    a.upload(256, np.arange(128, dtype=np.float32))
    np.testing.assert_array_equal(v.download(0, 512, np.float32), np.arange(128, dtype=np.float32))
    with pytest.raises(cuda.CudaError):
        a.view(100, 10)  # not 16-byte aligned
    with pytest.raises(cuda.CudaError):
        a.upload(990, np.zeros(20, np.uint8))
    with pytest.raises(cuda.CudaError):
        ctx.buffer(0)
    a.zero(256, 16)
    assert np.all(v.download(0, 16) == 0)
    v.free(); a.free(); b.free()
    assert ctx.allocated_bytes() == base


def test_grouped_equals_individual_and_abort_writes_nothing(ctx):
    """crates/metal/src/tests.rs:529-574."""
    n = 4096
    x = T.activations(0, 40, n)
    xb, y1, y2 = ctx.floats(x), ctx.floats(np.zeros(n)), ctx.floats(np.zeros(n))

    def chain(y):
        ctx.f32_scale(xb, y, 2.0, n)
        ctx.f32_axpy(xb, y, 0.5, n)
        ctx.silu_mul(y, xb, y, n)

    chain(y1)
    c0, l0 = ctx.committed_dispatches(), ctx.kernel_launches()
    ctx.grouped(lambda: chain(y2))
    assert ctx.committed_dispatches() == c0 + 1 and ctx.kernel_launches() == l0 + 3
    ctx.fence()
    assert ctx.completed_dispatches() == ctx.committed_dispatches()
    np.testing.assert_array_equal(f32(y1, n), f32(y2, n))
    y3 = ctx.floats(np.full(n, 9.0, np.float32))
    ctx.begin_group()
    chain(y3)
    with pytest.raises(cuda.CudaError):
        ctx.fence()  # fence with an open group is an error
    with pytest.raises(cuda.CudaError):
        y3.upload(0, np.zeros(4, np.float32))
    ctx.abort_group()
    ctx.fence()
    assert np.all(f32(y3, n) == 9.0)
    with pytest.raises(cuda.CudaError):
        ctx.end_group()
    # retained graph: replays with a device-held counter
    cnt = ctx.from_array(np.zeros(1, np.uint32))
    ctx.begin_group()
    ctx.u32_add(cnt, 0, 3)
    g = ctx.end_group_retain()
    assert int(cnt.download(0, 4, np.uint32)[0]) == 0
    for _ in range(5):
        g.launch()
    assert int(cnt.download(0, 4, np.uint32)[0]) == 15
    g.free()
    assert ctx.gpu_nanos_total() > 0


def test_download_after_reads_a_pipelined_result(ctx):
    """tm_metal.h's download_after contract: wait only for the target dispatch."""
    part, out = ctx.buffer(512), ctx.buffer(8, shared=True)
    out.zero()
    xs = [ctx.floats(np.roll(np.arange(1000, dtype=np.float32), s)) for s in (0, 1)]
    ctx.argmax_f32(xs[0], 1000, part, out, 0)
    target = ctx.committed_dispatches()
    ctx.argmax_f32(xs[1], 1000, part, out, 1)
    assert int(out.download_after(0, 4, target, np.uint32)[0]) == 999
    ctx.fence()
    assert int(out.download(4, 4, np.uint32)[0]) == 0
    with pytest.raises(cuda.CudaError):
        out.download_after(0, 4, ctx.committed_dispatches() + 5)
    priv = ctx.buffer(8)
    with pytest.raises(cuda.CudaError):
        priv.download_after(0, 4, 0)


def test_profile_table(ctx):
    ctx.set_profiling(True)
    x = ctx.floats(np.ones(256))
    for _ in range(3):
        ctx.f32_scale(x, x, 1.0, 256)
    ctx.fence()
    rows = dict((n, (ns, c)) for n, ns, c in ctx.profile_snapshot())
    assert rows["f32_scale"][1] == 3
    ctx.set_profiling(False)
    assert ctx.profile_snapshot() == []


@pytest.mark.parametrize("heads,kvh,hd,window,cap,pos0,n", [
    (16, 8, 128, 0, 600, 0, 512),      # the benchmark's prefill geometry
    (16, 8, 128, 0, 700, 130, 200),    # a later chunk: earlier keys plus the causal part
    (4, 1, 256, 512, 900, 300, 333),   # Gemma-style: wide heads (two value halves), sliding window, ragged n
    (4, 1, 256, 40, 300, 0, 130),      # window shorter than a key tile
    (4, 2, 32, 0, 100, 57, 6),         # the small test models' head size
    (12, 2, 64, 17, 150, 3, 70),
])
def test_tensor_core_chunk_attention_within_tolerance(ctx, oracle, heads, kvh, hd, window, cap, pos0, n):
    """The mma.sync prefill form against the blockwise kernel (itself pinned to
    the scalar executor above) and, on sampled rows, against the oracle: binary16
    Q / softmax weights cost about 1e-3 of the output scale."""
    group = heads // kvh
    kf = T.activations(0, 10, kvh * cap * hd).astype(np.float16).reshape(kvh, cap, hd)
    vf = T.activations(0, 11, kvh * cap * hd).astype(np.float16).reshape(kvh, cap, hd)
    q = T.activations(0, 12, n * heads * hd).reshape(n, heads, hd)
    kc, vc, qb = ctx.from_array(kf), ctx.from_array(vf), ctx.floats(q)
    ob, o2, sb = ctx.buffer(q.size * 4), ctx.buffer(q.size * 4), ctx.buffer(16)
    scale = 1.0 / np.sqrt(np.float32(hd))
    ctx.qwen35_attention_chunk(qb, kc, vc, ob, sb, heads, pos0, cap, hd, group, scale, n, window)
    ctx.attention_chunk_mma(qb, kc, vc, o2, heads, pos0, cap, hd, group, scale, n, window)
    ref = f32(ob, q.size).reshape(n, heads, hd)
    got = f32(o2, q.size).reshape(n, heads, hd)
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - ref)) <= 2e-3 * max(1.0, float(np.max(np.abs(ref))))
    k32, v32 = kf.astype(np.float32), vf.astype(np.float32)
    for t in sorted({0, n // 2, n - 1}):
        seq = pos0 + t + 1
        start = seq - window if (window and seq > window) else 0
        for h in (0, heads - 1):
            cpu = oracle.attend_head(q[t, h], k32[h // group], v32[h // group], start, seq, scale)
            assert rel_err(got[t, h], cpu) <= 3e-3


@pytest.mark.parametrize("rows,cols", [(1, 1152), (7, 1024), (300, 640), (3, 4097)])
def test_rmsnorm_add_equals_rmsnorm_then_axpy(ctx, rows, cols):
    """The fused output norm + residual add is the two launches it replaces, bit for bit."""
    p = T.activations(5, 1, rows * cols)
    x = T.activations(5, 2, rows * cols)
    w = (1 + 0.1 * T.activations(5, 3, cols)).astype(np.float32)
    wb = ctx.floats(w)
    pa, xa = ctx.floats(p), ctx.floats(x)
    ctx.rmsnorm(pa, wb, pa, rows, cols, 1e-6)
    ctx.f32_axpy(pa, xa, 1.0, rows * cols)
    pb, xb = ctx.floats(p), ctx.floats(x)
    ctx.rmsnorm_add(pb, wb, xb, rows, cols, 1e-6)
    np.testing.assert_array_equal(f32(xb, rows * cols), f32(xa, rows * cols))
    np.testing.assert_array_equal(f32(pb, rows * cols), p)  # the input is left alone


@pytest.mark.parametrize("world,n_rows,cols", [(2, 1, 1024), (4, 1, 4096), (8, 3, 1152), (3, 40, 96), (1, 2, 64)])
def test_rank_reduction_adds_in_rank_order(ctx, world, n_rows, cols):
    """tm_cuda_reduce_ranks_add_f32 (the reduction of a column-split projection): x += slot 0 + slot 1 + ...
    in that order, bit for bit; with a norm weight the sum goes through the RMS norm exactly as
    tm_cuda_rmsnorm_add_f32 would take it."""
    slots = (T.activations(3, 1, world * n_rows * cols) * np.float32(3.0)).reshape(world, n_rows, cols)
    x0 = T.activations(3, 2, n_rows * cols).reshape(n_rows, cols)
    acc = slots[0].copy()
    for r in range(1, world):
        acc = (acc + slots[r]).astype(np.float32)
    xb, sb = ctx.floats(x0), ctx.floats(slots)
    ctx.reduce_ranks_add(sb, xb, None, world, n_rows, cols)
    np.testing.assert_array_equal(f32(xb, n_rows * cols).reshape(n_rows, cols), (x0 + acc).astype(np.float32))
    np.testing.assert_array_equal(f32(sb, world * n_rows * cols).reshape(world, n_rows, cols), slots)  # untouched
    w = (1 + 0.1 * T.activations(3, 3, cols)).astype(np.float32)
    wb, want = ctx.floats(w), ctx.floats(x0)
    ctx.rmsnorm_add(ctx.floats(acc), wb, want, n_rows, cols, 1e-6)
    xb2, sb2 = ctx.floats(x0), ctx.floats(slots)
    ctx.reduce_ranks_add(sb2, xb2, wb, world, n_rows, cols, 1e-6)
    np.testing.assert_array_equal(f32(xb2, n_rows * cols), f32(want, n_rows * cols))
    with pytest.raises(cuda.CudaError):
        ctx.reduce_ranks_add(sb, xb, None, world + 1, n_rows, cols)


def test_l2_prefetch_is_only_a_hint(ctx):
    """tm_cuda_prefetch_l2 forks a side stream and rejoins it: alone, and inside a recorded group
    between dependent operators, nothing about the results changes."""
    n = 1 << 16
    x = T.activations(9, 1, n)
    big = ctx.floats(T.activations(9, 2, 1 << 20))
    xb, y1, y2 = ctx.floats(x), ctx.floats(np.zeros(n)), ctx.floats(np.zeros(n))
    ctx.prefetch_l2([big, xb])
    ctx.f32_scale(xb, y1, 2.0, n)
    ctx.f32_axpy(xb, y1, 0.5, n)
    ctx.begin_group()
    ctx.prefetch_l2([big])
    ctx.f32_scale(xb, y2, 2.0, n)
    ctx.prefetch_l2([big, xb])
    ctx.f32_axpy(xb, y2, 0.5, n)
    g = ctx.end_group_retain()
    for _ in range(3):
        y2.zero()
        g.launch()
    ctx.fence()
    g.free()
    np.testing.assert_array_equal(f32(y2, n), f32(y1, n))
    with pytest.raises(cuda.CudaError):
        ctx.prefetch_l2([])
