"""The persistent decode program through the C ABI and through the engine.

A program records the operators of a decode step and runs them as one kernel
(include/tm_cuda.h, tm_cuda_begin_program).  Recorded operators must compute what
the same calls compute when dispatched one by one: the GEMV within the
reference's 1e-4 rule (crates/metal/src/tests.rs:367-381; the partial sums are
added in another order), the attention core to rounding of the split merge
(same arithmetic, same split), the greedy choice exactly.  The engine's decode loop on the program must
give the oracle's tokens, like the graph of kernels it replaces
(crates/tuckcore/src/executor.rs:2204-2230).  The bounded waits are made to run
out from the host (consumers told to expect sequence numbers that no producer writes,
with a short polling limit) and must end in a status word, not a hang."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err
from tuckmill_b200 import cuda, engine as E, testing as T

pytestmark = pytest.mark.gpu
TOL = 1e-4


def f32(buf, n):
    return buf.download(0, n * 4, np.float32)


@pytest.mark.parametrize("hidden,ffn,vocab", [(1024, 3072, 5000), (1152, 6912, 3001), (4096, 12288, 1000)])
def test_recorded_gemv_chain_equals_dispatched_operators(ctx, oracle, hidden, ffn, vocab):
    """norm-fused gate|up, activation-fused down with residual add, norm-fused head and the greedy
    choice: as a program and as single dispatches, from the same inputs."""
    eps = 1e-6
    raw_gu = T.q8_0_matrix(5, 1, 2 * ffn, hidden)
    raw_dn = T.q8_0_matrix(5, 2, hidden, ffn)
    raw_hd = T.q8_0_matrix(5, 3, vocab, hidden)
    w_gu, w_dn, w_hd = (ctx.q8_0_matrix(r, *r.shape[:1], c) for r, c in ((raw_gu, hidden), (raw_dn, ffn), (raw_hd, hidden)))
    norm = ctx.floats((1 + 0.1 * T.activations(5, 4, hidden)).astype(np.float32))
    x0 = T.activations(5, 5, hidden)
    results = []
    for recorded in (False, True):
        x = ctx.floats(x0)
        gu, logits = ctx.buffer(2 * ffn * 4), ctx.buffer(vocab * 4)
        g_view, u_view = gu.view(0, ffn * 4), gu.view(ffn * 4, ffn * 4)
        part, out = ctx.buffer(512), ctx.from_array(np.zeros(4, np.uint32))
        if recorded:
            ctx.begin_program(16)
        ctx.q8_0_gemv_fused(w_gu, x, gu, 2 * ffn, hidden, cuda.PRO_RMSNORM, norm, eps, cuda.EPI_STORE)
        ctx.q8_0_gemv_fused(w_dn, g_view, x, hidden, ffn, cuda.PRO_SILU_MUL, u_view, 0.0, cuda.EPI_ADD)
        ctx.q8_0_gemv_fused(w_hd, x, logits, vocab, hidden, cuda.PRO_RMSNORM, norm, eps, cuda.EPI_STORE)
        ctx.argmax_f32(logits, vocab, part, out, 2)
        if recorded:
            prog = ctx.end_program()
            launches = ctx.kernel_launches()
            prog.launch()
            ctx.fence()
            assert ctx.kernel_launches() == launches + 1
            assert prog.status() == 0
            prog.free()
        ctx.fence()
        results.append((f32(gu, 2 * ffn), f32(x, hidden), f32(logits, vocab), out.download(0, 16, np.uint32).copy()))
    (gu_a, x_a, lg_a, tok_a), (gu_b, x_b, lg_b, tok_b) = results
    assert rel_err(gu_b, gu_a) <= TOL and rel_err(x_b, x_a) <= TOL and rel_err(lg_b, lg_a) <= TOL
    # and against the oracle's arithmetic
    h = oracle.rmsnorm(x0, f32(norm, hidden), eps)
    ref_gu = oracle.matmul_q8_0(raw_gu, 2 * ffn, hidden, h)
    assert rel_err(gu_b, ref_gu) <= TOL
    act = np.array([oracle.silu(v) for v in ref_gu[:ffn]], np.float32) * ref_gu[ffn:]
    ref_x = x0 + oracle.matmul_q8_0(raw_dn, hidden, ffn, act)
    assert rel_err(x_b, ref_x) <= TOL
    ref_lg = oracle.matmul_q8_0(raw_hd, vocab, hidden, oracle.rmsnorm(ref_x, f32(norm, hidden), eps))
    assert rel_err(lg_b, ref_lg) <= TOL
    assert int(tok_b[2]) == int(np.argmax(lg_b)) and list(tok_b[[0, 1, 3]]) == [0, 0, 0]
    if np.partition(ref_lg, -2)[-1] - np.partition(ref_lg, -2)[-2] > 1e-3:
        assert int(tok_b[2]) == oracle.argmax(ref_lg) == int(tok_a[2])


@pytest.mark.parametrize("heads,kvh,hd,window,cap,filled", [(16, 8, 128, 0, 700, 600), (4, 1, 256, 70, 300, 200),
                                                            (32, 8, 128, 0, 200, 0), (8, 8, 128, 0, 5000, 4500)])
def test_recorded_attention_equals_the_decode_kernel(ctx, oracle, heads, kvh, hd, window, cap, filled):
    """Three consecutive positions: cache rows and the advanced position agree to the bit, outputs to
    rounding of the split merge."""
    eps, scale = 1e-6, 1.0 / np.sqrt(np.float32(hd))
    qn = ctx.floats((1 + 0.1 * T.activations(0, 20, hd)).astype(np.float32))
    kn = ctx.floats((1 + 0.1 * T.activations(0, 21, hd)).astype(np.float32))
    inv = ctx.floats(oracle.rope_inv_freq(hd, 1e6))
    kfill = T.activations(1, 1, kvh * cap * hd).astype(np.float16)
    vfill = T.activations(1, 2, kvh * cap * hd).astype(np.float16)
    plane = kvh * cap * hd * 2
    status = ctx.buffer(4, shared=True)
    status.zero()
    results = []
    for recorded in (False, True):
        kc, vc = ctx.from_array(kfill), ctx.from_array(vfill)
        pos_buf = ctx.from_array(np.array([filled], np.uint32))
        scratch = ctx.buffer(cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
        scratch.zero()
        q, k, v = ctx.buffer(heads * hd * 4), ctx.buffer(kvh * hd * 4), ctx.buffer(kvh * hd * 4)
        out = ctx.buffer(heads * hd * 4)
        prog = None
        if recorded:
            ctx.begin_program(4, heads * hd, ctx.program_attention_elems(heads, hd, cap))
            ctx.attention_decode_dev(q, k, v, qn, kn, inv, kc, vc, out, scratch, pos_buf, 0, status, heads, kvh, hd, hd,
                                     cap, window, eps, scale, exact=False)
            ctx.u32_add(pos_buf, 0, 1)
            prog = ctx.end_program()
        outs = []
        for step in range(3):
            q.upload(0, T.activations(30 + step, 30, heads * hd))
            k.upload(0, T.activations(30 + step, 31, kvh * hd))
            v.upload(0, T.activations(30 + step, 32, kvh * hd))
            if recorded:
                prog.launch()
            else:
                ctx.attention_decode_dev(q, k, v, qn, kn, inv, kc, vc, out, scratch, pos_buf, 0, status, heads, kvh, hd,
                                         hd, cap, window, eps, scale, exact=False)
                ctx.u32_add(pos_buf, 0, 1)
            ctx.fence()
            outs.append(f32(out, heads * hd))
        if recorded:
            assert prog.status() == 0
            prog.free()
        results.append((outs, kc.download(0, plane).copy(), vc.download(0, plane).copy(),
                        int(pos_buf.download(0, 4, np.uint32)[0])))
    for a, b in zip(results[0][0], results[1][0]):
        assert np.all(np.isfinite(b)) and float(np.max(np.abs(b))) > 0
        # same arithmetic per split; the merge rescales every 4 splits instead of every 8
        assert rel_err(b, a) <= 1e-6
    np.testing.assert_array_equal(results[1][1], results[0][1])
    np.testing.assert_array_equal(results[1][2], results[0][2])
    assert results[0][3] == results[1][3] == filled + 3
    assert int(status.download(0, 4, np.uint32)[0]) == 0


def test_program_refuses_what_it_cannot_hold(ctx):
    x, y = ctx.buffer(4096), ctx.buffer(4096)
    w = ctx.q8_0_matrix(T.q8_0_matrix(0, 1, 8, 96), 8, 96)
    ctx.begin_program(4)
    try:
        with pytest.raises(cuda.CudaError) as e:
            ctx.f32_scale(x, y, 2.0, 16)  # not an operator of a decode step
        assert e.value.code == -5 and "persistent program" in e.value.message
        with pytest.raises(cuda.CudaError) as e:
            ctx.q8_0_gemv(w, x, y, 8, 96)  # 96 columns: not whole 64-column chunks
        assert e.value.code == -5
        with pytest.raises(cuda.CudaError):
            ctx.begin_group()
    finally:
        ctx.abort_program()
    with pytest.raises(cuda.CudaError):
        ctx.abort_program()
    ctx.begin_program(1)
    with pytest.raises(cuda.CudaError):
        ctx.end_program()  # empty
    assert cuda.load_library().tm_cuda_program_supports_attention(16, 8, 128, 128) == 1
    assert cuda.load_library().tm_cuda_program_supports_attention(4, 2, 32, 32) == 0
    assert cuda.load_library().tm_cuda_program_supports_gemv(1152) == 1
    assert cuda.load_library().tm_cuda_program_supports_gemv(96) == 0


def test_a_wait_that_cannot_be_satisfied_runs_out_and_reports(ctx):
    """Consumers are told to expect sequence numbers nobody writes, with a short polling limit: the
    second operator's wait for the first one's output must give up, raise status bit 1 and return; the
    program then stays stopped, the context stays usable and a fresh program of the same operators
    runs."""
    n = 1024
    raw = T.q8_0_matrix(7, 1, n, n)
    w = ctx.q8_0_matrix(raw, n, n)
    x, y, y2 = ctx.floats(T.activations(7, 2, n)), ctx.buffer(n * 4), ctx.buffer(n * 4)

    def record():
        ctx.begin_program(4, 2 * n)
        ctx.q8_0_gemv(w, x, y, n, n)
        ctx.q8_0_gemv(w, y, y2, n, n)  # consumes the first operator's output
        return ctx.end_program()

    prog = record()
    prog.debug(sequence_skew=7, spin_limit=20000)
    y2.zero()
    prog.launch()
    ctx.fence()
    assert prog.status() & 1, "the wait did not report that it ran out"
    assert np.all(f32(y2, n) == 0.0), "a stopping kernel must not publish results"
    prog.debug(sequence_skew=0)
    prog.launch()  # a stopped program computes nothing further
    ctx.fence()
    assert np.all(f32(y2, n) == 0.0) and prog.status() & 1
    prog.free()
    good = record()
    good.launch()
    ctx.fence()
    assert good.status() == 0
    ya, yb = ctx.buffer(n * 4), ctx.buffer(n * 4)
    ctx.q8_0_gemv(w, x, ya, n, n)
    ctx.q8_0_gemv(w, ya, yb, n, n)
    assert rel_err(f32(y, n), f32(ya, n)) <= TOL and rel_err(f32(y2, n), f32(yb, n)) <= 10 * TOL
    good.free()


@pytest.fixture(scope="module", params=["qwen3", "gemma3"])
def small_artifact(request, tmp_path_factory):
    shape = T.SMALL_QWEN3 if request.param == "qwen3" else T.SMALL_GEMMA3
    path = tmp_path_factory.mktemp("gguf") / f"small_{request.param}.gguf"
    T.write_gguf(path, shape, seed=4, norm_jitter=0.1)
    return path, shape


def test_engine_decodes_on_the_program_like_the_graph_and_the_oracle(ctx, oracle, small_artifact):
    path, shape = small_artifact
    prompt = T.token_ids(12, 70, shape.vocab)
    cpu = oracle.Model(path)
    cpu.reset(256)
    ref, margins = cpu.generate_greedy(prompt, 100, chunk=32)
    runs = {}
    for name, persistent in (("program", True), ("graph", False)):
        eng = E.Engine(path, context=256, prefill_batch=32, persistent_step=persistent)
        assert bool(eng.decode_program()) == persistent
        got, stats = eng.generate(prompt, 100)
        assert stats.generated == 100
        # one launch per decode step on the program; several per step on the graph
        runs[name] = (got, stats.kernel_launches)
        bad = np.nonzero(got != ref)[0]
        assert bad.size == 0 or margins[bad[0]] <= 1e-3, \
            f"{name}: first divergence at step {bad[0]} (oracle top-1 margin {margins[bad[0]]:.3g})"
        # teacher-forced decode logits against the oracle at a few positions
        eng.reset()
        eng.prefill(prompt, want_token=True)
        cpu.reset(256)
        cpu.forward(prompt, want_logits=False)
        for t in T.token_ids(13, 12, shape.vocab):
            want = cpu.forward([int(t)])
            out = eng.step(int(t))
            assert np.max(np.abs(out - want)) <= 2e-2 * max(1.0, float(np.max(np.abs(want))))
        eng.close()
    assert runs["program"][1] < runs["graph"][1]


def test_engine_refuses_to_return_tokens_after_a_wait_ran_out(ctx, small_artifact):
    """The engine reads the device status words before it hands tokens or logits to the caller: a decode
    program whose consumers are made to wait for sequence numbers nobody writes (short polling limit,
    set on the host) stops itself, and generate() / logits() answer with a typed Internal error
    naming the wait instead of tokens."""
    path, shape = small_artifact
    eng = E.Engine(path, context=128, prefill_batch=32, persistent_step=True)
    prog = eng.decode_program()
    assert prog
    good, _ = eng.generate(T.token_ids(3, 9, shape.vocab), 6)
    assert len(good) == 6
    L, err = cuda.load_library(), C.create_string_buffer(256)
    assert L.tm_cuda_program_debug(C.c_void_p(eng.cuda_ctx()), C.c_void_p(prog), 5, 20000, err, 256) == 0
    with pytest.raises(E.EngineError) as e:
        eng.generate(T.token_ids(3, 9, shape.vocab), 6)
    assert e.value.code == "INTERNAL" and "wait" in e.value.message
    with pytest.raises(E.EngineError) as e:
        eng.logits()
    assert e.value.code == "INTERNAL"
    eng.close()
    # the context of another engine is unaffected
    other = E.Engine(path, context=128, prefill_batch=32)
    again, _ = other.generate(T.token_ids(3, 9, shape.vocab), 6)
    np.testing.assert_array_equal(again, good)
    other.close()
