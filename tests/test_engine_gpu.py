"""Model-level parity of the CUDA engine against the CPU oracle on seeded Q8_0
artifacts -- the policy of crates/tuckcore/src/executor.rs:2143-2321 (logits
within 1e-2 * scale, equal top-1, equal greedy tokens) and the engine
invariants of crates/tuckcore/src/engine/metal.rs:3682-3774 (prefill == decode,
ledger == plan)."""
import numpy as np
import pytest

from tuckmill_b200 import engine as E, testing as T

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["qwen3", "gemma3"])
def artifact(request, tmp_path_factory):
    shape = T.TINY_QWEN3 if request.param == "qwen3" else T.TINY_GEMMA3
    path = tmp_path_factory.mktemp("gguf") / f"tiny_{request.param}.gguf"
    T.write_gguf(path, shape, seed=3, norm_jitter=0.1)
    return path, shape


def logit_scale(ref):
    return max(1.0, float(np.max(np.abs(ref))))


def test_teacher_forced_logits_match_oracle(ctx, oracle, artifact):
    path, shape = artifact
    toks = T.token_ids(5, 24, shape.vocab)
    cpu = oracle.Model(path)
    cpu.reset(64)
    ref = np.stack([cpu.forward([t]) for t in toks])
    eng = E.Engine(path, context=64, exact=True)
    got = eng.score(toks)
    for i in range(len(toks)):
        assert np.max(np.abs(got[i] - ref[i])) <= 1e-2 * logit_scale(ref[i]), f"position {i}"
        assert int(np.argmax(got[i])) == oracle.argmax(ref[i])
    # actual agreement is far tighter than the reference's policy bound
    assert np.max(np.abs(got - ref)) <= 1e-4 * logit_scale(ref)
    eng.close()


@pytest.mark.parametrize("n_prompt", [1, 3, 17, 40])
def test_prefill_equals_token_by_token_decode(ctx, artifact, n_prompt):
    """Exact mode: batched prefill is bit-identical to feeding the same tokens
    one at a time (lens straddle the 16-token prefill batch and Gemma's window 8)."""
    path, shape = artifact
    toks = T.token_ids(9, n_prompt, shape.vocab)
    eng = E.Engine(path, context=64, exact=True, prefill_batch=16)
    eng.reset()
    for t in toks[:-1]:
        eng.step(int(t), want_logits=False)
    by_token = eng.step(int(toks[-1]))
    eng.reset()
    eng.prefill(toks, want_token=True)
    np.testing.assert_array_equal(eng.logits(), by_token)
    assert eng.prefill_token() == int(np.argmax(by_token))
    eng.close()


def test_greedy_generation_matches_oracle(ctx, oracle, artifact):
    path, shape = artifact
    prompt = T.token_ids(11, 20, shape.vocab)
    cpu = oracle.Model(path)
    cpu.reset(64)
    ref, margins = cpu.generate_greedy(prompt, 24, chunk=16)
    for mode in (True, False):
        eng = E.Engine(path, context=64, exact=mode, prefill_batch=16)
        got, stats = eng.generate(prompt, 24)
        assert stats.generated == 24 and stats.prompt_tokens == 20
        # dispatches: 2 prefill chunks + 23 decode graph replays (+ bookkeeping)
        assert stats.kernel_launches > 0
        bad = np.nonzero(got != ref)[0]
        assert bad.size == 0, f"first divergence at step {bad[0]} (oracle top-1 margin {margins[bad[0]]:.3g})"
        eng.close()


def test_ledger_equals_plan_and_info(ctx, artifact):
    path, shape = artifact
    eng = E.Engine(path, context=48)
    i = eng.info
    assert i.allocated_bytes == i.plan_weights + i.plan_state + i.plan_scratch
    assert i.plan_state == shape.layers * 2 * shape.kv_heads * 48 * shape.head_dim * 2
    assert i.kernel_impl == b"cuda" and i.kernel_id == f"ADR011:{shape.arch}-q8_0+f16:cuda".encode()
    assert i.reservation + i.overhead + i.safety_reserve <= i.budget
    eng.close()


def test_requests_are_validated(ctx, artifact):
    path, shape = artifact
    eng = E.Engine(path, context=8)
    with pytest.raises(E.EngineError) as e:
        eng.step(shape.vocab)
    assert e.value.code == "INVALID_REQUEST"
    with pytest.raises(E.EngineError) as e:
        eng.prefill(np.zeros(9, np.uint32))
    assert e.value.code == "CONTEXT_EXCEEDS_BUDGET"
    eng.reset()
    eng.prefill(np.zeros(8, np.uint32))
    with pytest.raises(E.EngineError) as e:
        eng.step(0)
    assert e.value.code == "CONTEXT_EXCEEDS_BUDGET"
    toks, st = eng.generate(np.zeros(4, np.uint32), 100)  # stops at capacity, never past it
    assert len(toks) == 5
    eng.close()
    with pytest.raises(E.EngineError) as e:
        E.Engine(path, context=8, kernels="metal")
    assert e.value.code == "UNAVAILABLE"
    with pytest.raises(E.EngineError) as e:
        E.Engine(path, context=8, kernels="scalar")
    assert e.value.code == "INVALID_REQUEST"
    with pytest.raises(E.EngineError) as e:
        E.Engine(path, context=8, budget_bytes=1 << 20)
    assert e.value.code == "MODEL_EXCEEDS_BUDGET"


def test_folded_output_norms_are_bit_identical(ctx, artifact, monkeypatch):
    """TM_ENGINE_FOLD_NORMS=1 folds each output norm + residual add of a Gemma-style layer into the
    projection that follows it (tm_cuda_q8_0_gemv_addnorm): fewer launches, the same bits."""
    path, shape = artifact
    toks = T.token_ids(21, 12, shape.vocab)
    runs = []
    for fold in ("0", "1"):
        monkeypatch.setenv("TM_ENGINE_FOLD_NORMS", fold)
        eng = E.Engine(path, context=64, exact=True)
        got, stats = eng.generate(toks, 10)
        runs.append((eng.score(toks), got, stats.kernel_launches))
        eng.close()
    np.testing.assert_array_equal(runs[1][0], runs[0][0])
    np.testing.assert_array_equal(runs[1][1], runs[0][1])
    if shape.arch == "gemma3":
        assert runs[1][2] < runs[0][2]  # two launches fewer per layer and decode step
    else:
        assert runs[1][2] == runs[0][2]  # no output norms: nothing to fold
