"""The benchmark's own configuration end to end: a Qwen3-0.6B-shaped Q8_0 decoder,
512-token prompt, 256 greedy tokens, CUDA engine (default, tolerance-qualified
kernels: tensor-core prefill GEMM and attention) against the CPU oracle.  The
target is token identity over all 256 steps; a divergence is tolerated only where
the oracle itself is undecided (top-1 margin below 1e-3 of the logit scale), which
is the reference's own policy for quantised executors
(crates/tuckcore/src/executor.rs:2143-2321)."""
import numpy as np
import pytest

import bench
from tuckmill_b200 import engine as E, testing as T

pytestmark = pytest.mark.gpu


def test_qwen3_0_6b_512_in_256_out_greedy_tokens_equal_the_oracle(ctx, oracle):
    shape, prompt_n, decode_n = bench.WORKLOADS["qwen3-0.6b"]
    path = bench.artifact("qwen3-0.6b", 0)
    prompt = T.token_ids(0, prompt_n, shape.vocab)
    cpu = oracle.Model(path)
    cpu.reset(prompt_n + decode_n + 16)
    ref, margins = cpu.generate_greedy(prompt, decode_n, chunk=128)
    eng = E.Engine(path, context=prompt_n + decode_n + 16)
    got, stats = eng.generate(prompt, decode_n)
    assert stats.generated == decode_n and stats.prompt_tokens == prompt_n
    bad = np.nonzero(np.asarray(got) != np.asarray(ref))[0]
    if bad.size:
        first = int(bad[0])
        assert margins[first] <= 1e-3 * max(1.0, float(np.max(np.abs(margins)))), \
            f"diverged at step {first} where the oracle's top-1 margin is {margins[first]:.3g}"
    # the last logits of the prefill, position by position agreement of the distribution
    eng.reset()
    eng.prefill(prompt, want_token=True)
    cpu.reset(prompt_n + 16)
    last = None
    for i in range(0, prompt_n, 128):
        last = cpu.forward(prompt[i:i + 128], want_logits=i + 128 >= prompt_n)
    logits = eng.logits()
    scale = max(1.0, float(np.max(np.abs(last))))
    assert np.max(np.abs(logits - last)) <= 2e-2 * scale  # the f16-operand prefill bar, per logit
    assert int(np.argmax(logits)) == oracle.argmax(last)
    eng.close()
