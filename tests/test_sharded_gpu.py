"""Output-row split over two devices against the single-device engine and the
CPU oracle: one process per device, NCCL all-gathers on the engine's stream.
Needs two devices; on a single-device box the module skips."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tuckmill_b200 import cuda, engine as E, testing as T

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_ranks(world, path, mode, out):
    comm = E.comm_id().hex()
    env = {**os.environ, "PYTHONPATH": str(ROOT), "NCCL_NVLS_ENABLE": "0"}
    procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "_shard_gpu_worker.py"), str(r), str(world), comm,
                               str(path), mode, str(out)], cwd=ROOT, env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT) for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o.decode(errors="replace")[-3000:])
    assert all(p.returncode == 0 for p in procs), "\n----\n".join(logs)
    return np.load(out)


@pytest.mark.parametrize("mode", ["exact", "mma", "exact-pair", "mma-pair"])
def test_two_device_split_matches_single_device_and_oracle(oracle, tmp_path, mode):
    if cuda.available() < 2:
        pytest.skip("needs two devices")
    shape = T.TINY_QWEN3
    path = tmp_path / "tiny.gguf"
    T.write_gguf(path, shape, seed=3, norm_jitter=0.1)
    got = run_ranks(2, path, mode, tmp_path / "rank0.npz")

    toks = T.token_ids(5, 24, shape.vocab)
    one = E.Engine(path, context=96, exact=mode.startswith("exact"), prefill_batch=16)
    scored = one.score(toks)
    one.reset()
    one.prefill(toks, want_token=True)
    prefill_logits, prefill_token = one.logits(), one.prefill_token()
    one.reset()
    generated, _ = one.generate(T.token_ids(6, 19, shape.vocab), 40)
    allocated_one = one.refresh_info().allocated_bytes
    one.close()

    scale = max(1.0, float(np.max(np.abs(scored))))
    # The GEMV's column split depends on the matrix shape, so a rank's rows may be
    # summed in another order than the whole matrix's: tolerance, not identity.
    tol = 1e-4 if mode.startswith("exact") else 2e-2
    assert np.max(np.abs(got["scored"] - scored)) <= 1e-4 * scale
    assert np.max(np.abs(got["prefill_logits"] - prefill_logits)) <= tol * scale
    assert int(got["prefill_token"]) == prefill_token == int(np.argmax(got["prefill_logits"]))
    assert list(got["generated"]) == list(generated)
    assert int(got["allocated"]) < allocated_one

    cpu = oracle.Model(path)
    cpu.reset(96)
    ref = np.stack([cpu.forward([t]) for t in toks])
    assert np.max(np.abs(got["scored"] - ref)) <= 1e-4 * max(1.0, float(np.max(np.abs(ref))))
    cpu.reset(96)
    ref_tokens, _ = cpu.generate_greedy(T.token_ids(6, 19, shape.vocab), 40)
    assert list(got["generated"]) == list(ref_tokens)


@pytest.mark.parametrize("mode", ["batch-exact", "batch-mma"])
def test_two_device_split_decodes_several_sequences(tmp_path, mode):
    """generate_batch on a model split over two devices: every request's tokens are the ones the
    single-device engine produces for that request alone."""
    if cuda.available() < 2:
        pytest.skip("needs two devices")
    shape = T.TINY_QWEN3
    path = tmp_path / "tiny.gguf"
    T.write_gguf(path, shape, seed=3, norm_jitter=0.1)
    got = run_ranks(2, path, mode, tmp_path / "rank0.npz")
    prompts = [T.token_ids(30 + i, 4 + 5 * i, shape.vocab) for i in range(4)]
    one = E.Engine(path, context=64, exact=(mode == "batch-exact"), prefill_batch=16)
    total = 0
    for i, p in enumerate(prompts):
        want, _ = one.generate(p, 14)
        assert list(got[f"tokens{i}"]) == list(want), f"request {i}"
        total += len(want)
    assert int(got["generated"]) == total
    one.close()


def test_peer_memory_push_all_gather(tmp_path):
    """tm_cuda_push_rows_f32 over a symmetric arena: every rank receives every rank's
    rows at the interleaved position, round after round, eagerly and from a replayed
    dispatch group; no bounded wait ever ran out."""
    if cuda.available() < 2:
        pytest.skip("needs two devices")
    comm = cuda.comm_unique_id().hex()
    env = {**os.environ, "PYTHONPATH": str(ROOT), "NCCL_NVLS_ENABLE": "0"}
    procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "_push_worker.py"), str(r), "2", comm], cwd=ROOT,
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(2)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o.decode(errors="replace")[-3000:])
    assert all(p.returncode == 0 for p in procs), "\n----\n".join(logs)
