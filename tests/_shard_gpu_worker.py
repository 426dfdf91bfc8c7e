"""Child process of the multi-device tests: one rank of a row-split engine.
Every rank makes the same calls in the same order; rank 0 saves what it saw."""
import sys

import numpy as np


def main() -> None:
    rank, world, comm_hex, path, mode, out = sys.argv[1:7]
    rank, world = int(rank), int(world)
    from tuckmill_b200 import engine as E, testing as T

    shape = T.TINY_QWEN3
    if mode.startswith("batch-"):
        # several sequences on a split model: every exchange carries one row per sequence
        eng = E.Engine(path, context=64, device=rank, exact=(mode == "batch-exact"), prefill_batch=16, shard_rank=rank,
                       shard_world=world, comm_id=bytes.fromhex(comm_hex), sequences=5)
        info = eng.refresh_info()
        assert info.allocated_bytes == info.plan_weights + info.plan_state + info.plan_scratch
        prompts = [T.token_ids(30 + i, 4 + 5 * i, shape.vocab) for i in range(4)]
        first, _ = eng.generate_batch(prompts, 14)
        again, stats = eng.generate_batch(prompts, 14)
        assert all(list(a) == list(b) for a, b in zip(first, again))
        if rank == 0:
            np.savez(out, **{f"tokens{i}": np.asarray(t, dtype=np.int64) for i, t in enumerate(first)},
                     generated=stats.generated)
        eng.close()
        return
    import os
    # a decode step's exchanges: single launches of (value, number) pairs, or push + reduction
    os.environ["TM_ENGINE_PAIR_EXCHANGE"] = "1" if mode.endswith("-pair") else "0"
    eng = E.Engine(path, context=96, device=rank, exact=mode.startswith("exact"), prefill_batch=16, shard_rank=rank,
                   shard_world=world, comm_id=bytes.fromhex(comm_hex))
    info = eng.refresh_info()
    assert info.allocated_bytes == info.plan_weights + info.plan_state + info.plan_scratch
    toks = T.token_ids(5, 24, shape.vocab)
    scored = eng.score(toks)                      # token-by-token decode, logits gathered each step
    eng.reset()
    eng.prefill(toks, want_token=True)            # chunked prefill (16 + 8)
    prefill_logits = eng.logits()
    prefill_token = eng.prefill_token()
    eng.reset()
    generated, _ = eng.generate(T.token_ids(6, 19, shape.vocab), 40)
    if rank == 0:
        np.savez(out, scored=scored, prefill_logits=prefill_logits, prefill_token=prefill_token,
                 generated=np.asarray(generated, dtype=np.int64), allocated=info.allocated_bytes)
    eng.close()


if __name__ == "__main__":
    main()
