"""Child process of the world_size-2 CPU tests: one rank of an output-row split
over gloo.  Each rank multiplies only its own rows with the CPU oracle, the
ranks all-gather, and every rank checks the reassembled result against the
whole-matrix product."""
import os
import sys

import numpy as np


def run(rank: int, world: int, port: int, out_path: str) -> None:
    import torch
    import torch.distributed as dist

    import oracle
    from tuckmill_b200 import sharding as S, testing as T

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols, n = 96, 256, 5
        r0, r1 = S.row_range(rank, world, rows)
        # The generator is a function of (seed, tensor, row index): a rank builds only its rows.
        w_local = T.q8_0_rows(0, 7, r0, r1 - r0, cols)
        x = np.stack([T.activations(0, 100 + t, cols) for t in range(n)])
        y_local = oracle.matmul_q8_0(w_local, r1 - r0, cols, x, threads=1).reshape(n, r1 - r0)

        # Row all-gather: rank-major on the wire, [n][world * width] in the activation.
        parts = [torch.empty(n, r1 - r0) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(y_local)))
        wire = np.stack([p.numpy() for p in parts])
        y = S.interleave_rows(wire, world, n, r1 - r0)
        whole = oracle.matmul_q8_0(T.q8_0_matrix(0, 7, rows, cols), rows, cols, x, threads=1).reshape(n, rows)
        assert np.array_equal(y, whole), "row split + all-gather differs from the whole product"

        # Column split (o, down): each rank multiplies its column range by its slice of the input; the
        # full-width partial products are exchanged and added in rank order, identically on every rank.
        c0, c1 = S.col_range(rank, world, cols)
        raw = T.q8_0_matrix(0, 7, rows, cols)  # [rows][cols / 32][34]
        w_cols = np.ascontiguousarray(raw[:, c0 // 32:c1 // 32])
        part = oracle.matmul_q8_0(w_cols, rows, c1 - c0, np.ascontiguousarray(x[:, c0:c1]), threads=1).reshape(n, rows)
        slots = [torch.empty(n, rows) for _ in range(world)]
        dist.all_gather(slots, torch.from_numpy(np.ascontiguousarray(part)))
        summed = S.reduce_ranks([p.numpy() for p in slots])
        assert np.max(np.abs(summed - whole)) <= 1e-4 * max(1.0, float(np.max(np.abs(whole)))), "column split + reduce"
        check = [torch.empty(n, rows) for _ in range(world)]
        dist.all_gather(check, torch.from_numpy(summed))
        assert all(np.array_equal(c.numpy(), summed) for c in check), "ranks disagree on the reduced product"

        # The decode row's exchange as (value, number) words: two exchanges in turn on two slot views; a
        # stale view (the number of an earlier exchange) is recognised, the sum is the rank-ordered one.
        views = [None, None]
        for number in (1, 2, 3):
            row = part[number % n]
            mine = torch.from_numpy(S.pair_words(row, number).view(np.int64))
            got = [torch.empty(rows, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(got, mine)
            views[number % 2] = np.stack([g.numpy().view(np.uint64) for g in got])
            vals = [S.read_pairs(views[number % 2][r], number) for r in range(world)]
            assert np.array_equal(vals[rank], row)
            row_slots = [torch.empty(rows) for _ in range(world)]
            dist.all_gather(row_slots, torch.from_numpy(np.ascontiguousarray(row)))
            assert np.array_equal(S.reduce_ranks(vals), S.reduce_ranks([p.numpy() for p in row_slots]))
        try:
            S.read_pairs(views[0][0], 3)  # view 0 still holds exchange 2
            raise AssertionError("a stale word passed for a fresh one")
        except ValueError:
            pass

        # Sharded greedy choice: 8 bytes per rank instead of the logits.
        picks = []
        for t in range(n):
            logits = whole[t].copy()
            if t == 1:  # the same maximum on both ranks: the lower global index must win
                logits[5] = logits[rows - 3] = np.float32(1e9)
            if t == 2:  # a maximum that only the last rank holds
                logits[rows - 1] = np.float32(1e9)
            v, i = S.local_argmax(logits[r0:r1], r0)
            pairs = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
            dist.all_gather(pairs, torch.tensor([float(v), float(i)], dtype=torch.float64))
            choice = S.merge_argmax([(np.float32(p[0].item()), int(p[1].item())) for p in pairs])
            assert choice == oracle.argmax(logits), (t, choice, oracle.argmax(logits))
            picks.append(choice)
        assert picks[1] == 5 and picks[2] == rows - 1
        if rank == 0:
            np.save(out_path, np.asarray(picks, dtype=np.int64))
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    run(int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4])
