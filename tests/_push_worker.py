"""Child process of the peer-memory exchange test: one rank pushes its slices into
symmetric buffers for several rounds; every rank checks what it received."""
import sys

import numpy as np


def main() -> None:
    rank, world, comm_hex = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    from tuckmill_b200 import cuda

    ctx = cuda.CudaContext(rank)
    ctx.comm_init(bytes.fromhex(comm_hex), rank, world)
    n_rows, width = 5, 96
    arena = ctx.symm_buffer(2 * n_rows * width * world * 4 + 4 * 300 * world * 4)
    # two ragged-size views used in turn, plus a wide single-row one (the decode shape)
    a = arena.view(0, n_rows * width * world * 4)
    b = arena.view(n_rows * width * world * 4, n_rows * width * world * 4)
    wide = arena.view(2 * n_rows * width * world * 4, 300 * world * 4)
    for rnd in range(6):
        dst = a if rnd % 2 == 0 else b
        mine = (np.arange(n_rows * width, dtype=np.float32) + 1000 * rank + 7 * rnd).reshape(n_rows, width)
        src = ctx.floats(mine)
        ctx.push_rows_f32(src, dst, n_rows, width)
        got = dst.download(0, n_rows * width * world * 4, np.float32).reshape(n_rows, world, width)
        for r in range(world):
            want = (np.arange(n_rows * width, dtype=np.float32) + 1000 * r + 7 * rnd).reshape(n_rows, width)
            assert np.array_equal(got[:, r, :], want), (rnd, r)
        w_src = ctx.floats(np.full(300, rank + 0.5 + rnd, np.float32))
        ctx.push_rows_f32(w_src, wide, 1, 300)
        gw = wide.download(0, 300 * world * 4, np.float32).reshape(world, 300)
        assert all(np.all(gw[r] == r + 0.5 + rnd) for r in range(world)), rnd
    # the same exchange recorded in a dispatch group and replayed
    src = ctx.floats(np.full(n_rows * width, float(rank), np.float32))
    ctx.begin_group()
    ctx.push_rows_f32(src, a, n_rows, width)
    ctx.push_rows_f32(src, b, n_rows, width)
    g = ctx.end_group_retain()
    for _ in range(3):
        g.launch()
    ctx.fence()
    got = b.download(0, n_rows * width * world * 4, np.float32).reshape(n_rows, world, width)
    assert all(np.all(got[:, r, :] == r) for r in range(world))
    assert ctx.symm_status(arena) == 0
    g.free()

    # The one-row exchange with the sum folded in (8-byte value/number pairs, one launch): two views
    # in turn, eagerly and from a replayed dispatch group, against the rank-ordered f32 sum.
    for width in (300, 4096):
        pairs = ctx.symm_buffer(2 * width * world * 8)
        views = [pairs.view(i * width * world * 8, width * world * 8) for i in range(2)]
        y_host = np.linspace(-1, 1, width, dtype=np.float32)
        y = ctx.floats(y_host)

        def part(r, rnd):
            return (np.sin(np.arange(width, dtype=np.float32) * (r + 1) + rnd) * (1 + r)).astype(np.float32)

        def expect(yh, rnd):
            p = part(0, rnd)
            for r in range(1, world):
                p = (p + part(r, rnd)).astype(np.float32)
            return (yh + p).astype(np.float32)

        for rnd in range(8):
            src = ctx.floats(part(rank, rnd))
            ctx.exchange_add_ll(src, views[rnd % 2], y, width)
            y_host = expect(y_host, rnd)
            assert np.array_equal(y.download(0, width * 4, np.float32), y_host), (width, rnd)
        src = ctx.floats(part(rank, 99))
        ctx.begin_group()
        for i in range(4):
            ctx.exchange_add_ll(src, views[i % 2], y, width)
        g = ctx.end_group_retain()
        for _ in range(3):
            g.launch()
        ctx.fence()
        for _ in range(12):
            y_host = expect(y_host, 99)
        assert np.array_equal(y.download(0, width * 4, np.float32), y_host), width
        assert ctx.symm_status(pairs) == 0
        g.free()

    # GEMM and exchange as one kernel: this rank multiplies its rows and its epilogue writes them
    # into every rank's gathered Y; the result must be the whole product on every rank.
    import oracle
    from tuckmill_b200 import testing as T
    for rows, cols, batch in [(512, 256, 300), (1024, 1024, 77)]:
        local = rows // world
        w_full = T.q8_0_matrix(4, 11, rows, cols)
        w = ctx.q8_0_matrix(T.q8_0_rows(4, 11, rank * local, local, cols), local, cols)
        X = T.activations(4, 12, batch * cols).reshape(batch, cols)
        ys = ctx.symm_buffer(2 * batch * rows * 4)
        views = [ys.view(i * batch * rows * 4, batch * rows * 4) for i in range(2)]
        xb = ctx.floats(X)
        for i in range(4):
            ctx.q8_0_gemm_mma_push(w, xb, views[i % 2], local, cols, batch)
        got = views[1].download(0, batch * rows * 4, np.float32).reshape(batch, rows)
        want = oracle.matmul_q8_0(w_full, rows, cols, X)
        assert float(np.max(np.abs(got - want))) <= 2e-2, (rows, cols, batch, float(np.max(np.abs(got - want))))
        assert np.array_equal(got, views[0].download(0, batch * rows * 4, np.float32).reshape(batch, rows))
        assert ctx.symm_status(ys) == 0 and not ctx.mma_aborted()
    print("rank", rank, "ok", flush=True)


if __name__ == "__main__":
    main()
