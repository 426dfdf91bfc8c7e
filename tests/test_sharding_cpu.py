"""CPU checks of the output-row split: the per-rank preflight, the refusals, and
a world_size-2 run over gloo of the split / all-gather / sharded-argmax rules."""
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from tuckmill_b200 import cuda, engine as E, sharding as S, testing as T

ROOT = Path(__file__).resolve().parent.parent


def test_row_ranges_tile_the_matrix():
    for rows, world in [(151936, 8), (4096, 4), (12288, 2), (96, 1)]:
        spans = [S.row_range(r, world, rows) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    # 151936 / 8 = 18992 rows per rank: a multiple of 16, not of 128 (the kernels keep a row tail).
    assert S.row_range(1, 8, 151936) == (18992, 37984) and 18992 % 16 == 0 and 18992 % 128 != 0
    with pytest.raises(ValueError):
        S.row_range(0, 3, 4096)
    g = S.shard_geometry(T.QWEN3_8B, 8)
    assert (g.heads, g.kv_heads, g.ffn, g.hidden, g.vocab) == (4, 1, 1536, 512, 18992)
    with pytest.raises(ValueError):
        S.shard_geometry(T.GEMMA3_1B, 2)  # one KV head cannot be divided


def test_column_ranges_are_whole_blocks():
    assert S.col_range(1, 4, 4096) == (1024, 2048)
    assert [S.col_range(r, 2, 64) for r in range(2)] == [(0, 32), (32, 64)]
    with pytest.raises(ValueError):
        S.col_range(0, 4, 96)  # 24 columns per rank: not whole Q8_0 blocks
    with pytest.raises(ValueError):
        S.col_range(2, 2, 64)
    parts = [np.full(3, 0.1, np.float32), np.full(3, 0.2, np.float32), np.full(3, 0.3, np.float32)]
    want = np.float32(np.float32(np.float32(0.1) + np.float32(0.2)) + np.float32(0.3))
    assert np.all(S.reduce_ranks(parts) == want)


def test_per_rank_plan_divides_projections_and_kv(tmp_path):
    """The preflight of rank r prices 1/W of every projection and of the KV
    cache, the whole embedding table and the norm vectors (per-rank plans of the
    reference's single-device preflight, crates/tuckcore/src/qwen35_gpu.rs:1181-1193)."""
    path = tmp_path / "t.gguf"
    s = T.TINY_QWEN3
    T.write_gguf(path, s, seed=2)
    whole = E.plan(path, 64, 8 << 30)
    W = 2
    ranks = [E.plan(path, 64, 8 << 30, r, W) for r in range(W)]
    assert ranks[0].plan_weights == ranks[1].plan_weights
    assert ranks[0].plan_state * W == whole.plan_state
    g = S.shard_geometry(s, W)
    hd = s.head_dim
    mats = s.layers * sum(cuda.packed_bytes(o, i) for o, i in
                          [((g.heads + 2 * g.kv_heads) * hd, s.hidden), (g.hidden, s.heads * hd),
                           (2 * g.ffn, s.hidden), (g.hidden, s.ffn)])
    mats += cuda.packed_bytes(s.vocab, s.hidden) + cuda.packed_bytes(g.vocab, s.hidden)  # embedding whole, head split
    norms = 4 * (s.layers * (2 * s.hidden + 2 * hd) + s.hidden)
    assert ranks[0].plan_weights == mats + norms
    assert ranks[0].plan_weights < whole.plan_weights
    # the one-row exchange slots of every layer (o and down): one 8-byte (value, number) pair per
    # column and rank, priced on every rank alike
    assert ranks[0].plan_scratch == ranks[1].plan_scratch
    assert ranks[0].plan_scratch >= s.layers * 2 * s.hidden * W * 8


def test_split_refusals_are_typed(tmp_path):
    path = tmp_path / "g.gguf"
    T.write_gguf(path, T.TINY_GEMMA3, seed=2)
    with pytest.raises(E.EngineError) as e:
        E.plan(path, 64, 8 << 30, 0, 2)  # one KV head
    assert e.value.code == "INVALID_REQUEST"
    path = tmp_path / "q.gguf"
    T.write_gguf(path, T.TINY_QWEN3, seed=2)
    with pytest.raises(E.EngineError) as e:
        E.plan(path, 64, 8 << 30, 2, 2)  # rank outside the split
    assert e.value.code == "INVALID_REQUEST"
    with pytest.raises(E.EngineError):
        E.plan(path, 64, 8 << 30, 0, 3)


def test_interleave_and_argmax_rules():
    wire = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    y = S.interleave_rows(wire, 2, 3, 4)
    assert y.shape == (3, 8) and list(y[1]) == [4, 5, 6, 7, 16, 17, 18, 19]
    assert S.merge_argmax([(np.float32(2), 9), (np.float32(2), 3), (np.float32(1), 0)]) == 3
    assert S.merge_argmax([(np.float32(-1), 0), (np.float32(5), 70)]) == 70


def test_world_size_2_row_split_over_gloo(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "picks.npy"
    procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "_shard_worker.py"), str(r), "2", str(port), str(out)],
                              cwd=ROOT, env={**__import__("os").environ, "PYTHONPATH": str(ROOT)},
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(2)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o.decode(errors="replace"))
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    assert np.load(out).shape == (5,)
