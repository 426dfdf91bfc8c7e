"""Host arithmetic of the split of one model over W devices (one process per device).

Every Q8_0 row is an independent byte range and every output element depends on
one weight row and the whole input vector, so rank r owns rows [r*N/W, (r+1)*N/W)
of q|k|v, gate|up and the head (`row_range`; an all-gather reassembles such an
output).  Whole attention heads and a slice of the FFN width therefore stay on one
rank, and the two projections that consume them, o and down, are cut the other
way: rank r holds the COLUMNS that multiply its own heads / FFN slice
(`col_range`, whole 32-column blocks), produces a full-width partial product, and
the partials are added in rank order (`reduce_ranks`) -- one exchange per
projection, every rank computing the same bits (for one decode row the exchange and
the sum are one launch of 8-byte words, `pair_words` / `read_pairs`).  The reference runs on one device;
this module states the rules the C++ engine (csrc/engine/engine.cpp) and the
exchanges (csrc/tm_cuda_comm.cu) follow, so launchers and tests can share them.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def row_range(rank: int, world: int, rows: int) -> tuple[int, int]:
    """Half-open global row range of `rank`; rows must divide evenly."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a split of {world}")
    if rows % world:
        raise ValueError(f"{rows} rows do not divide over {world} devices")
    per = rows // world
    return rank * per, (rank + 1) * per


def col_range(rank: int, world: int, cols: int, block: int = 32) -> tuple[int, int]:
    """Half-open column range of `rank` for a projection cut by input columns; ranges are whole
    quantisation blocks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside a split of {world}")
    if cols % world or (cols // world) % block:
        raise ValueError(f"{cols} columns do not divide into {world} ranges of whole {block}-column blocks")
    per = cols // world
    return rank * per, (rank + 1) * per


def reduce_ranks(partials) -> np.ndarray:
    """Sum of the ranks' partial products, added in rank order in f32 (what every rank computes)."""
    acc = np.array(partials[0], dtype=np.float32, copy=True)
    for p in partials[1:]:
        acc = (acc + np.asarray(p, dtype=np.float32)).astype(np.float32)
    return acc


def pair_words(values, number: int) -> np.ndarray:
    """The wire format of the one-launch decode exchange (tm_cuda_exchange_add_ll_f32): every f32 value
    travels as one 8-byte word, value bits in the low half and the exchange number in the high half, so
    a word is complete or absent -- never half written."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return bits | (np.uint64(number & 0xFFFFFFFF) << np.uint64(32))


def read_pairs(words, number: int) -> np.ndarray:
    """Values of the words that carry `number`; a word with another number has not arrived yet (the
    kernel polls it again) and makes this host model raise."""
    w = np.ascontiguousarray(words, dtype=np.uint64)
    if np.any((w >> np.uint64(32)) != np.uint64(number & 0xFFFFFFFF)):
        raise ValueError("a word of another exchange")
    return (w & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32)


@dataclass(frozen=True)
class ShardGeometry:
    """Per-rank sizes of a dense decoder under the split."""

    world: int
    heads: int      # query heads on this rank
    kv_heads: int   # KV heads on this rank (the KV cache is divided with them)
    ffn: int        # gate / up rows (and down columns) on this rank
    hidden: int     # hidden size / world (head rows are counted in `vocab`)
    vocab: int      # head rows on this rank


def shard_geometry(shape, world: int) -> ShardGeometry:
    """Refuses what the engine refuses: a head count, FFN width, hidden size or
    vocabulary that does not divide, or a split that would cut a KV group."""
    for name in ("heads", "kv_heads", "ffn", "hidden", "vocab"):
        if getattr(shape, name) % world:
            raise ValueError(f"{name} = {getattr(shape, name)} does not divide over {world} devices")
    return ShardGeometry(world, shape.heads // world, shape.kv_heads // world, shape.ffn // world,
                         shape.hidden // world, shape.vocab // world)


def interleave_rows(gathered: np.ndarray, world: int, n_rows: int, width: int) -> np.ndarray:
    """An all-gather of per-rank [n_rows][width] slices arrives rank-major,
    [world][n_rows][width]; the activation layout is [n_rows][world * width]."""
    g = np.asarray(gathered).reshape(world, n_rows, width)
    return np.ascontiguousarray(g.transpose(1, 0, 2)).reshape(n_rows, world * width)


def local_argmax(x: np.ndarray, index_offset: int) -> tuple[np.float32, int]:
    """(value, global index) of the first maximum of one rank's slice."""
    i = int(np.argmax(x))
    return np.float32(x[i]), index_offset + i


def merge_argmax(pairs) -> int:
    """The larger value wins; equal values go to the lower GLOBAL index, so the
    sharded choice equals the single-device one (first maximum)."""
    best_v, best_i = None, None
    for v, i in pairs:
        if best_v is None or v > best_v or (v == best_v and i < best_i):
            best_v, best_i = v, i
    return int(best_i)
