"""Row sharding of a Llama-style stack across the GPUs of one box (host-side plan).

Every weight matrix is cut by output rows, so block-quantised rows stay intact and no
re-quantisation is needed: q/k/v by head (each rank owns `n_kv_head / world` KV heads and the
query heads that map to them, which also shards the KV cache by KV head and keeps attention
local), o_proj / down by rows of the hidden vector, gate/up by rows of the FFN vector, the LM
head by vocabulary rows.  The partial output vectors are combined by all-gather.  The same
arithmetic is applied inside `rnb_b200_decoder_set_layer`; this module is what the host uses
to reason about it (and what the CPU tests exercise with gloo).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class RowRange:
    begin: int
    end: int

    @property
    def rows(self) -> int:
        return self.end - self.begin


@dataclass(frozen=True)
class ShardPlan:
    world: int
    rank: int
    wq: RowRange
    wk: RowRange
    wv: RowRange
    wo: RowRange
    gate: RowRange
    up: RowRange
    down: RowRange
    output: RowRange
    kv_heads: RowRange
    q_heads: RowRange


def _even(total: int, world: int, rank: int, unit: int, what: str) -> RowRange:
    if total % (world * unit) != 0:
        raise ValueError(f"{what}={total} does not split into {world} shards of multiples of {unit}")
    per = total // world
    return RowRange(rank * per, (rank + 1) * per)


def plan(n_head: int, n_kv_head: int, hidden: int, n_ff: int, vocab: int, world: int, rank: int,
         head_dim: int = 128) -> ShardPlan:
    """Shard plan of one rank; raises ValueError when the shapes do not split evenly
    (the conditions `rnb_b200_decoder_create` enforces)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} out of range for world size {world}")
    if n_head % n_kv_head != 0:
        raise ValueError("n_head must be a multiple of n_kv_head")
    kvh = _even(n_kv_head, world, rank, 1, "n_kv_head")
    group = n_head // n_kv_head
    qh = RowRange(kvh.begin * group, kvh.end * group)
    scale = lambda r: RowRange(r.begin * head_dim, r.end * head_dim)  # noqa: E731
    return ShardPlan(
        world=world, rank=rank, wq=scale(qh), wk=scale(kvh), wv=scale(kvh),
        wo=_even(hidden, world, rank, 256, "hidden"), gate=_even(n_ff, world, rank, 256, "n_ff"),
        up=_even(n_ff, world, rank, 256, "n_ff"), down=_even(hidden, world, rank, 256, "hidden"),
        output=_even(vocab, world, rank, 1, "vocab"), kv_heads=kvh, q_heads=qh)


def shard_rows(data, row_bytes: int, rows: RowRange):
    """The contiguous byte range of a row-major block-quantised matrix that holds `rows`."""
    return data[rows.begin * row_bytes: rows.end * row_bytes]
