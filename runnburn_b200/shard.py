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


class PeerLeft(RuntimeError):
    """Raised before a step when another rank has announced that it left (or stopped beating)."""

    def __init__(self, rank: int, why: str):
        super().__init__(f"rank {rank} {why}")
        self.rank = rank


class StepGuard:
    """Host-side failure detection for the sharded decoder.  The exchange kernels of a step wait on
    flags that every rank raises, so a rank may only leave BETWEEN steps, and the others have to
    learn of it on the host before they launch the next step (a launch that waited for a missing
    rank would only end through the kernels' bounded waits and the device error word).

    Every rank writes `beat/<rank>` = step number into the job's key-value store before a step and
    reads the others' keys; `leave()` writes `left/<rank>`.  `check()` raises PeerLeft when a rank
    has left, or when a rank's beat is more than `max_lag` steps behind and `stale_after` seconds
    old.  The store is torch.distributed's (TCPStore / c10d), no collective is involved, so the
    check cannot hang on the rank that is gone."""

    def __init__(self, store, rank: int, world: int, max_lag: int = 1, stale_after: float = 30.0):
        self.store, self.rank, self.world = store, rank, world
        self.max_lag, self.stale_after = max_lag, stale_after
        self._seen = {}          # rank -> (last step seen, when it was first seen)
        self.store.set(f"beat/{rank}", "-1")

    def beat(self, step: int) -> None:
        self.store.set(f"beat/{self.rank}", str(step))

    def leave(self, why: str = "left") -> None:
        self.store.set(f"left/{self.rank}", why)

    def check(self, step: int) -> None:
        import time
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            if self.store.check([f"left/{r}"]):
                raise PeerLeft(r, "left the job: " + self.store.get(f"left/{r}").decode())
            if not self.store.check([f"beat/{r}"]):
                continue                           # not started yet: the rendezvous covers that
            s = int(self.store.get(f"beat/{r}").decode())
            last = self._seen.get(r)
            if last is None or last[0] != s:
                self._seen[r] = (s, now)
            elif step - s > self.max_lag and now - last[1] > self.stale_after:
                raise PeerLeft(r, f"stopped at step {s} ({now - last[1]:.0f} s ago)")

    def step(self, step: int) -> None:
        """Call before launching step `step`."""
        self.check(step)
        self.beat(step)
