"""Row sharding + all-gather, checked among CPU ranks (gloo, world size 2): every rank computes
its row slices with the oracle, the slices are all-gathered, and the result must equal the
unsharded oracle bit for bit — the algebra the multi-GPU decoder relies on."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r); sys.path.insert(0, %r)
    import numpy as np, torch, torch.distributed as dist
    import oracle as orc
    from runnburn_b200 import shard
    from synth import llama_description
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    desc = llama_description(seed=3, n_layer=1, hidden=512, n_head=4, n_kv_head=2, n_ff=1024, vocab=512)
    cfg, L = desc["cfg"], desc["layers"][0]
    p = shard.plan(cfg["n_head"], cfg["n_kv_head"], cfg["hidden"], cfg["n_ff"], cfg["vocab"], world, rank)
    rng = np.random.default_rng(0)
    x = rng.standard_normal(cfg["hidden"]).astype(np.float32)

    def sharded_gemv(pair, rows_total, cols, rr, vec):
        t, data = pair
        rb = orc.row_bytes(t, cols)
        mine = orc.gemv(t, shard.shard_rows(data, rb, rr), vec, rr.rows, cols)
        parts = [torch.empty(rr.rows) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(mine))
        full = torch.cat(parts).numpy()
        ref = orc.gemv(t, data, vec, rows_total, cols)
        assert np.array_equal(full.view(np.uint32), ref.view(np.uint32))
        return full

    q = sharded_gemv(L["wq"], cfg["n_head"] * 128, cfg["hidden"], p.wq, x)
    k = sharded_gemv(L["wk"], cfg["n_kv_head"] * 128, cfg["hidden"], p.wk, x)
    g = sharded_gemv(L["gate"], cfg["n_ff"], cfg["hidden"], p.gate, x)
    d = sharded_gemv(L["down"], cfg["hidden"], cfg["n_ff"], p.down, g)
    # attention is local to a rank's KV heads: its query heads only need its own K/V columns
    assert p.q_heads.begin // (cfg["n_head"] // cfg["n_kv_head"]) == p.kv_heads.begin
    # LM head: per-shard argmax candidates (value, global index) -> last index of the maximum
    t, data = desc["output"]
    rb = orc.row_bytes(t, cfg["hidden"])
    logits_l = orc.gemv(t, shard.shard_rows(data, rb, p.output), x, p.output.rows, cfg["hidden"])
    li = orc.argmax_last(logits_l)
    cand = [None] * world
    dist.all_gather_object(cand, (float(logits_l[li]), int(li + p.output.begin)))
    best = max(cand, key=lambda c: (c[0], c[1]))[1]
    assert best == orc.argmax_last(orc.gemv(t, data, x, cfg["vocab"], cfg["hidden"]))
    # a rank that fails is seen by the others as an error, not a hang
    dist.barrier()
    dist.destroy_process_group()
    sys.stdout.write("rank %%d ok\\n" %% rank)
    sys.stdout.flush()
""")


def test_row_shard_allgather_two_cpu_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % (str(ROOT), str(ROOT / "tests")))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_shard_plan_rules():
    from runnburn_b200 import shard
    p = shard.plan(64, 8, 8192, 28672, 128256, 8, 3)
    assert (p.wq.begin, p.wq.end) == (3 * 1024, 4 * 1024) and p.wk.rows == 128 and p.wo.rows == 1024
    assert p.gate.rows == 3584 and p.output.rows == 16032 and p.kv_heads.rows == 1 and p.q_heads.rows == 8
    with pytest.raises(ValueError):
        shard.plan(32, 8, 4096, 14336, 128256, 16, 0)      # more GPUs than KV heads
    with pytest.raises(ValueError):
        shard.plan(32, 8, 4096 + 256, 14336, 128256, 8, 0)  # hidden slices must stay block-aligned


def test_reference_arm_under_torchrun_prints_once():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29732", str(ROOT / "bench.py"), "--gpus", "2",
                        "--impl", "reference", "--steps", "1", "--warmup", "1", "--workload", "tiny-llama-ctx256"],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1 and '"impl": "reference"' in lines[0]


LEAVER = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, %r)
    import torch, torch.distributed as dist
    from datetime import timedelta
    from runnburn_b200.shard import PeerLeft, StepGuard
    dist.init_process_group("gloo", timeout=timedelta(seconds=20))
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    guard = StepGuard(store, rank, world)
    dist.barrier()
    done = 0
    try:
        for step in range(6):
            if rank == 1 and step == 3:
                # leaves BETWEEN steps: nothing of its own in flight, says so, exits cleanly
                guard.leave("planned exit after step 2")
                sys.stdout.write("rank 1 left\\n"); sys.stdout.flush()
                os._exit(0)
            if rank == 0 and step == 3:
                time.sleep(1.0)                      # the note has time to land
            guard.step(step)
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)                       # the step's exchange: needs every rank
            assert float(t[0]) == 3.0
            done += 1
    except PeerLeft as e:
        sys.stdout.write("rank %%d saw rank %%d leave after %%d steps: %%s\\n" %% (rank, e.rank, done, e)); sys.stdout.flush()
        os._exit(0)                                  # no collective was started with the rank missing
    sys.stdout.write("rank %%d finished %%d steps\\n" %% (rank, done)); sys.stdout.flush()
""")


def test_cpu_rank_leaves_between_steps_and_the_other_learns_on_the_host(tmp_path):
    """World size 2 on CPU (gloo).  Rank 1 leaves between steps 2 and 3; rank 0 must learn of it from the
    store BEFORE starting step 3's exchange, i.e. end cleanly after exactly 3 steps without a hung or
    timed-out collective."""
    script = tmp_path / "leaver.py"
    script.write_text(LEAVER % (str(ROOT),))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29733", str(script)],
                       capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 1 left" in r.stdout
    assert "rank 0 saw rank 1 leave after 3 steps" in r.stdout, r.stdout[-2000:]


def test_step_guard_flags_a_rank_whose_beat_went_stale():
    from runnburn_b200.shard import PeerLeft, StepGuard

    class FakeStore(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

        def check(self, keys):
            return all(k in self for k in keys)

    st = FakeStore()
    a, b = StepGuard(st, 0, 2, max_lag=1, stale_after=0.0), StepGuard(st, 1, 2)
    for step in range(3):
        b.step(step)
        a.step(step)
    a.step(3)                    # rank 1 is one step behind: tolerated
    with pytest.raises(PeerLeft) as e:
        a.check(4)               # two behind and its beat has not moved since it was last read
    assert e.value.rank == 1
