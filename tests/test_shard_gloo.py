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
