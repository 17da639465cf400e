#!/usr/bin/env python
"""Headline benchmark: batch-1 greedy decode tok/s of a random-init Q4_K_M Llama stack.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

N = 1 runs BASELINE config 2 (Llama-3-8B shape, 4096-token context already in the fp16 KV
cache); N > 1 runs BASELINE config 5 (Llama-3-70B shape, context 32768) row-sharded over N
GPUs, one process per GPU, launched by torch.distributed.run.  A step is one decode token.
One JSON line is printed by rank 0.  `--impl reference` times the CPU oracle (the
restatement of the reference's rnb-cpu path; the Rust original cannot be built here) on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (shape, context, description)
    "llama3-8b-q4km-ctx4096": (dict(n_layer=32, hidden=4096, n_head=32, n_kv_head=8, n_ff=14336, vocab=128256), 4096),
    "llama3-70b-q4km-ctx32768": (dict(n_layer=80, hidden=8192, n_head=64, n_kv_head=8, n_ff=28672, vocab=128256), 32768),
    # two layers of the 8B shapes + its LM head: the capture-sized case for ncu (about 1 GB resident)
    "llama3-8b-2layers-ctx4096": (dict(n_layer=2, hidden=4096, n_head=32, n_kv_head=8, n_ff=14336, vocab=128256), 4096),
    # BASELINE config 4: Qwen3-30B-A3B shape, 128 experts top-8 (Q4_K), attention in Q6_K
    "qwen3-30b-a3b-moe-ctx8192": (dict(n_layer=48, hidden=2048, n_head=32, n_kv_head=4, n_ff=0, vocab=128256, n_expert=128, n_expert_used=8,
                                       n_ff_expert=768, rope_neox=1), 8192),
    # eight layers of the MoE shapes + its LM head: the capture-sized case for ncu (about 3 GB resident, 0.6 GB streamed per token)
    "qwen3-30b-a3b-moe-8layers-ctx8192": (dict(n_layer=8, hidden=2048, n_head=32, n_kv_head=4, n_ff=0, vocab=128256, n_expert=128, n_expert_used=8,
                                               n_ff_expert=768, rope_neox=1), 8192),
    "tiny-llama-ctx256": (dict(n_layer=2, hidden=512, n_head=4, n_kv_head=2, n_ff=1024, vocab=2048), 256),
}
DRAM_TRAFFIC_OVER_ALGORITHMIC = 459.77 / 456.19   # ncu, gemv_mma_kernel_1: LM head + q/k/v + o launches (profiles/gemv_mma_kernel_llama3-8b-2layers-ctx4096.md)
REPEATS = 5
METRIC = "decode_tok_per_s_batch1"
UNIT = "tok/s"


def row_bytes(t: int, cols: int) -> int:
    return {12: cols // 256 * 144, 14: cols // 256 * 210}[t]


def q8k_bytes(cols: int) -> int:
    return cols // 256 * 292


def algorithmic_bytes_per_token(shape: dict, ctx: int) -> dict:
    """Bytes one decode token must move (Q4_K_M convention: attn_v, ffn_down, LM head in
    Q6_K): weights once, the visible KV rows once, activations (Q8_K in, f32 out)."""
    H, qd, kvd, ff, V, L = shape["hidden"], shape["n_head"] * 128, shape["n_kv_head"] * 128, shape["n_ff"], shape["vocab"], shape["n_layer"]
    if shape.get("n_expert", 0):
        # attention in Q6_K, f32 router, the k routed experts' gate/up/down in Q4_K
        k, ffe = shape["n_expert_used"], shape["n_ff_expert"]
        mats = [(14, qd, H), (14, kvd, H), (14, kvd, H), (14, H, qd)] + [(12, ffe, H)] * (2 * k) + [(12, H, ffe)] * k
        w_layer = sum(r * row_bytes(t, c) for t, r, c in mats) + shape["n_expert"] * H * 4
    else:
        mats = [(12, qd, H), (12, kvd, H), (14, kvd, H), (12, H, qd), (12, ff, H), (12, ff, H), (14, H, ff)]
        w_layer = sum(r * row_bytes(t, c) for t, r, c in mats)
    act_layer = sum(q8k_bytes(c) + r * 4 for t, r, c in mats)
    w = L * w_layer + V * row_bytes(14, H) + row_bytes(12, H)   # + LM head + one embedding row
    act = L * act_layer + q8k_bytes(H) + V * 4
    kv = L * 2 * (ctx + 1) * kvd * 2
    return {"weights": w, "kv": kv, "activations": act, "total": w + kv + act}


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                p = [c.strip() for c in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx.append(float(p[2]))
                except ValueError:
                    continue
                for n, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle (restatement of rnb-cpu's x86 path) on a bounded sample of the workload.
# One "step" = the decode work of one layer (norms, Q8_K, q/k/v/o/gate/up/down matvecs, RoPE,
# f16 KV append, decode attention over the context) plus 1/n_layer of the LM head; a token is
# n_layer such steps, so tok/s = 1 / (n_layer * layer_time + lm_head_time).
# ------------------------------------------------------------------------------------------------
def _blocks(rng, t, rows, cols):
    if t == 12:
        w = rng.integers(0, 256, size=(rows, cols // 256, 144), dtype=np.uint8)
        d = np.abs(rng.standard_normal((rows, cols // 256, 2)) * 1e-3).astype(np.float16)
        w[:, :, 0:4] = d.view(np.uint8).reshape(rows, cols // 256, 4)
    else:
        w = rng.integers(0, 256, size=(rows, cols // 256, 210), dtype=np.uint8)
        d = (rng.standard_normal((rows, cols // 256, 1)) * 1e-3).astype(np.float16)
        w[:, :, 208:210] = d.view(np.uint8).reshape(rows, cols // 256, 2)
    return np.ascontiguousarray(w.reshape(-1))


class CpuSample:
    def __init__(self, shape: dict, ctx: int, seed: int = 0):
        import oracle as orc
        self.orc = orc
        orc.build()
        self.shape, self.ctx = shape, ctx
        self.threads = orc.n_threads()
        rng = np.random.default_rng(seed)
        H, qd, kvd, ff = shape["hidden"], shape["n_head"] * 128, shape["n_kv_head"] * 128, shape["n_ff"]
        self.mats = {n: (t, _blocks(rng, t, r, c), r, c) for n, t, r, c in (
            ("q", 12, qd, H), ("k", 12, kvd, H), ("v", 14, kvd, H), ("o", 12, H, qd),
            ("gate", 12, ff, H), ("up", 12, ff, H), ("down", 14, H, ff))}
        # LM head: a slice of the rows is timed and scaled (the full matrix is 0.4-0.9 GB)
        self.head_rows = min(shape["vocab"], 16384)
        self.head = _blocks(rng, 14, self.head_rows, H)
        self.x = rng.standard_normal(H).astype(np.float32)
        self.norm = np.ones(H, np.float32)
        self.k = rng.integers(0, 0x3C00, size=(ctx + 1) * kvd, dtype=np.uint16)
        self.v = rng.integers(0, 0x3C00, size=(ctx + 1) * kvd, dtype=np.uint16)

    def layer(self) -> float:
        orc, s, T = self.orc, self.shape, self.threads
        H, qd, kvd, ff = s["hidden"], s["n_head"] * 128, s["n_kv_head"] * 128, s["n_ff"]
        t0 = time.perf_counter()
        h = orc.rms_norm(self.x, self.norm, 1e-5)
        q = orc.gemv(*self.mats["q"][:2], h, qd, H, threads=T)
        k = orc.gemv(*self.mats["k"][:2], h, kvd, H, threads=T)
        v = orc.gemv(*self.mats["v"][:2], h, kvd, H, threads=T)
        q = orc.rope(q, self.ctx, 128, qd, 5e5)
        k = orc.rope(k, self.ctx, 128, kvd, 5e5)
        self.k[self.ctx * kvd:] = orc.f32_to_f16_bits(k)
        self.v[self.ctx * kvd:] = orc.f32_to_f16_bits(v)
        a = orc.attention_decode(q, self.k, self.v, s["n_head"], s["n_kv_head"], 128, self.ctx + 1,
                                 1.0 / np.sqrt(128.0), threads=T)
        x = self.x + orc.gemv(*self.mats["o"][:2], a, H, qd, threads=T)
        h = orc.rms_norm(x, self.norm, 1e-5)
        g = orc.gemv(*self.mats["gate"][:2], h, ff, H, threads=T)
        u = orc.gemv(*self.mats["up"][:2], h, ff, H, threads=T)
        act = orc.silu_mul(g, u)
        x = x + orc.gemv(*self.mats["down"][:2], act, H, ff, threads=T)
        return time.perf_counter() - t0

    def lm_head(self) -> float:
        t0 = time.perf_counter()
        self.orc.gemv(14, self.head, self.x, self.head_rows, self.shape["hidden"], threads=self.threads)
        return (time.perf_counter() - t0) * self.shape["vocab"] / self.head_rows

    def tok_per_s(self, layer_s: float, head_s: float) -> float:
        return 1.0 / (self.shape["n_layer"] * layer_s + head_s)

    def describe(self) -> str:
        return (f"one layer's decode work (7 matvecs on seeded uniform-quant blocks, RoPE, KV append, "
                f"attention over {self.ctx + 1} f16 KV rows) and {self.head_rows} LM-head rows, "
                f"scaled to {self.shape['n_layer']} layers + {self.shape['vocab']} vocab rows")


def cpu_baseline(shape, ctx, reps: int, warmup: int, min_seconds: float = 0.0):
    """Times the layer sample `reps` times, and keeps going until `min_seconds` of CPU work."""
    s = CpuSample(shape, ctx)
    for _ in range(max(warmup, 1)):
        s.layer()
    s.lm_head()
    layer = [s.layer() for _ in range(max(reps, 1))]
    while sum(layer) < min_seconds and len(layer) < 20000:
        layer.append(s.layer())
    head = [s.lm_head() for _ in range(3)]
    return s, layer, head


def run_reference(args, shape, ctx, name, rank, world):
    """`--impl reference`: rank 0 times the CPU path on all host threads; other ranks idle."""
    if rank != 0:
        return None
    s, layer, head = cpu_baseline(shape, ctx, args.steps, args.warmup)
    total = sum(layer)
    value = s.tok_per_s(total / len(layer), min(head))
    cb = {"value": value, "unit": UNIT, "cores": s.threads, "kind": "port", "sample": s.describe()}
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            # a step is one decode token: the timed layer sample scaled to the whole stack plus the LM head
            "warmup": args.warmup, "ms_per_step": 1000.0 / value, "ms_per_layer_sample": 1000.0 * total / len(layer), "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "int8xint4->int32, f32 accumulate",
            "data": "synthetic", "config": {"workload": name, "context": ctx, "kv_cache": "f16",
                                            "timed": "%d repetitions of one layer's decode work on the host CPU, scaled to %d layers + LM head" % (len(layer), shape["n_layer"])},
            "cpu_baseline": cb, "gpu_launches": 0,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 1400.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def prefill_gemm_bench(shape: dict, seq: int, reps: int = 3) -> dict:
    """Secondary measurement (BASELINE config 3): the seven matmuls of one 8B layer over `seq`
    tokens on the tcgen05 kernel, device-resident operands, CUDA events on torch's current stream
    (the kernel is launched on that stream).  Weights are random bytes with sane super-scales."""
    import ctypes as C

    import torch

    import runnburn_b200 as r
    L = r.load()
    H, qd, kvd, ff = shape["hidden"], shape["n_head"] * 128, shape["n_kv_head"] * 128, shape["n_ff"]
    # launches of a layer: (q, k, v) share the normed hidden state, (gate, up) likewise
    groups = [[(12, qd, H), (12, kvd, H), (14, kvd, H)], [(12, H, qd)], [(12, ff, H), (12, ff, H)], [(14, H, ff)]]
    g = torch.Generator(device="cuda").manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = load_peaks()
    rows_out, flops_total, ms_total = [], 0.0, 0.0
    for grp in groups:
        cols = grp[0][2]
        ws, ys = [], []
        for t, rows, _ in grp:
            blk = 144 if t == 12 else 210
            w = torch.randint(0, 256, (rows, cols // 256, blk), dtype=torch.uint8, device="cuda", generator=g)
            if t == 12:
                w[..., 1] = 0x10; w[..., 3] = 0x10      # f16 d, dmin ~ 5e-4
            else:
                w[..., 209] = 0x10
            ws.append(w)
            ys.append(torch.empty(seq, rows, device="cuda"))
        x = torch.randn(seq, cols, device="cuda", generator=g)
        xb = torch.empty(seq * cols, dtype=torch.int16, device="cuda")
        n = len(grp)
        types = (C.c_int * n)(*[t for t, _, _ in grp])
        wp = (C.c_void_p * n)(*[w.data_ptr() for w in ws])
        rws = (C.c_size_t * n)(*[r_ for _, r_, _ in grp])
        yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])

        # gate + up run as the prefill driver runs them: one launch whose epilogue writes silu(gate) * up as bf16
        fused = n == 2 and grp[0] == grp[1]
        act = torch.empty(seq, grp[0][1], dtype=torch.bfloat16, device="cuda") if fused else None

        def run():
            if fused:
                rc = L.rnb_b200_dev_prefill_gemm_silu(grp[0][0], ws[0].data_ptr(), ws[1].data_ptr(), grp[0][1], cols, x.data_ptr(), seq, xb.data_ptr(),
                                                      act.data_ptr(), stream)
            else:
                rc = L.rnb_b200_dev_prefill_gemm_multi(n, types, wp, rws, yp, cols, x.data_ptr(), seq, xb.data_ptr(), stream)
            if rc != 0:
                raise RuntimeError(L.rnb_b200_last_error().decode())
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        fl = sum(2.0 * r_ * cols * seq for _, r_, _ in grp)
        flops_total += fl
        ms_total += ms
        rows_out.append({"matrices": ["%s %dx%d" % ("Q4_K" if t == 12 else "Q6_K", r_, c_) for t, r_, c_ in grp], "ms": ms, "tflops": fl / ms / 1e9,
                         **({"epilogue": "silu(gate) * up -> bf16"} if fused else {})})
        del ws, ys, x, xb, act
    if r.ops.dev_error_flag() != 0:
        raise RuntimeError("device error flag set by the prefill matmul")
    tf = flops_total / ms_total / 1e9
    return {"workload": "llama3-8b layer matmuls, %d tokens" % seq, "tflops": tf, "peak_tflops": peaks["bf16_tflops"],
            "frac_of_bf16_peak": tf / peaks["bf16_tflops"], "frac_of_sustained_bf16_peak": tf / peaks["bf16_tflops_sustained"],
            "peak_source": peaks["source"], "ms_per_layer": ms_total, "includes": "f32->bf16 conversion of the tokens and in-kernel dequantisation",
            "launches": rows_out}


def moe_decode_bench(args) -> dict:
    """Secondary measurement (BASELINE config 2): batch-1 decode of the Qwen3-30B-A3B-shaped MoE stack
    (48 layers, 128 experts, top-8, context 8192) with device-resident token ids, CUDA events on the
    decoder's stream; median of REPEATS timed regions."""
    import runnburn_b200 as r
    name = "qwen3-30b-a3b-moe-ctx8192"
    shape, ctx = WORKLOADS[name]
    K, W = min(args.steps, 32), 3
    dec = r.Decoder(r.ModelConfig(max_ctx=ctx + (REPEATS + 1) * K + W + 8, **shape))
    dec.fill_synthetic(seed=0, sigma=0.02)
    dec.fill_kv_synthetic(ctx, seed=0)
    st = dec.stats()
    dec.step(1, ctx)
    dec.time_steps(ctx + 1, W)
    pos, all_ms = ctx + 1 + W, []
    for _ in range(REPEATS):
        all_ms.append(dec.time_steps(pos, K))
        pos += K
    dec.close()
    ms = float(np.median(all_ms))
    alg = algorithmic_bytes_per_token(shape, ctx)
    peaks = load_peaks()
    gbs = alg["total"] / (ms / K / 1000.0) / 1e9
    return {"workload": name, "value": K / (ms / 1000.0), "unit": UNIT, "ms_per_step": ms / K, "steps": K, "repeats": REPEATS,
            "launches_per_step": int(st["launches_per_step"]), "algorithmic_bytes_per_token": alg,
            "whole_step_hbm": {"achieved_gbs": gbs, "peak_gbs": peaks["hbm_gbs"], "frac": gbs / peaks["hbm_gbs"]},
            "what": "router matvec + top-8 + the 8 selected experts' gate/up/down streamed per layer, expert ids chosen on the device"}


def matvec_shape_bench(shapes=None, min_total_bytes=1 << 30, reps=5) -> list:
    """BASELINE config 1: each batch-1 matvec shape timed alone.  Every shape gets enough distinct
    weight copies to exceed 1 GiB (far more than the 126 MB L2), one launch per copy is captured
    into a CUDA graph, and the graph is replayed `reps` times between two CUDA events on the
    launching stream.  Bytes are the algorithmic ones: rows * row_bytes + Q8_K activation + f32 out."""
    import torch

    import runnburn_b200 as r
    L = r.load()
    shapes = shapes or [(12, 4096, 4096), (12, 1024, 4096), (12, 14336, 4096), (12, 4096, 14336), (14, 1024, 4096), (14, 4096, 14336), (14, 128256, 4096)]
    peaks = load_peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    out = []
    for t, rows, cols in shapes:
        rb = row_bytes(t, cols)
        wbytes = rows * rb
        n = max(2, -(-min_total_bytes // wbytes))
        blk = 144 if t == 12 else 210
        w = torch.randint(0, 256, (n, rows, cols // 256, blk), dtype=torch.uint8, device="cuda", generator=g)
        if t == 12:
            w[..., 1] = 0x10; w[..., 3] = 0x10      # f16 d, dmin ~ 5e-4
        else:
            w[..., 209] = 0x10
        x = torch.randn(cols, device="cuda", generator=g)
        xq = torch.empty(int(L.rnb_b200_dev_q8k_bytes(cols)) + 16, dtype=torch.uint8, device="cuda")
        y = torch.empty(n, rows, device="cuda")
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            sp = st.cuda_stream
            if L.rnb_b200_dev_quantize_q8k(x.data_ptr(), cols, 1, xq.data_ptr(), None, sp) != 0:
                raise RuntimeError(L.rnb_b200_last_error().decode())

            def run():
                for i in range(n):
                    if L.rnb_b200_dev_gemv(t, w[i].data_ptr(), rows, cols, xq.data_ptr(), y[i].data_ptr(), 0, sp) != 0:
                        raise RuntimeError(L.rnb_b200_last_error().decode())
            run()
            st.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                run()
            for _ in range(3):
                graph.replay()
            st.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for _ in range(reps):
                graph.replay()
            e1.record(st)
            st.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / (reps * n)
        alg = wbytes + q8k_bytes(cols) + rows * 4
        gbs = alg / us / 1e3
        out.append({"type": "Q4_K" if t == 12 else "Q6_K", "rows": rows, "cols": cols, "us": us, "algorithmic_bytes": alg, "gbs": gbs,
                    "frac": gbs / peaks["hbm_gbs"], "frac_of_8TBs_nominal": gbs / 8000.0, "copies": n})
        del w, y
        torch.cuda.empty_cache()
    if r.ops.dev_error_flag() != 0:
        raise RuntimeError("device error flag set by a matvec")
    return out


def run_gpu(args, shape, ctx, name, rank, world, local_rank):
    import torch

    os.environ["RNB_CUDA_DEVICE"] = str(local_rank)
    import runnburn_b200 as r
    from runnburn_b200 import build, ops
    from runnburn_b200.decoder import nccl_unique_id

    if rank == 0:
        build.build_library()
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
    ops.open()
    K, W = args.steps, args.warmup
    R = REPEATS                                   # the timed region runs R times; the median is reported
    max_ctx = ctx + (R + 1) * K + 2 * max(W, 3) + 8
    cfg = r.ModelConfig(max_ctx=max_ctx, world_size=world, rank=rank, **shape)
    dec = r.Decoder(cfg)
    # "peer": producers store their slices into the peers' buffers (measured: 11.3 against 12.1 ms per token at 4 GPUs);
    # "nccl": ncclAllGather (13.0 against 13.8 ms at 2 GPUs, where one peer makes the gather a single copy)
    transport = os.environ.get("RNB_B200_TRANSPORT", "nccl" if world == 2 else "peer")
    if world > 1 and transport == "nccl":
        ids = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        dec.attach_nccl(ids[0])
    elif world > 1:
        handles = [None] * world
        dist.all_gather_object(handles, dec.exchange_handle())
        dec.attach_peers(handles)
    dec.fill_synthetic(seed=0, sigma=0.02)
    dec.fill_kv_synthetic(ctx, seed=0)
    stats = dec.stats()

    def barrier():
        if dist is not None:
            dist.barrier()
        dec.sync()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def drive(d, sync, reduce_max):
        """The measured sequence on decoder `d`: K device-chained steps timed R times with CUDA events
        on the decoder's stream (token ids never leave the GPU), then K steps through the host-facing
        call (token id H2D, next id D2H, a sync per step) under a wall clock.  Returns the R step
        timings in ms, the end-to-end seconds and every token id the host-facing steps returned."""
        tok = d.step(1, ctx)                       # seeds the device-side token with a real argmax
        d.time_steps(ctx + 1, max(W, 3))           # warm-up
        pos = ctx + 1 + max(W, 3)
        all_ms = []
        for _ in range(R):
            sync()
            all_ms.append(reduce_max(d.time_steps(pos, K)))
            pos += K
        ids = []
        for i in range(max(W, 3)):
            tok = d.step(tok, pos + i)
            ids.append(int(tok))
        sync()
        t0 = time.perf_counter()
        for i in range(K):
            tok = d.step(tok, pos + max(W, 3) + i)
            ids.append(int(tok))
        sync()
        return all_ms, reduce_max(time.perf_counter() - t0), ids

    barrier()
    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
    all_ms, e2e_s, ids = drive(dec, barrier, max_over_ranks)
    clk = clocks.stop() if rank == 0 else None
    ms = float(np.median(all_ms))

    # -- N > 1: the same model unsharded on rank 0's GPU (the synthetic fill gives a row shard the bytes
    # the whole matrix has there), driven through the same sequence: its ids must equal the sharded run's,
    # and its timing is the 1-GPU base that the N-GPU figure scales from
    def short_ids(d):
        """24 greedy steps from an empty context.  Contexts this short run the reference-order attention
        kernel, so a sharded step and the unsharded one are the same arithmetic in the same order: the ids
        must be identical (at the benchmark's long context the chunk counts differ with the number of KV
        heads per GPU, and nearly flat random-init logits turn 1e-6 attention differences into other ids)."""
        tok, out = 1, []
        for pos in range(24):
            tok = d.step(tok, pos)
            out.append(int(tok))
        return out

    shard = None
    if world > 1:
        s_ids = short_ids(dec)
        mine = [None] * world
        dist.all_gather_object(mine, (ids, s_ids))
        shard = {"ranks_agree": all(m == mine[0] for m in mine)}
        if rank == 0 and not args.no_scaling_base:
            try:
                base = r.Decoder(r.ModelConfig(max_ctx=max_ctx, world_size=1, rank=0, **shape))
                base.fill_synthetic(seed=0, sigma=0.02)
                base.fill_kv_synthetic(ctx, seed=0)

                def base_sync():
                    base.sync()
                b_ms, b_e2e, b_ids = drive(base, base_sync, float)
                b_short = short_ids(base)
                base.close()
                bm = float(np.median(b_ms))
                shard["ids_equal"] = b_short == s_ids
                shard["n_ids"] = len(s_ids)
                shard["what"] = "24 greedy ids from an empty context, sharded run against the same model unsharded on one GPU (reference-order attention: same arithmetic)"
                shard["long_context_ids_equal"] = b_ids == ids
                shard["base"] = {"workload": name, "n_gpus": 1, "value": K / (bm / 1000.0), "unit": UNIT, "ms_per_step": bm / K,
                                 "e2e": K / b_e2e, "what": "the same model unsharded on one GPU of this box, same steps"}
            except Exception as e:   # the base must not lose the headline line
                shard["base_error"] = str(e)[:200]
        barrier()

    # -- dominant kernel: every matvec launch of a step, timed alone over the model's own weights
    mv = dec.time_matvecs(iters=max(3, min(K, 16))) if shape.get("n_expert", 0) == 0 else None
    barrier()
    if rank != 0:
        dec.close()
        dist.destroy_process_group()
        return None
    peaks = load_peaks()
    alg = algorithmic_bytes_per_token(shape, ctx)
    value = K / (ms / 1000.0)
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": max(W, 3),
        "ms_per_step": ms / K, "repeats": R, "ms_per_step_all": [m / K for m in all_ms], "timing": "median of %d timed regions of %d steps each, max over ranks per region" % (R, K),
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "int8xint4->int32, f32 accumulate", "data": "synthetic",
        "config": {"workload": name, "context": ctx, "kv_cache": "f16", "weights": ("random-init N(0,0.02): attention and LM head Q6_K, f32 router, experts Q4_K, generated on device" if shape.get("n_expert", 0) else "random-init N(0,0.02), Q4_K_M layout (attn_v/ffn_down/output Q6_K), generated on device"),
                   "parallelism": (f"row-sharded x{world}, all-gather by " + ("ncclAllGather" if transport == "nccl" else "peer-memory stores over NVLink from the producing kernels' epilogues, consumers wait on arrival flags (no exchange launch)")) if world > 1 else "single GPU",
                   "l2": "each step streams its whole weight set and KV cache (GBs), far more than the 126 MB L2: no flush needed",
                   "algorithmic_bytes_per_token": alg},
        "e2e": {"value": K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "gpu_launches": int(stats["launches_per_step"]) * K,
        "clocks": clk,
        "whole_step_hbm": {"achieved_gbs": alg["total"] / world / (ms / K / 1000.0) / 1e9, "peak_gbs": peaks["hbm_gbs"],
                           "frac": alg["total"] / world / (ms / K / 1000.0) / 1e9 / peaks["hbm_gbs"]},
    }
    if shard is not None:
        out["shard_ids_equal"] = bool(shard.get("ids_equal", False)) and shard["ranks_agree"]
        out["shard_check"] = {k: v for k, v in shard.items() if k != "base"}
        if "base" in shard:
            out["scaling_base"] = shard["base"]
    if mv:
        per_launch_bytes = mv["bytes_per_iter"] / mv["launches_per_iter"]
        per_launch_s = mv["ms"] / 1000.0 / (mv["iters"] * mv["launches_per_iter"])
        ach = per_launch_bytes / per_launch_s / 1e9
        out["roofline"] = {"kernel": "gemv_mma_kernel_1 (q/k/v, o, down, LM head: integer tensor-core matvec) and gemv_pair_q4k_kernel (gate/up)", "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                           "frac": ach / peaks["hbm_gbs"], "frac_of_8TBs_nominal": ach / 8000.0, "peak_source": peaks["source"],
                           # DRAM read+write bytes per launch: the ncu capture of three matvec launches (LM head, q/k/v, o)
                           # gave 459.8 MB of traffic for 456.2 MB of algorithmic bytes (summary under profiles/)
                           "traffic": per_launch_bytes * DRAM_TRAFFIC_OVER_ALGORITHMIC,
                           "traffic_source": "ncu dram__bytes_read.sum+dram__bytes_write.sum of three launches of gemv_mma_kernel_1 (LM head, q/k/v, o), scaled by algorithmic bytes",
                           "launches_per_step": mv["launches_per_iter"],
                           "algorithmic_bytes_per_launch": per_launch_bytes, "avg_launch_us": per_launch_s * 1e6,
                           "how": "CUDA events around all matvec launches of a step on the decoder stream, model's own weights"}
    if world == 1 and shape.get("n_expert", 0) == 0 and not args.no_prefill:
        # secondary measurement (BASELINE config 3): prefill of a 2048-token random prompt through the
        # decoder's tensor-core path, device time between two events on the decoder's stream
        try:
            n_tok = min(2048, ctx)
            ids = np.random.default_rng(0).integers(0, shape["vocab"], n_tok).astype(np.uint32)
            dec.prefill(ids, 0, timed=True)
            _, pms = dec.prefill(ids, 0, timed=True)
            out["prefill"] = {"tokens": int(n_tok), "ms": pms, "tok_per_s": n_tok / (pms / 1000.0),
                              "what": "embed, 32 x (RMSNorm, q/k/v matmul, RoPE + f16 KV append, causal attention, o_proj, RMSNorm, gate/up, SiLU*up, down), "
                                      "final norm + LM head + argmax of the last token; matmuls on tcgen05 (bf16), causal attention on mma.sync tensor cores (split-f16 operands, fp32 accumulate)"}
        except Exception as e:   # a secondary figure must not lose the headline line
            out["prefill"] = {"error": str(e)[:200]}
    dec.close()
    if dist is not None:
        dist.destroy_process_group()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary prefill-matmul measurement")
    ap.add_argument("--no-per-shape", action="store_true", help="skip the per-shape matvec table of the roofline block")
    ap.add_argument("--no-moe", action="store_true", help="skip the secondary MoE decode measurement")
    ap.add_argument("--no-scaling-base", action="store_true", help="N > 1: skip the unsharded 1-GPU run of the same model")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    name = args.workload or ("llama3-8b-q4km-ctx4096" if args.gpus == 1 else "llama3-70b-q4km-ctx32768")
    shape, ctx = WORKLOADS[name]
    if args.impl == "reference":
        out = run_reference(args, shape, ctx, name, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return
    if world == 1 and args.gpus > 1:
        sys.stderr.write("bench.py --gpus N>1 must be launched with torch.distributed.run (one rank per GPU)\n")
        sys.exit(2)
    out = run_gpu(args, shape, ctx, name, rank, world, local_rank)
    if out is None:
        return
    if world == 1 and shape.get("hidden") == 4096 and not args.no_prefill:
        try:
            out["prefill_gemm"] = prefill_gemm_bench(shape, 2048)
        except Exception as e:   # a secondary figure must not lose the headline line
            out["prefill_gemm"] = {"error": str(e)[:200]}
    if world == 1 and "roofline" in out and not args.no_per_shape:
        # BASELINE config 1: the layer's and the LM head's matvec shapes each timed alone
        try:
            ps = matvec_shape_bench([(12, 4096, 4096), (12, 14336, 4096), (12, 4096, 14336), (14, 1024, 4096), (14, 4096, 14336), (14, 128256, 4096)]
                                    if shape.get("hidden") == 4096 else None)
            out["roofline"]["per_shape"] = ps
            out["roofline"]["per_shape_mean_frac"] = float(np.mean([p_["frac"] for p_ in ps]))
            out["roofline"]["per_shape_how"] = ("each shape alone: enough distinct weight copies to exceed 1 GiB, one launch per copy in a CUDA graph, "
                                                "graph replayed between two CUDA events on the launching stream; algorithmic bytes = rows * row_bytes + Q8_K activation + f32 out")
        except Exception as e:
            out["roofline"]["per_shape"] = {"error": str(e)[:200]}
    if world == 1 and args.workload is None and not args.no_moe:
        # BASELINE config 2 as a secondary figure of the default line: Qwen3-30B-A3B-shaped MoE decode
        try:
            out["moe"] = moe_decode_bench(args)
        except Exception as e:
            out["moe"] = {"error": str(e)[:200]}
    if world == 1 and not args.no_cpu_baseline:
        s, layer, head = cpu_baseline(shape, ctx, reps=5, warmup=1, min_seconds=10.0)   # about 10 s of CPU work
        out["cpu_baseline"] = {"value": s.tok_per_s(min(layer), min(head)), "unit": UNIT, "cores": s.threads, "kind": "port",
                               "sample": s.describe() + "; %d repetitions, %.1f s of CPU time, best repetition used" % (len(layer), sum(layer))}
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
