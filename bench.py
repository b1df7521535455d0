#!/usr/bin/env python
"""Benchmark of the paged-KV batched decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1 and every rank at N>1): a Llama-3-8B-shaped model with random weights — 32 layers, d_model 4096,
32 query x 128 / 8 KV heads, SwiGLU FFN 14336, vocabulary 128256, RoPE theta 500000; projections and head
~N(0, 0.02) quantized to Q4_0 (token embedding and norms f32); f16 paged KV with 16-token pages; batch 32 prompts of
512 random token ids (fed one token per step through the decode path), then greedy decode. One "step" is one
decode step of the whole batch (32 tokens). All inputs are synthetic (seeded); there is no dataset.

Printed JSON line (rank 0):
  value     decode tokens/s with ids, tables and weights resident in HBM: K steps replayed as one CUDA graph per step
            (etc_decoder_generate_greedy), timed with CUDA events, max over ranks
  e2e       the same metric through the reference-facing call (Executable.executeSampled): every step copies the
            step's token ids / lane descriptors / page tables host->device and reads the sampled tokens back
  roofline  the dominant kernel (tcgen05 Q4_0 linear, fused gate/up shape [28672 x 4096], 32 vectors) timed alone with
            CUDA events on the launching stream (graph replays) over weight sets larger than L2
  cpu_baseline  the CPU oracle (restatement of the reference CPU backend) on a bounded sample, host cores stated
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = dict(layers=32, d_model=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256, rms_eps=1e-5,
             rope_theta=500000.0)
BATCH, PROMPT, BLOCK = 32, 512, 16
Q4_0 = 2
METRIC = "decode tokens/s, Llama-3-8B-shape Q4_0 batch 32; kernel HBM GB/s vs peak"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def algorithmic_bytes_per_step(model, batch, mean_ctx):
    """Weights read once per step + KV read once per KV head per step (bytes)."""
    d, qw, kvw, ffn, V, L = (model["d_model"], model["q_heads"] * model["head_dim"], model["kv_heads"] * model["head_dim"],
                             model["ffn"], model["vocab"], model["layers"])
    per_layer = (qw + 2 * kvw) * d + d * qw + 2 * ffn * d + d * ffn
    weights = (L * per_layer + V * d) * 18 / 32
    kv = batch * mean_ctx * L * 2 * kvw * 2
    return weights + kv


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU reference arm
def cpu_sample(model, batch, ctx, threads, fraction, seed=3):
    """Times the CPU oracle on a bounded sample of one decode step and scales it to the whole step.

    Every projection of one layer and the head are timed on a row slice (`fraction` of the rows, all columns,
    all `batch` vectors); paged attention is timed on `fraction` of the lanes at context `ctx`; norms, RoPE and
    SwiGLU are timed at full size. Slice times are divided by their fraction and the layer time is multiplied by
    the layer count. Returns (tokens/s, seconds of CPU work done, description)."""
    import oracle as orc
    rng = np.random.default_rng(seed)
    d, qw, kvw, ffn, V, L = (model["d_model"], model["q_heads"] * model["head_dim"], model["kv_heads"] * model["head_dim"],
                             model["ffn"], model["vocab"], model["layers"])
    work = 0.0

    def linear_seconds(rows, cols):
        nonlocal work
        r = min(rows, max(32, int(rows * fraction) // 32 * 32))
        w = rng.standard_normal((r, cols), dtype=np.float32) * np.float32(0.02)
        packed = orc.quantize(orc.Q4_0, w)
        x = rng.standard_normal((batch, cols), dtype=np.float32)
        t0 = time.perf_counter()
        orc.qlinear(orc.Q4_0, x, packed, r, cols, threads=threads)
        dt = time.perf_counter() - t0
        work += dt
        return dt * rows / r

    layer = sum(linear_seconds(r, c) for r, c in ((qw, d), (kvw, d), (kvw, d), (d, qw), (ffn, d), (ffn, d), (d, ffn)))
    head = linear_seconds(V, d)
    lanes = max(1, int(round(batch * fraction)))
    max_tokens = lanes * ((ctx + 1 + BLOCK - 1) // BLOCK) * BLOCK
    pool = orc.Pool(1, model["kv_heads"], model["head_dim"], max_tokens, BLOCK, orc.F16)
    seqs = [pool.make_sequence() for _ in range(lanes)]
    for s_ in seqs:  # context written straight into the pages: the prefill is not part of the decode sample
        for _ in range((ctx + BLOCK - 1) // BLOCK):
            s_.push_block(pool.alloc_block())
        rows = np.concatenate([np.arange(BLOCK) + int(b) * BLOCK for b in s_.blocks])[:ctx]
        pool.write_rows(0, 0, rows, rng.standard_normal((ctx, kvw), dtype=np.float32))
        pool.write_rows(0, 1, rows, rng.standard_normal((ctx, kvw), dtype=np.float32))
        s_.set_cursor(ctx)
        s_.set_advance(1)
    q = rng.standard_normal((lanes, model["q_heads"], 1, model["head_dim"]), dtype=np.float32)
    k = rng.standard_normal((lanes, model["kv_heads"], 1, model["head_dim"]), dtype=np.float32)
    t0 = time.perf_counter()
    orc.kv_attention(pool, 0, seqs, lanes, q, k, k, 1.0 / np.sqrt(model["head_dim"]), mode=1, threads=threads)
    dt = time.perf_counter() - t0
    work += dt
    layer += dt * batch / lanes
    h = rng.standard_normal((batch, d), dtype=np.float32)
    g = rng.standard_normal((batch, ffn), dtype=np.float32)
    t0 = time.perf_counter()
    orc.rms_norm(h, np.ones(d, np.float32), model["rms_eps"])
    orc.rms_norm(h, np.ones(d, np.float32), model["rms_eps"])
    orc.rotary(rng.standard_normal((batch, model["q_heads"] + model["kv_heads"], 1, model["head_dim"]), dtype=np.float32),
               np.full(batch, ctx), model["rope_theta"])
    orc.silu_mul(g, g)
    dt = time.perf_counter() - t0
    work += dt
    layer += dt
    step_seconds = layer * L + head
    sample = (f"one batch-{batch} decode step at context {ctx} of the CPU oracle (restatement of the reference CPU backend; fair "
              f"variant: every block decoded once per row, attention scores cached) on {threads} threads: {fraction:.4f} of the "
              f"rows of each projection and of the lanes of paged attention in 1 of {L} layers, plus the head slice, scaled to "
              f"the full step (extrapolated)")
    return batch / step_seconds, work, sample


def calibrated_fraction(model, batch, threads, budget_seconds):
    """Fraction of one layer's rows whose CPU time fits `budget_seconds` (probed on a 1/64 slice)."""
    _, work, _ = cpu_sample(model, batch, PROMPT, threads, 1.0 / 64)
    return float(min(1.0, max(1.0 / 256, (1.0 / 64) * budget_seconds / max(work, 1e-6))))


def run_reference_arm(args, rank):
    if rank != 0:
        return
    import oracle as orc
    threads = orc.max_threads()
    total = args.warmup + args.steps
    fraction = calibrated_fraction(MODEL, BATCH, threads, 150.0 / max(total, 1))
    values, sample = [], ""
    for i in range(total):
        v, _, sample = cpu_sample(MODEL, BATCH, PROMPT + i, threads, fraction, seed=3 + i)
        if i >= args.warmup:
            values.append(v)
    value = float(np.mean(values))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * BATCH / value, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "llama3-8b-shape Q4_0 paged decode, batch 32, prompt 512 (bounded CPU sample per step)",
                   "global_batch": BATCH, "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def build_decoder(rt, et, torch, model, batch, max_tokens, seed, shared_seed=None):
    """Random-init weights of the model's shape. `shared_seed`: tensors that tensor-parallel ranks replicate (embedding,
    head) are drawn from it so that every rank holds the same values; the projections are this rank's own shard."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    shared = gen
    if shared_seed is not None:
        shared = torch.Generator(device="cuda")
        shared.manual_seed(shared_seed)
    dec = et.Executable(rt, layers=model["layers"], d_model=model["d_model"], q_heads=model["q_heads"], kv_heads=model["kv_heads"],
                        head_dim=model["head_dim"], ffn=model["ffn"], vocab=model["vocab"], rms_eps=model["rms_eps"],
                        rope_theta=model["rope_theta"], batch=batch, max_tokens=max_tokens, block_size=BLOCK, kv_dtype=et.KV_F16,
                        exact=False, max_advance=1)
    d, qw, kvw, ffn, V = (model["d_model"], model["q_heads"] * model["head_dim"], model["kv_heads"] * model["head_dim"], model["ffn"],
                          model["vocab"])

    def normal(rows, cols, g=None):
        w = torch.randn((rows, cols), generator=g or gen, device="cuda", dtype=torch.float32)
        w.mul_(0.02)
        return w

    def quantized(rows, cols, g=None):
        w = normal(rows, cols, g)
        packed = torch.empty((rows, cols // 32 * 18), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        rt.quantize_into(Q4_0, w, rows, cols, packed)
        rt.synchronize()
        return packed

    def bind(slot, layer, tensor, codec=0, rows=None, cols=None):
        torch.cuda.synchronize()
        dec.set_weight(slot, layer, tensor, codec=codec, rows=rows, columns=cols)

    bind(et.W_TOK_EMBD, 0, normal(V, d, shared))
    ones = torch.ones(d, device="cuda", dtype=torch.float32)
    for l in range(model["layers"]):
        bind(et.W_ATTN_NORM, l, ones)
        bind(et.W_FFN_NORM, l, ones)
        for slot, (r, c) in ((et.W_Q, (qw, d)), (et.W_K, (kvw, d)), (et.W_V, (kvw, d)), (et.W_O, (d, qw)), (et.W_GATE, (ffn, d)),
                             (et.W_UP, (ffn, d)), (et.W_DOWN, (d, ffn))):
            bind(slot, l, quantized(r, c), Q4_0, r, c)
    bind(et.W_OUT_NORM, 0, ones)
    bind(et.W_HEAD, 0, quantized(V, d, shared), Q4_0, V, d)
    dec.finalize()
    torch.cuda.empty_cache()
    return dec


def time_dominant_kernel(rt, et, torch, model, vectors, iters=40):
    """The fused gate/up linear [2*ffn x d_model] at `vectors` input rows, alone, over more weight copies than L2 holds."""
    d, ffn = model["d_model"], model["ffn"]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    copies = []
    for _ in range(4):  # 4 x 66 MB > 126 MB L2
        parts = []
        for _ in range(2):
            w = torch.randn((ffn, d), generator=gen, device="cuda", dtype=torch.float32) * 0.02
            packed = torch.empty((ffn, d // 32 * 18), dtype=torch.uint8, device="cuda")
            torch.cuda.synchronize()
            rt.quantize_into(Q4_0, w, ffn, d, packed)
            rt.synchronize()
            parts.append(packed)
        copies.append(et.QWeight(rt, Q4_0, parts, [ffn, ffn], d, interleave8=True))
        del parts
    x = torch.randn((vectors, d), device="cuda", dtype=torch.float32)
    out = torch.empty((vectors, ffn), device="cuda", dtype=torch.float32)
    scratch_bytes = copies[0].scratch_bytes(vectors)
    scratch = torch.empty(max(scratch_bytes, 4), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(rt.stream)
    for i in range(8):
        copies[i % 4].linear_into(x, vectors, out, epilogue=et.EPILOGUE_SWIGLU, scratch=scratch, scratch_bytes=scratch_bytes)
    rt.synchronize()
    # a Python launch loop is slower than the kernel: capture the launches once and time replays of the graph
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(iters):
            copies[i % 4].linear_into(x, vectors, out, epilogue=et.EPILOGUE_SWIGLU, scratch=scratch, scratch_bytes=scratch_bytes)
    with torch.cuda.stream(stream):
        graph.replay()
        start.record()
        graph.replay()
        graph.replay()
        stop.record()
    rt.synchronize()
    ms = start.elapsed_time(stop) / (2 * iters)
    algorithmic = 2 * ffn * (d // 32) * 18 + 4 * vectors * d + 4 * vectors * ffn
    for c in copies:
        c.close()
    return ms, algorithmic


def run_attention_microbench(args):
    """Paged-attention decode alone (the survey's microbench shape): 64 sequences, 32 query / 8 KV heads of 128, f16 pool of
    65 536 pages x 16 tokens, contexts ~U[128, 4096] (rounded to 64), one query token per sequence. Prints one JSON line."""
    import torch
    import effect_torch_b200 as et

    torch.cuda.set_device(0)
    rt = et.Runtime(0)
    B, Hq, Hkv, D, pages = 64, 32, 8, 128, 65536
    rng = np.random.default_rng(1)
    ctx = np.sort((rng.integers(128, 4097, size=B) // 64) * 64)[::-1].copy()
    pool = et.NativeKvPool(rt, 1, Hkv, D, pages * BLOCK, BLOCK, et.KV_F16)
    seqs = [pool.makeSequence() for _ in range(B)]
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    chunk = 64
    kv = torch.randn((B, Hkv, chunk, D), generator=gen, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    filler = np.arange(chunk, dtype=np.uint32)
    for start in range(0, int(ctx.max()), chunk):  # sequences are sorted by length: the first `active` still grow
        active = int((ctx > start).sum())
        rt.kv_append_into(pool, 0, seqs[:active], B, active, chunk, kv, kv, chunk)
        for s in seqs[:active]:
            s.commit(filler)
    q = torch.randn((B, Hq, D), generator=gen, device="cuda", dtype=torch.float32)
    k1 = torch.randn((B, Hkv, D), generator=gen, device="cuda", dtype=torch.float32)
    out = torch.empty((B, Hq, D), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    scale = 1.0 / np.sqrt(D)
    stream = torch.cuda.ExternalStream(rt.stream)
    start_ev, stop_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(0)
    for _ in range(max(args.warmup, 3)):
        rt.kv_attention_decode_into(pool, 0, seqs, B, B, q, k1, k1, Hq, scale, out=out)
    rt.synchronize()
    sampler.start()
    iters = max(args.steps, 20)
    with torch.cuda.stream(stream):
        start_ev.record()
        for _ in range(iters):
            rt.kv_attention_decode_into(pool, 0, seqs, B, B, q, k1, k1, Hq, scale, out=out)
        stop_ev.record()
    rt.synchronize()
    clocks = sampler.stop()
    ms = start_ev.elapsed_time(stop_ev) / iters
    total_ctx = int(ctx.sum()) + B
    algorithmic = total_ctx * 2 * Hkv * D * 2 + B * Hq * D * 8 + 4 * int(np.ceil((ctx + 1) / BLOCK).sum())
    peaks, peak_kind = measured_peaks()
    achieved = algorithmic / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "paged attention decode, HBM GB/s vs peak", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": iters,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f16 KV, f16 MMA operands, f32 softmax/accumulate",
        "data": "synthetic", "config": {"workload": f"paged attention microbench: {B} sequences, {Hq} query / {Hkv} KV heads x {D}, contexts "
                                                    f"{int(ctx.min())}..{int(ctx.max())} (sum {total_ctx}), {pages} pages x {BLOCK} tokens, "
                                                    "each step appends one token per sequence (host lane/table upload included) and attends",
                                        "l2": f"KV read per step {algorithmic / 1e6:.0f} MB exceeds the 126 MB L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "traffic": None, "peak_kind": peak_kind, "kernel": "attention_mma_kernel<128,f16> + merge + kv append",
                     "algorithmic_bytes_per_launch": algorithmic},
        "clocks": clocks}), flush=True)


def run_linear_microbench(args):
    """The quantized-matmul microbench shapes: Q4_0 and Q8_0, [4096x4096], [14336x4096], [4096x14336], 1 / 8 / 64 / 512 input
    vectors, each timed through graph replays over enough weight copies to exceed L2. One JSON line with a table."""
    import torch
    import effect_torch_b200 as et

    torch.cuda.set_device(0)
    rt = et.Runtime(0)
    peaks, peak_kind = measured_peaks()
    rows_out = []
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2)
    stream = torch.cuda.ExternalStream(rt.stream)
    for codec, bb, name in ((Q4_0, 18, "Q4_0"), (8, 34, "Q8_0")):
        for n, k in ((4096, 4096), (14336, 4096), (4096, 14336)):
            packed_bytes = n * (k // 32) * bb
            copies = max(2, int(np.ceil(300e6 / packed_bytes)))
            weights = []
            for _ in range(copies):
                w = torch.randn((n, k), generator=gen, device="cuda", dtype=torch.float32) * 0.02
                p = torch.empty((n, k // 32 * bb), dtype=torch.uint8, device="cuda")
                torch.cuda.synchronize()
                rt.quantize_into(codec, w, n, k, p)
                rt.synchronize()
                weights.append(et.QWeight(rt, codec, [p], [n], k))
                del w, p
            for m in (1, 8, 64, 512):
                x = torch.randn((m, k), generator=gen, device="cuda", dtype=torch.float32)
                out = torch.empty((m, n), device="cuda", dtype=torch.float32)
                need = weights[0].scratch_bytes(m)
                scratch = torch.empty(max(need, 4), dtype=torch.uint8, device="cuda")
                torch.cuda.synchronize()
                for i in range(copies):
                    weights[i].linear_into(x, m, out, scratch=scratch, scratch_bytes=need)
                rt.synchronize()
                iters = 2 * copies
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(iters):
                        weights[i % copies].linear_into(x, m, out, scratch=scratch, scratch_bytes=need)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(stream):
                    graph.replay()
                    a.record()
                    graph.replay()
                    graph.replay()
                    b.record()
                rt.synchronize()
                us = a.elapsed_time(b) / (2 * iters) * 1e3
                algorithmic = packed_bytes + 4 * m * k + 4 * m * n
                flops = 2.0 * m * n * k
                rows_out.append({"codec": name, "rows": n, "columns": k, "vectors": m, "us": us, "gbs": algorithmic / us / 1e3,
                                 "hbm_frac": algorithmic / us / 1e3 / peaks["hbm_gbs"], "tflops": flops / us / 1e6})
                del graph
            for w in weights:
                w.close()
            torch.cuda.empty_cache()
    print(json.dumps({"metric": "quantized linear microbench, HBM GB/s and TFLOP/s per shape", "unit": "GB/s", "n_gpus": 1,
                      "data": "synthetic", "config": {"workload": "tcgen05 dequant linear, graph replays over > 300 MB of weight copies per shape"},
                      "peak": peaks, "peak_kind": peak_kind, "table": rows_out}), flush=True)


MODEL_70B = dict(layers=80, d_model=8192, q_heads=64, kv_heads=8, head_dim=128, ffn=28672, vocab=128256, rms_eps=1e-5,
                 rope_theta=500000.0)


def run_tp_70b(args, rank, world):
    """Llama-3-70B-shape Q4_0 decode, batch 64, contexts ~U[1024, 8192], tensor parallel over `world` ranks. KV is written
    straight into the pages (N(0,1) rows; a decode benchmark needs no real prefill) and the steps run device-resident."""
    import torch
    import torch.distributed as dist
    import effect_torch_b200 as et
    from effect_torch_b200 import tensor_parallel

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rt = et.Runtime(local)
    full = dict(MODEL_70B)
    if args.layers:
        full["layers"] = args.layers
    model = tensor_parallel.local_config(full, world)
    B, K, W, chunk = 64, args.steps, args.warmup, 256
    rng = np.random.default_rng(4)  # the same contexts and tokens on every rank
    ctx = np.sort((rng.integers(1024, 8193, size=B) // chunk) * chunk)[::-1].copy()
    per_seq = ((int(ctx.max()) + W + K + BLOCK) // BLOCK + 1) * BLOCK
    max_tokens = ((int(ctx.sum()) + B * (W + K + 2 * BLOCK)) // BLOCK + B) * BLOCK
    dec = build_decoder(rt, et, torch, model, B, max_tokens, seed=40 + rank, shared_seed=4)
    if world > 1:
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            ident = torch.frombuffer(bytearray(et.tensor_parallel_id()), dtype=torch.uint8).cuda()
        dist.broadcast(ident, src=0)
        dec.set_tensor_parallel(rank, world, bytes(ident.cpu().tolist()))
        if args.tp_allreduce == "peer":
            mine = torch.frombuffer(bytearray(dec.peer_exchange_handle()), dtype=torch.uint8).cuda()
            table = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(table, mine)
            dec.use_peer_allreduce([bytes(t.cpu().tolist()) for t in table])
    pool = et.NativeKvPool(rt, model["layers"], model["kv_heads"], model["head_dim"], max_tokens, BLOCK, et.KV_F16)
    seqs = [pool.makeSequence() for _ in range(B)]
    kv = torch.randn((B, model["kv_heads"], chunk, model["head_dim"]), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    filler = np.arange(chunk, dtype=np.uint32)
    for start in range(0, int(ctx.max()), chunk):  # sorted by length: the first `active` sequences still grow
        active = int((ctx > start).sum())
        for layer in range(model["layers"]):
            rt.kv_append_into(pool, layer, seqs[:active], B, active, chunk, kv, kv, chunk)
        for s in seqs[:active]:
            s.commit(filler)
    del kv
    tok = rng.integers(0, full["vocab"], size=B).astype(np.uint32)
    sampler = ClockSampler(local)
    if W:
        out, _ = dec.generate_greedy(pool, seqs, tok, W)
        tok = out[-1]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    out, device_ms = dec.generate_greedy(pool, seqs, tok, K)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    times = torch.tensor([device_ms / 1000.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        mine = torch.from_numpy(out.astype(np.int64)).cuda()
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not torch.equal(lo, hi):
            raise RuntimeError("tensor-parallel ranks generated different tokens")
    seconds = float(times.cpu()[0])
    if rank == 0:
        mean_ctx = float(ctx.mean()) + W + (K + 1) / 2.0
        step_bytes = algorithmic_bytes_per_step(full, B, mean_ctx)
        peaks, peak_kind = measured_peaks()
        print(json.dumps({
            "metric": "decode tokens/s, Llama-3-70B-shape Q4_0 batch 64, tensor parallel", "value": B * K / seconds, "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": 1000.0 * seconds / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 MMA operands, f32 accumulate (Q4_0 weights, f16 KV)", "data": "synthetic",
            "config": {"workload": f"llama3-70b-shape Q4_0 paged decode: {full['layers']} layers, batch {B}, contexts {int(ctx.min())}.."
                                   f"{int(ctx.max())} (mean {ctx.mean():.0f}) written directly into the pages, {K} greedy steps",
                       "global_batch": B, "parallelism": f"tp{world}, {args.tp_allreduce if world > 1 else 'no'} all-reduce, head replicated"},
            "gpu_launches": dec.diagnostics()["launches_per_step"] * K,
            "step_roofline": {"algorithmic_bytes_per_step_all_ranks": step_bytes, "achieved_gbs_per_rank": step_bytes / world * K / seconds / 1e9,
                              "frac_of_" + peak_kind: step_bytes / world * K / seconds / 1e9 / peaks["hbm_gbs"]},
            "clocks": clocks}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_gpu_arm(args, rank, world):
    import torch
    import torch.distributed as dist
    import effect_torch_b200 as et

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rt = et.Runtime(local)
    model = dict(MODEL)
    if args.layers:
        model["layers"] = args.layers
    # N > 1: independent replicas by default; --parallelism tp cuts one model over the ranks (an all-reduce after the o
    # and down projections)
    tp = world > 1 and args.parallelism == "tp"
    if tp:
        from effect_torch_b200 import tensor_parallel
        model = tensor_parallel.local_config(model, world)  # this rank's share of heads and ffn
    K, W = args.steps, args.warmup
    # every sequence: prompt + warm-up + timed steps, twice (end-to-end leg, then device-resident leg)
    per_seq = ((PROMPT + W + K + BLOCK) // BLOCK + 1) * BLOCK
    max_tokens = 2 * BATCH * per_seq
    dec = build_decoder(rt, et, torch, model, BATCH, max_tokens, seed=3 + rank, shared_seed=3 if tp else None)
    if tp:
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            ident = torch.frombuffer(bytearray(et.tensor_parallel_id()), dtype=torch.uint8).cuda()
        dist.broadcast(ident, src=0)
        dec.set_tensor_parallel(rank, world, bytes(ident.cpu().tolist()))
        if args.tp_allreduce == "peer":  # one-shot kernel over peer memory instead of NCCL
            mine = torch.frombuffer(bytearray(dec.peer_exchange_handle()), dtype=torch.uint8).cuda()
            table = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(table, mine)
            dec.use_peer_allreduce([bytes(t.cpu().tolist()) for t in table])
    pool = et.NativeKvPool(rt, model["layers"], model["kv_heads"], model["head_dim"], max_tokens, BLOCK, et.KV_F16)
    rng = np.random.default_rng(3 if tp else 3 + rank)  # tensor-parallel ranks decode the same sequences
    prompts = rng.integers(0, model["vocab"], size=(BATCH, PROMPT)).astype(np.uint32)

    def prefill():
        seqs = [pool.makeSequence() for _ in range(BATCH)]
        if args.prefill == "direct":
            # profiling shortcut: N(0,1) K/V rows written straight into the pages (one launch per layer), so that a
            # profiler capture reaches the decode steps after a few hundred launches instead of ~170k
            kv = torch.randn((BATCH, model["kv_heads"], PROMPT - 1, model["head_dim"]), device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            for layer in range(model["layers"]):
                rt.kv_append_into(pool, layer, seqs, BATCH, BATCH, PROMPT - 1, kv, kv, PROMPT - 1)
            for i, s in enumerate(seqs):
                s.commit(prompts[i, :PROMPT - 1])
            return seqs, dec.executeSampled(pool, seqs, prompts[:, PROMPT - 1:PROMPT])
        tok = None
        for t in range(PROMPT):  # the prompt goes through the decode path one token per step
            tok = dec.executeSampled(pool, seqs, prompts[:, t:t + 1])
        return seqs, tok

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    # ---- leg 1: end to end through executeSampled (host token ids in, sampled ids out, every step)
    seqs, tok = prefill()
    for _ in range(W):
        tok = dec.executeSampled(pool, seqs, tok[:, None])
    barrier()
    sampler.start()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = dec.executeSampled(pool, seqs, tok[:, None])
    barrier()
    e2e_seconds = time.perf_counter() - t0
    launches_per_step = dec.diagnostics()["launches_per_step"]
    for s in seqs:
        s.release()
    # ---- leg 2: device resident (ids, tables and cursors stay in HBM; one CUDA graph replay per step)
    seqs, tok = prefill()
    if W:
        out, _ = dec.generate_greedy(pool, seqs, tok, W)
        tok = out[-1]
    barrier()
    out, device_ms = dec.generate_greedy(pool, seqs, tok, K)
    barrier()
    clocks = sampler.stop()
    times = torch.tensor([device_ms / 1000.0, e2e_seconds], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    if tp:  # every rank must have generated the same tokens
        mine = torch.from_numpy(out.astype(np.int64)).cuda()
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not torch.equal(lo, hi):
            raise RuntimeError("tensor-parallel ranks generated different tokens")
    device_seconds, e2e_seconds = [float(v) for v in times.cpu()]
    graph_launches = dec.diagnostics()["launches_per_step"]
    mean_ctx = PROMPT + W + (K + 1) / 2.0
    step_bytes = algorithmic_bytes_per_step(model, BATCH, mean_ctx)
    peaks, peak_kind = measured_peaks()

    line = None
    if rank == 0:
        if args.no_kernel_timing:
            kernel_ms, kernel_bytes = float("nan"), 0
        else:
            kernel_ms, kernel_bytes = time_dominant_kernel(rt, et, torch, model, BATCH)
        achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
        jobs = 1 if tp else world  # replicas each decode their own batch; tensor-parallel ranks share one
        value = jobs * BATCH * K / device_seconds
        e2e_value = jobs * BATCH * K / e2e_seconds
        max_blocks = max_tokens // BLOCK + 3
        h2d = BATCH * 4 + BATCH * 16 + BATCH * 8 + BATCH * max_blocks * 4
        d2h = BATCH * 4 + 32
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            import oracle as orc
            threads = orc.max_threads()
            fraction = calibrated_fraction(MODEL, BATCH, threads, 15.0)
            v, seconds, sample = cpu_sample(MODEL, BATCH, PROMPT, threads, fraction)
            cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample, "cpu_seconds": seconds}
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1000.0 * device_seconds / K, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
            "dtype": "f16 MMA operands, f32 accumulate (Q4_0 weights, f16 KV)", "data": "synthetic",
            "config": {"workload": f"llama3-8b-shape Q4_0 paged decode: {model['layers']} layers, batch {BATCH}, prompt {PROMPT}, "
                                   f"{K} greedy steps, f16 KV 16-token pages",
                       "global_batch": BATCH * jobs,
                       "parallelism": "single GPU" if world == 1 else (f"tp{world}: rows of q/k/v/gate/up and columns of o/down cut over the ranks, "
                                                                       f"{args.tp_allreduce} all-reduce of [batch, d_model] f32 after o and down, head replicated"
                                                                       if tp else f"{world} independent replicas"),
                       "l2": "per-step working set (weights 4.2 GB + KV) exceeds the 126 MB L2; no flush needed"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1000.0 * e2e_seconds / K, "launches_per_step": launches_per_step},
            "gpu_launches": graph_launches * K,
            "step_roofline": {"algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes * K / device_seconds / 1e9,
                              "frac_of_" + peak_kind: step_bytes * K / device_seconds / 1e9 / peaks["hbm_gbs"]},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         # DRAM bytes per launch of the main kernel: dram__bytes_read.sum + dram__bytes_write.sum of this very launch
                         # (grid 224, one split) from the ncu capture summarised under profiles/
                         "traffic": 66390784 + 531968,
                         "traffic_source": "profiles/qlinear_umma_q4_0_decode_step.md (ncu --set full, gate/up launch)",
                         "peak_kind": peak_kind,
                         "kernel": "qlinear_umma_kernel<Q4_0,32> fused gate/up [28672x4096], 32 vectors, with its f16 conversion and split-K sum launches",
                         "ms_per_launch": kernel_ms, "algorithmic_bytes_per_launch": kernel_bytes},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tp-allreduce", default="peer", choices=["peer", "nccl"],
                    help="--parallelism tp: all-reduce by the library's one-shot peer-memory kernel or by NCCL")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers than the 8B shape (the result is then not a bench value)")
    ap.add_argument("--workload", default="decode", choices=["decode", "attention", "linear", "decode-70b"],
                    help="decode: the headline 8B-shape decode step (the bench contract); attention / linear: the paged-attention and "
                         "quantized-matmul microbenchmarks, one extra JSON line each (single GPU); decode-70b: the 70B shape, batch 64, "
                         "tensor parallel over --gpus ranks")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--parallelism", default="replicas", choices=["replicas", "tp"],
                    help="N > 1: N independent replicas, each decoding its own batch (weak scaling; the 8B shape fits one GPU), or "
                         "one tensor-parallel model over the ranks (strong scaling)")
    ap.add_argument("--prefill", default="model", choices=["model", "direct"],
                    help="model: the prompt runs through the decode path (the benchmark); direct: K/V rows are written "
                         "straight into the pages (profiling shortcut, not a bench value)")
    ap.add_argument("--no-kernel-timing", action="store_true", help="skip the stand-alone timing of the dominant kernel")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.workload == "decode-70b":
        run_tp_70b(args, rank, world)
        return
    if args.workload != "decode":
        if rank == 0:
            (run_attention_microbench if args.workload == "attention" else run_linear_microbench)(args)
        return
    run_gpu_arm(args, rank, world)


if __name__ == "__main__":
    main()
