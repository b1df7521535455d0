#!/usr/bin/env python
"""Benchmark of the paged-KV batched decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N=1 and every rank at N>1): a Llama-3-8B-shaped model with random weights — 32 layers, d_model 4096,
32 query x 128 / 8 KV heads, SwiGLU FFN 14336, vocabulary 128256, RoPE theta 500000; projections and head
~N(0, 0.02) quantized to Q4_0 (token embedding and norms f32); f16 paged KV with 16-token pages; batch 32 prompts of
512 random token ids, prefilled in chunks, then greedy decode. One "step" is one decode step of the whole batch
(32 tokens). All inputs are synthetic (seeded); there is no dataset.

Printed JSON line (rank 0):
  value     decode tokens/s with ids, tables and weights resident in HBM: K steps replayed as one CUDA graph per step
            (etc_decoder_generate_greedy), timed with CUDA events, max over ranks
  e2e       the same metric through the reference-facing call (Executable.executeSampled): every step copies the
            step's token ids / lane descriptors / page tables host->device and reads the sampled tokens back
  roofline  the dominant kernel (tcgen05 Q4_0 linear, fused gate/up shape [28672 x 4096], 32 vectors) timed alone with
            CUDA events on the launching stream (graph replays) over weight sets larger than L2
  roofline_by_projection / roofline_attention   the other launches of a decode step, timed the same way
  linear_microbench / attention_microbench      the quantized-matmul and paged-attention microbenchmark shapes
  cpu_baseline  the CPU oracle (restatement of the reference CPU backend) on a bounded sample, host cores stated
  tp        the Llama-3-70B shape, batch 64, tensor parallel over the N ranks (at N=1: the whole model on one GPU)
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
MODEL_70B = dict(layers=80, d_model=8192, q_heads=64, kv_heads=8, head_dim=128, ffn=28672, vocab=128256, rms_eps=1e-5,
                 rope_theta=500000.0)
BATCH, PROMPT, BLOCK = 32, 512, 16
Q4_0, Q8_0 = 2, 8
METRIC = "decode tokens/s, Llama-3-8B-shape Q4_0 batch 32; kernel HBM GB/s vs peak"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def profile_number(file_name, key):
    """A figure from a committed ncu summary: the first line of profiles/<file_name> that reads `key: <number>`."""
    path = os.path.join(ROOT, "profiles", file_name)
    try:
        with open(path) as f:
            for line in f:
                if line.strip().startswith(key + ":"):
                    return float(line.split(":", 1)[1].split()[0].replace(",", ""))
    except OSError:
        pass
    return None


def host_threads():
    """Cores this process may run on (a launcher may have set OMP_NUM_THREADS=1; the CPU arm passes its thread count
    to the oracle explicitly)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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
def cpu_sample(model, batch, ctx, threads, fraction, seed=3, faithful=False):
    """Times the CPU oracle on a bounded sample of one decode step and scales it to the whole step.

    Every projection of one layer and the head are timed on a row slice (`fraction` of the rows, all columns,
    all `batch` vectors); paged attention is timed on `fraction` of the lanes at context `ctx`; norms, RoPE and
    SwiGLU are timed at full size. Slice times are divided by their fraction and the layer time is multiplied by
    the layer count. `faithful`: the reference's own loop structure on one thread (every block decoded again for every
    vector, attention scores recomputed per output column); otherwise the same arithmetic with every block decoded once
    per row and scores cached, over `threads` threads. Returns (tokens/s, seconds of CPU work done, description)."""
    import oracle as orc
    rng = np.random.default_rng(seed)
    d, qw, kvw, ffn, V, L = (model["d_model"], model["q_heads"] * model["head_dim"], model["kv_heads"] * model["head_dim"],
                             model["ffn"], model["vocab"], model["layers"])
    work = 0.0
    lin_threads = 0 if faithful else threads  # 0 selects the reference-faithful scalar loop of the oracle

    def linear_seconds(rows, cols):
        nonlocal work
        r = min(rows, max(32, int(rows * fraction) // 32 * 32))
        w = rng.standard_normal((r, cols), dtype=np.float32) * np.float32(0.02)
        packed = orc.quantize(orc.Q4_0, w)
        x = rng.standard_normal((batch, cols), dtype=np.float32)
        t0 = time.perf_counter()
        orc.qlinear(orc.Q4_0, x, packed, r, cols, threads=lin_threads)
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
    orc.kv_attention(pool, 0, seqs, lanes, q, k, k, 1.0 / np.sqrt(model["head_dim"]), mode=0 if faithful else 1,
                     threads=1 if faithful else threads)
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
    variant = ("reference-faithful variant: one thread, every block decoded again for every vector, attention scores recomputed per "
               "output column" if faithful else
               f"fair variant: every block decoded once per row, attention scores cached, {threads} threads")
    sample = (f"one batch-{batch} decode step at context {ctx} of the CPU oracle (restatement of the reference CPU backend; {variant}): "
              f"{fraction:.4f} of the rows of each projection and of the lanes of paged attention in 1 of {L} layers, plus the head "
              f"slice, scaled to the full step (extrapolated)")
    return batch / step_seconds, work, sample


def calibrated_fraction(model, batch, threads, budget_seconds, faithful=False):
    """Fraction of one layer's rows whose CPU time fits `budget_seconds` (probed on a small slice)."""
    probe = 1.0 / 256 if faithful else 1.0 / 64
    _, work, _ = cpu_sample(model, batch, PROMPT, threads, probe, faithful=faithful)
    return float(min(1.0, max(1.0 / 512, probe * budget_seconds / max(work, 1e-6))))


def run_reference_arm(args, rank):
    if rank != 0:
        return
    threads = host_threads()
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
        "warmup": args.warmup, "ms_per_step": 1000.0 * BATCH / value, "ms_per_step_is": "extrapolated from the bounded sample of each step",
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"llama3-8b-shape Q4_0 paged decode: {MODEL['layers']} layers, batch {BATCH}, prompt {PROMPT}, "
                               f"{args.steps} greedy steps, f16 KV 16-token pages",
                   "sample": "each step is a bounded CPU sample of that workload, scaled to the full step",
                   "global_batch": BATCH, "parallelism": "cpu"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------ GPU arm
# K-quants (256-value blocks): bytes per block in the file, byte offsets of the f16 block scales, and the bytes the tiled
# form streams per 32 values (Q4_K: nibbles + two f16; the others: int8 codes + two f16)
K_BLOCK_BYTES = {11: 110, 12: 144, 13: 176, 14: 210}
K_SCALE_FIELDS = {11: (108,), 12: (0, 2), 13: (0, 2), 14: (208,)}
K_TILED_BYTES_PER_32 = {11: 36, 12: 20, 13: 36, 14: 36}
K_NAMES = {11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}


def device_random_k_quant(torch, codec, rows, cols, gen):
    """Packed K-quant rows from random bytes with a small finite f16 block scale: every bit pattern of the code and
    sub-scale bytes is legal, the library has no K-quant quantizer, and the kernel's time does not depend on the values."""
    bb, blocks = K_BLOCK_BYTES[codec], cols // 256
    packed = torch.randint(0, 256, (rows, blocks, bb), generator=gen, device="cuda", dtype=torch.uint8)
    scale = torch.tensor([1e-4], dtype=torch.float16).view(torch.uint8).to("cuda")
    for off in K_SCALE_FIELDS[codec]:
        packed[:, :, off:off + 2] = scale
    torch.cuda.synchronize()  # drawn on torch's stream, read on the library's
    return packed.view(rows, blocks * bb)


def device_quantized(rt, torch, codec, rows, cols, gen):
    """[rows, cols] ~ N(0, 0.02) drawn on the device in slabs and packed by the library's quantizer."""
    if codec in K_BLOCK_BYTES:
        return device_random_k_quant(torch, codec, rows, cols, gen)
    bb = 18 if codec == Q4_0 else 34
    packed = torch.empty((rows, cols // 32 * bb), dtype=torch.uint8, device="cuda")
    step = 32768
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        w = torch.randn((r1 - r0, cols), generator=gen, device="cuda", dtype=torch.float32)
        w.mul_(0.02)
        torch.cuda.synchronize()
        rt.quantize_into(codec, w, r1 - r0, cols, packed[r0:r1])
        rt.synchronize()
        del w
    return packed


def build_decoder(rt, et, torch, model, batch, max_tokens, seed, shared_seed=None, max_advance=1):
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
                        exact=False, max_advance=max_advance, vocab_global=model.get("vocab_global"),
                        head_first_row=model.get("head_first_row", 0))
    d, qw, kvw, ffn, V = (model["d_model"], model["q_heads"] * model["head_dim"], model["kv_heads"] * model["head_dim"], model["ffn"],
                          model["vocab"])
    V_embd = model.get("vocab_global", V)

    def bind(slot, layer, tensor, codec=0, rows=None, cols=None):
        torch.cuda.synchronize()
        dec.set_weight(slot, layer, tensor, codec=codec, rows=rows, columns=cols)

    embd = torch.randn((V_embd, d), generator=shared, device="cuda", dtype=torch.float32)
    embd.mul_(0.02)
    bind(et.W_TOK_EMBD, 0, embd)
    del embd
    ones = torch.ones(d, device="cuda", dtype=torch.float32)
    for l in range(model["layers"]):
        bind(et.W_ATTN_NORM, l, ones)
        bind(et.W_FFN_NORM, l, ones)
        for slot, (r, c) in ((et.W_Q, (qw, d)), (et.W_K, (kvw, d)), (et.W_V, (kvw, d)), (et.W_O, (d, qw)), (et.W_GATE, (ffn, d)),
                             (et.W_UP, (ffn, d)), (et.W_DOWN, (d, ffn))):
            bind(slot, l, device_quantized(rt, torch, Q4_0, r, c, gen), Q4_0, r, c)
    bind(et.W_OUT_NORM, 0, ones)
    # a sharded head: every rank draws its own rows (the ranks only have to agree on what they replicate)
    bind(et.W_HEAD, 0, device_quantized(rt, torch, Q4_0, V, d, gen if "vocab_global" in model else shared), Q4_0, V, d)
    dec.finalize()
    torch.cuda.empty_cache()
    return dec


def time_linear(rt, et, torch, codec, rows, cols, vectors, interleave=False, epilogue=0, residual=False, target_bytes=300e6, gen=None):
    """One tiled linear shape alone: CUDA events around replays of a graph that walks over more weight copies than L2
    holds. Returns (microseconds per call, algorithmic bytes per call). The call includes the linear's own f16 conversion
    of the activations and, above 16 vectors, its split-K sum launch."""
    # bytes of weights one call streams: the file's encoding for Q4_0 / Q8_0, the re-cut tiled form for the K-quants
    bb = K_TILED_BYTES_PER_32[codec] if codec in K_BLOCK_BYTES else (18 if codec == Q4_0 else 34)
    nparts = 2 if interleave else 1
    packed_bytes = rows * (cols // 32) * bb
    copies = max(3, int(np.ceil(target_bytes / packed_bytes)))
    if gen is None:
        gen = torch.Generator(device="cuda")
        gen.manual_seed(rows + cols + codec)
    weights = []
    for _ in range(copies):
        parts = [device_quantized(rt, torch, codec, rows // nparts, cols, gen) for _ in range(nparts)]
        weights.append(et.QWeight(rt, codec, parts, [rows // nparts] * nparts, cols, interleave8=interleave))
        del parts
    out_cols = rows // 2 if epilogue == et.EPILOGUE_SWIGLU else rows
    x = torch.randn((vectors, cols), generator=gen, device="cuda", dtype=torch.float32)
    out = torch.empty((vectors, out_cols), device="cuda", dtype=torch.float32)
    res = torch.randn((vectors, out_cols), generator=gen, device="cuda", dtype=torch.float32) if residual else None
    need = weights[0].scratch_bytes(vectors)
    scratch = torch.empty(max(need, 4), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(rt.stream)

    def call(i):
        weights[i % copies].linear_into(x, vectors, out, residual=res, epilogue=epilogue, scratch=scratch, scratch_bytes=need)

    for i in range(copies):
        call(i)
    rt.synchronize()
    iters = 2 * copies
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(iters):
            call(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        graph.replay()
        a.record()
        graph.replay()
        graph.replay()
        b.record()
    rt.synchronize()
    us = a.elapsed_time(b) / (2 * iters) * 1e3
    algorithmic = packed_bytes + 4 * vectors * cols + 4 * vectors * out_cols
    del graph
    for w in weights:
        w.close()
    torch.cuda.empty_cache()
    return us, algorithmic


def roofline_entry(us, algorithmic, peaks, peak_kind, kernel, traffic=None, traffic_source=None):
    achieved = algorithmic / us / 1e3
    entry = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
             "traffic": traffic, "peak_kind": peak_kind, "kernel": kernel, "ms_per_launch": us / 1e3,
             "algorithmic_bytes_per_launch": algorithmic}
    if traffic_source:
        entry["traffic_source"] = traffic_source
    return entry


def projection_rooflines(rt, et, torch, model, vectors, peaks, peak_kind):
    """Every linear launch of a decode step at `vectors` rows, timed alone (see time_linear)."""
    d, qw, kvw, ffn, V = (model["d_model"], model["q_heads"] * model["head_dim"], model["kv_heads"] * model["head_dim"], model["ffn"],
                          model["vocab"])
    shapes = [("qkv", qw + 2 * kvw, d, False, et.EPILOGUE_NONE, False), ("o", d, qw, False, et.EPILOGUE_RESIDUAL, True),
              ("gate_up", 2 * ffn, d, True, et.EPILOGUE_SWIGLU, False), ("down", d, ffn, False, et.EPILOGUE_RESIDUAL, True),
              ("head", V, d, False, et.EPILOGUE_NONE, False)]
    nv = 32 if vectors <= 32 else 64 if vectors <= 64 else 128 if vectors <= 128 else 256
    kernel = "qlinear_mv_kernel<Q4_0>" if vectors <= 16 else f"qlinear_umma_kernel<Q4_0,{nv}> (+ f16 conversion and split-K sum launches)"
    out = {}
    for name, rows, cols, interleave, epilogue, residual in shapes:
        us, algorithmic = time_linear(rt, et, torch, Q4_0, rows, cols, vectors, interleave, epilogue, residual)
        out[name] = roofline_entry(us, algorithmic, peaks, peak_kind, f"{kernel} [{rows}x{cols}], {vectors} vectors")
    return out


def linear_microbench_table(rt, et, torch, peaks):
    """The quantized-matmul microbenchmark: Q4_0 and Q8_0, [4096x4096], [14336x4096], [4096x14336], 1 / 8 / 64 / 512
    vectors, f32 activations; HBM fraction up to 64 vectors, TFLOP/s at 512."""
    rows_out = []
    for codec, name in ((Q4_0, "Q4_0"), (Q8_0, "Q8_0")):
        for n, k in ((4096, 4096), (14336, 4096), (4096, 14336)):
            for m in (1, 8, 64, 512):
                us, algorithmic = time_linear(rt, et, torch, codec, n, k, m)
                rows_out.append({"codec": name, "rows": n, "columns": k, "vectors": m, "us": round(us, 2),
                                 "gbs": round(algorithmic / us / 1e3, 1), "hbm_frac": round(algorithmic / us / 1e3 / peaks["hbm_gbs"], 3),
                                 "tflops": round(2.0 * m * n * k / us / 1e6, 1),
                                 "tensor_frac": round(2.0 * m * n * k / us / 1e6 / peaks["bf16_tflops"], 3)})
    return rows_out


def k_quant_microbench_table(rt, et, torch, peaks):
    """One row per K-quant with a tiled form: the FFN up-projection shape [14336x4096] at 32 and 512 vectors through the
    tcgen05 linear. `gbs` counts the bytes the re-cut form streams (20 B per 32 values for Q4_K, 36 B for the others)."""
    rows_out = []
    for codec in sorted(K_BLOCK_BYTES):
        for m in (32, 512):
            try:
                us, algorithmic = time_linear(rt, et, torch, codec, 14336, 4096, m)
                rows_out.append({"codec": K_NAMES[codec], "rows": 14336, "columns": 4096, "vectors": m, "us": round(us, 2),
                                 "gbs": round(algorithmic / us / 1e3, 1), "hbm_frac": round(algorithmic / us / 1e3 / peaks["hbm_gbs"], 3),
                                 "tflops": round(2.0 * m * 14336 * 4096 / us / 1e6, 1),
                                 "tensor_frac": round(2.0 * m * 14336 * 4096 / us / 1e6 / peaks["bf16_tflops"], 3)})
            except Exception as error:  # a row that cannot be timed is reported, it does not cost the line
                rows_out.append({"codec": K_NAMES[codec], "rows": 14336, "columns": 4096, "vectors": m, "error": str(error)[:200]})
    return rows_out


def shuffled_pool(rt, et, torch, layers, kv_heads, head_dim, pages, seed):
    """A pool whose free pages come back in a seeded random order: every page goes to a one-page sequence, the sequences
    are released in shuffled order, and later allocations draw page numbers like a permutation of the pool."""
    pool = et.NativeKvPool(rt, layers, kv_heads, head_dim, pages * BLOCK, BLOCK, et.KV_F16)
    holders = [pool.makeSequence() for _ in range(pages)]
    zeros = torch.zeros((256, kv_heads, BLOCK, head_dim), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    for i in range(0, pages, 256):
        group = holders[i:i + 256]
        rt.kv_append_into(pool, 0, group, len(group), len(group), BLOCK, zeros, zeros, BLOCK)
    for i in np.random.default_rng(seed).permutation(pages):
        holders[int(i)].release()
    return pool


def time_attention(rt, et, torch, batch, q_heads, kv_heads, head_dim, ctx, pool_pages, peaks, peak_kind, label, iters=40):
    """Paged attention decode alone over a shuffled page pool: `batch` sequences of the given context lengths, one query
    token each. The launch is the host-state-free operator over device-resident lane descriptors and tables, captured into a
    CUDA graph (several pools' worth of KV is not needed: one pass already reads more than L2 holds for the microbenchmark
    shape; for the in-step shape the graph alternates between two disjoint sets of sequences)."""
    ctx = np.asarray(ctx)
    sets = 1 if int(ctx.sum()) * 2 * kv_heads * head_dim * 2 > 200e6 else 2 + int(200e6 // max(1, int(ctx.sum()) * 2 * kv_heads * head_dim * 2))
    pool = shuffled_pool(rt, et, torch, 1, kv_heads, head_dim, pool_pages, seed=11)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    chunk = 64
    order = np.argsort(-ctx)
    lanes_dev, tables_dev, keep = [], [], []
    for _ in range(sets):
        seqs = [pool.makeSequence() for _ in range(batch)]
        kv = torch.randn((batch, kv_heads, chunk, head_dim), generator=gen, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        total = ctx + 1  # the new token's K/V row is part of what the step attends over
        for start in range(0, int(total.max()), chunk):
            group = [seqs[int(i)] for i in order if total[i] - start >= chunk]
            if group:
                rt.kv_append_into(pool, 0, group, len(group), len(group), chunk, kv, kv, chunk)
                for s in group:
                    s.commit(np.arange(chunk, dtype=np.uint32))
        for i in range(batch):  # ragged tails
            tail = int(total[i]) % chunk
            if tail:
                rt.kv_append_into(pool, 0, [seqs[i]], 1, 1, tail, kv, kv, tail)
                seqs[i].commit(np.arange(tail, dtype=np.uint32))
        lanes = np.zeros((batch, 4), dtype=np.int32)
        flat = []
        for i in range(batch):
            blocks, head = seqs[i].blocks
            lanes[i] = (int(ctx[i]), 1, 0, len(flat) - head)
            flat.extend(int(b) for b in blocks)
        lanes_dev.append(torch.from_numpy(lanes).cuda())
        tables_dev.append(torch.from_numpy(np.asarray(flat, dtype=np.int32)).cuda())
        keep.append(seqs)  # a dropped handle returns its pages to the pool
    max_pages = int(np.ceil((ctx + 1) / BLOCK).max())
    plan = et.attention_plan(batch, q_heads, kv_heads, head_dim, max_pages, sm_count=rt.capabilities()["sm_count"])
    scratch = torch.empty(max(plan["partial_bytes"], 4), dtype=torch.uint8, device="cuda")
    q = torch.randn((batch, q_heads, head_dim), generator=gen, device="cuda", dtype=torch.float32)
    out = torch.empty((batch, q_heads, head_dim), device="cuda", dtype=torch.float32)
    scale = 1.0 / np.sqrt(head_dim)
    torch.cuda.synchronize()
    stream = torch.cuda.ExternalStream(rt.stream)

    def call(i):
        rt.paged_attention_into(pool, 0, lanes_dev[i % sets], tables_dev[i % sets], batch, max_pages, q, q_heads, scale, out, scratch,
                                plan["partial_bytes"])

    for i in range(max(3, sets)):
        call(i)
    rt.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(iters):
            call(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        graph.replay()
        a.record()
        graph.replay()
        graph.replay()
        b.record()
    rt.synchronize()
    us = a.elapsed_time(b) / (2 * iters) * 1e3
    total_ctx = int((ctx + 1).sum())
    algorithmic = total_ctx * 2 * kv_heads * head_dim * 2 + batch * q_heads * head_dim * 8 + 4 * int(np.ceil((ctx + 1) / BLOCK).sum())
    entry = roofline_entry(us, algorithmic, peaks, peak_kind, f"attention_mma_kernel<{head_dim},f16> (+ merge when split): {label}")
    entry.update({"splits": plan["splits"], "kv_sets_rotated": sets, "tables": "drawn from a shuffled page pool",
                  "operands": "f32 queries (rounded to f16 for the MMA), f16 K / V pages"})
    del graph
    keep.clear()
    pool.close()
    torch.cuda.empty_cache()
    return entry


def run_tp_70b(args, rank, world, rt, et, torch, dist, steps, warmup):
    """Llama-3-70B-shape Q4_0 decode, batch 64, contexts ~U[1024, 8192], tensor parallel over `world` ranks (the whole model
    on one GPU at world 1). KV is written straight into the pages (N(0,1) rows; a decode benchmark needs no real prefill)
    and the steps run device-resident. Returns the `tp` object of the bench line (rank 0) or None."""
    from effect_torch_b200 import tensor_parallel

    local = int(os.environ.get("LOCAL_RANK", "0"))
    full = dict(MODEL_70B)
    if args.layers:
        full["layers"] = args.layers
    shard_head = world > 1 and args.tp_head == "sharded"
    model = tensor_parallel.local_config(full, world, shard_head=shard_head, rank=rank)
    if world == 1 and args.rank_of > 1:
        # one rank's share of the work of a tensor-parallel group of that size, alone on one GPU and without the exchange:
        # what is left of a real rank's step time after this is communication and waiting for peers
        model = tensor_parallel.local_config(full, args.rank_of, shard_head=args.tp_head == "sharded", rank=0)
        model.pop("vocab_global", None)
        model.pop("head_first_row", None)
    B, K, W, chunk = 64, steps, warmup, 256
    rng = np.random.default_rng(4)  # the same contexts and tokens on every rank
    whole_model_on_one_gpu = world == 1 and args.rank_of <= 1
    lo, hi = (256, 1024) if whole_model_on_one_gpu else (1024, 8192)  # one GPU: 138 GB of weights leave room for an eighth of the KV
    ctx = np.sort((rng.integers(lo, hi + 1, size=B) // chunk) * chunk)[::-1].copy()
    max_tokens = ((int(ctx.sum()) + B * (W + K + 2 * BLOCK)) // BLOCK + B) * BLOCK
    dec = build_decoder(rt, et, torch, model, B, max_tokens, seed=40 + rank, shared_seed=4)
    allreduce = "none"
    if world > 1:
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            ident = torch.frombuffer(bytearray(et.tensor_parallel_id()), dtype=torch.uint8).cuda()
        dist.broadcast(ident, src=0)
        dec.set_tensor_parallel(rank, world, bytes(ident.cpu().tolist()))
        allreduce = args.tp_allreduce if args.tp_allreduce != "auto" else "peer"
        if shard_head and allreduce != "peer":
            raise RuntimeError("a sharded head exchanges its picks over the peer regions: use --tp-allreduce peer or --tp-head replicated")
        if allreduce == "peer":
            mine = torch.frombuffer(bytearray(dec.peer_exchange_handle()), dtype=torch.uint8).cuda()
            table = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(table, mine)
            dec.use_peer_allreduce([bytes(t.cpu().tolist()) for t in table])
            forced = os.environ.get("ETC_TP_TWO_SHOT")
            two_shot = world >= 8 if forced is None else forced != "0"
            allreduce = "peer memory, reduce-scatter + all-gather" if two_shot else "peer memory, one shot"
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
    tok = rng.integers(0, model.get("vocab_global", model["vocab"]), size=B).astype(np.uint32)
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
    agree = True
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        mine = torch.from_numpy(out.astype(np.int64)).cuda()
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        agree = bool(torch.equal(lo, hi))
    seconds = float(times.cpu()[0])
    launches = dec.diagnostics()["launches_per_step"]
    pool.close()
    dec.close()
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    mean_ctx = float(ctx.mean()) + W + (K + 1) / 2.0
    step_bytes = algorithmic_bytes_per_step(full, B, mean_ctx)
    peaks, peak_kind = measured_peaks()
    return {
        "metric": "decode tokens/s, Llama-3-70B-shape Q4_0 batch 64, tensor parallel", "value": B * K / seconds, "unit": "tokens/s",
        "tp": world, "steps": K, "warmup": W, "ms_per_step": 1000.0 * seconds / K, "scaling": "strong",
        "config": {"workload": f"llama3-70b-shape Q4_0 paged decode: {full['layers']} layers, batch {B}, contexts {int(ctx.min())}.."
                               f"{int(ctx.max())} (mean {ctx.mean():.0f}) written directly into the pages, {K} greedy steps",
                   "parallelism": (f"one rank's share of a tp{args.rank_of} group, alone and without the exchange" if args.rank_of > 1 else
                                   "one GPU holds the whole model") if world == 1 else
                                  f"tp{world}: rows of q/k/v/gate/up and columns of o/down cut over the ranks, {allreduce} all-reduce of "
                                  "[batch, d_model] f32 after o and down (split-K partials summed in the same kernel), head "
                                  + ("cut by rows, (logit, token) picks exchanged" if shard_head else "replicated")},
        "launches_per_step": launches, "all_reduce": allreduce, "ranks_agree_on_tokens": agree,
        "step_roofline": {"algorithmic_bytes_per_step_all_ranks": step_bytes,
                          "achieved_gbs_per_rank": step_bytes / max(world, args.rank_of, 1) * K / seconds / 1e9,
                          "frac_of_" + peak_kind + "_per_rank": step_bytes / max(world, args.rank_of, 1) * K / seconds / 1e9 / peaks["hbm_gbs"]},
        "clocks": clocks}


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
    chunk = max(1, min(args.prefill_chunk, PROMPT))
    # every sequence: prompt + warm-up + timed steps, twice (end-to-end leg, then device-resident leg)
    per_seq = ((PROMPT + W + K + BLOCK) // BLOCK + 1) * BLOCK
    max_tokens = 2 * BATCH * per_seq
    dec = build_decoder(rt, et, torch, model, BATCH, max_tokens, seed=3 + rank, shared_seed=3 if tp else None, max_advance=chunk)
    allreduce = args.tp_allreduce if args.tp_allreduce != "auto" else ("peer" if world <= 2 else "nccl")
    if tp:
        ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            ident = torch.frombuffer(bytearray(et.tensor_parallel_id()), dtype=torch.uint8).cuda()
        dist.broadcast(ident, src=0)
        dec.set_tensor_parallel(rank, world, bytes(ident.cpu().tolist()))
        if allreduce == "peer":  # one-shot kernel over peer memory instead of NCCL
            mine = torch.frombuffer(bytearray(dec.peer_exchange_handle()), dtype=torch.uint8).cuda()
            table = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(table, mine)
            dec.use_peer_allreduce([bytes(t.cpu().tolist()) for t in table])
    pool = et.NativeKvPool(rt, model["layers"], model["kv_heads"], model["head_dim"], max_tokens, BLOCK, et.KV_F16)
    rng = np.random.default_rng(3 if tp else 3 + rank)  # tensor-parallel ranks decode the same sequences
    prompts = rng.integers(0, model["vocab"], size=(BATCH, PROMPT)).astype(np.uint32)
    prefill_seconds = []

    def prefill():
        """The prompt in chunks of `chunk` tokens per sequence through the same executable (teacher-forced; the last chunk's
        sampled tokens start the decode). Returns (sequences, first generated tokens)."""
        seqs = [pool.makeSequence() for _ in range(BATCH)]
        if args.prefill == "direct":
            # profiling shortcut: N(0,1) K/V rows written straight into the pages (one launch per layer), so that a
            # profiler capture reaches the decode steps after a few hundred launches
            kv = torch.randn((BATCH, model["kv_heads"], PROMPT - 1, model["head_dim"]), device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            for layer in range(model["layers"]):
                rt.kv_append_into(pool, layer, seqs, BATCH, BATCH, PROMPT - 1, kv, kv, PROMPT - 1)
            for i, s in enumerate(seqs):
                s.commit(prompts[i, :PROMPT - 1])
            return seqs, dec.executeSampled(pool, seqs, prompts[:, PROMPT - 1:PROMPT])
        tok = None
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for start in range(0, PROMPT, chunk):
            tok = dec.executeSampled(pool, seqs, prompts[:, start:min(PROMPT, start + chunk)])
        prefill_seconds.append(time.perf_counter() - t0)
        return seqs, tok

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    # ---- leg 1: end to end through executeSampled (host token ids in, sampled ids out, every step)
    seqs, tok = prefill()
    first_tokens = tok.copy()
    for _ in range(W):
        tok = dec.executeSampled(pool, seqs, tok[:, None])
    barrier()
    sampler.start()
    e2e_tokens = []
    t0 = time.perf_counter()
    for _ in range(K):
        tok = dec.executeSampled(pool, seqs, tok[:, None])
        e2e_tokens.append(tok)
    barrier()
    e2e_seconds = time.perf_counter() - t0
    launches_per_step = dec.diagnostics()["launches_per_step"]
    for s in seqs:
        s.release()
    # ---- leg 2: device resident (ids, tables and cursors stay in HBM; one CUDA graph replay per step)
    seqs, tok = prefill()
    same_first = bool(np.array_equal(tok, first_tokens))
    if W:
        out, _ = dec.generate_greedy(pool, seqs, tok, W)
        tok = out[-1]
    barrier()
    out, device_ms = dec.generate_greedy(pool, seqs, tok, K)
    barrier()
    clocks = sampler.stop()
    tokens_agree = same_first and bool(np.array_equal(np.stack(e2e_tokens), out))
    times = torch.tensor([device_ms / 1000.0, e2e_seconds], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ranks_agree = True
    if tp:  # every rank must have generated the same tokens
        mine = torch.from_numpy(out.astype(np.int64)).cuda()
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ranks_agree = bool(torch.equal(lo, hi))
    device_seconds, e2e_seconds = [float(v) for v in times.cpu()]
    graph_launches = dec.diagnostics()["launches_per_step"]
    mean_ctx = PROMPT + W + (K + 1) / 2.0
    step_bytes = algorithmic_bytes_per_step(model, BATCH, mean_ctx)
    peaks, peak_kind = measured_peaks()
    pool.close()
    dec.close()
    torch.cuda.empty_cache()

    line = None
    if rank == 0:
        jobs = 1 if tp else world  # replicas each decode their own batch; tensor-parallel ranks share one
        value = jobs * BATCH * K / device_seconds
        e2e_value = jobs * BATCH * K / e2e_seconds
        max_blocks = max_tokens // BLOCK + 3
        h2d = BATCH * 4 + BATCH * 16 + BATCH * 8 + BATCH * max_blocks * 4
        d2h = BATCH * 4 + 32
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": 1000.0 * device_seconds / K, "higher_is_better": True, "scaling": "strong" if tp else "weak", "vs_baseline": None,
            "dtype": "f16 MMA operands, f32 accumulate (Q4_0 weights, f16 KV)", "data": "synthetic",
            "config": {"workload": f"llama3-8b-shape Q4_0 paged decode: {model['layers']} layers, batch {BATCH}, prompt {PROMPT}, "
                                   f"{K} greedy steps, f16 KV 16-token pages",
                       "global_batch": BATCH * jobs,
                       "parallelism": "single GPU" if world == 1 else (f"tp{world}: rows of q/k/v/gate/up and columns of o/down cut over the ranks, "
                                                                       f"{allreduce} all-reduce of [batch, d_model] f32 after o and down, head replicated"
                                                                       if tp else f"{world} independent replicas"),
                       "l2": "per-step working set (weights 4.2 GB + KV) exceeds the 126 MB L2; no flush needed"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1000.0 * e2e_seconds / K, "launches_per_step": launches_per_step},
            "e2e_check": {"tokens_agree_with_device_resident_leg": tokens_agree, "tokens_compared": int(BATCH * (K + 1)),
                          "tensor_parallel_ranks_agree": ranks_agree},
            "gpu_launches": graph_launches * K,
            "step_roofline": {"algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes * K / device_seconds / 1e9,
                              "frac_of_" + peak_kind: step_bytes * K / device_seconds / 1e9 / peaks["hbm_gbs"]},
            "clocks": clocks,
        }
        if prefill_seconds:
            line["prefill"] = {"tokens_per_s": jobs * BATCH * PROMPT / float(np.mean(prefill_seconds)), "chunk": chunk,
                               "seconds": float(np.mean(prefill_seconds)),
                               "path": "chunks through Executable.executeSampled: tcgen05 linears at batch x chunk rows, RoPE + KV append "
                                       "for the whole chunk in one launch, tensor-core chunked-prefill attention"}
        if not args.no_kernel_timing:
            us, algorithmic = time_linear(rt, et, torch, Q4_0, 2 * model["ffn"], model["d_model"], BATCH, True, et.EPILOGUE_SWIGLU, False, 264e6)
            # DRAM bytes per launch of this very kernel and shape, from the committed ncu summary
            traffic = profile_number("qlinear_umma_q4_0_decode_step.md", "gate_up_dram_bytes_per_launch")
            line["roofline"] = roofline_entry(
                us, algorithmic, peaks, peak_kind,
                f"qlinear_umma_kernel<Q4_0,32> fused gate/up [{2 * model['ffn']}x{model['d_model']}], {BATCH} vectors, with its f16 conversion launch",
                traffic, "ncu --set full capture of this launch on the 2-layer case, summary under profiles/" if traffic else None)
            line["roofline_by_projection"] = projection_rooflines(rt, et, torch, model, BATCH, peaks, peak_kind)
            ctx_step = np.full(BATCH, int(mean_ctx))
            pages = int(np.ceil((ctx_step + 1) / BLOCK).sum()) * 6 + 256
            line["roofline_attention"] = time_attention(rt, et, torch, BATCH, model["q_heads"], model["kv_heads"], model["head_dim"], ctx_step,
                                                        pages, peaks, peak_kind, f"the decode step's launch: {BATCH} sequences at context {int(mean_ctx)}")
        if not args.no_microbench and world == 1:
            line["linear_microbench"] = linear_microbench_table(rt, et, torch, peaks)
            line["k_quant_microbench"] = k_quant_microbench_table(rt, et, torch, peaks)
            rng_c2 = np.random.default_rng(1)
            ctx_c2 = rng_c2.integers(128, 4097, size=64)
            line["attention_microbench"] = time_attention(rt, et, torch, 64, 32, 8, 128, ctx_c2, 65536, peaks, peak_kind,
                                                          "64 sequences, contexts ~U[128, 4096], pool of 65536 pages")
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = host_threads()
            fraction = calibrated_fraction(MODEL, BATCH, threads, 12.0)
            v, seconds, sample = cpu_sample(MODEL, BATCH, PROMPT, threads, fraction)
            cpu = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample, "cpu_seconds": seconds}
            ffrac = calibrated_fraction(MODEL, BATCH, 1, 6.0, faithful=True)
            fv, fseconds, fsample = cpu_sample(MODEL, BATCH, PROMPT, 1, ffrac, faithful=True)
            cpu["reference_faithful"] = {"value": fv, "unit": "tokens/s", "cores": 1, "sample": fsample, "cpu_seconds": fseconds}
        line["cpu_baseline"] = cpu
    tp_line = None
    if not args.no_tp70b and not args.layers:
        free_bytes = torch.cuda.mem_get_info()[0]
        try:
            if world == 1 and free_bytes < 168e9:
                raise RuntimeError(f"only {free_bytes / 1e9:.0f} GB free on the device: the 70B shape needs 160 GB on one GPU")
            tp_line = run_tp_70b(args, rank, world, rt, et, torch, dist, steps=min(K, args.tp_steps), warmup=min(W, 3))
        except Exception as exc:  # the headline must survive a failure of the extra workload
            tp_line = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    if rank == 0:
        if tp_line is not None:
            line["tp"] = tp_line
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line


_JSON_OUT = None


def emit(line):
    """The JSON line goes to the process's real stdout; everything else a library prints meanwhile (NCCL's version
    banner for one) was sent to stderr by main()."""
    text = json.dumps(line) + "\n"
    if _JSON_OUT is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_JSON_OUT, text.encode())


def main():
    global _JSON_OUT
    sys.stdout.flush()
    _JSON_OUT = os.dup(1)
    os.dup2(2, 1)  # stray prints of libraries must not mix with the one JSON line
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tp-allreduce", default="auto", choices=["auto", "peer", "nccl"],
                    help="tensor parallel: all-reduce by the library's one-shot peer-memory kernel or by NCCL (auto: peer at 2 ranks, "
                         "NCCL above)")
    ap.add_argument("--tp-head", default="sharded", choices=["sharded", "replicated"],
                    help="tensor parallel: the head cut by rows over the ranks (every rank scores vocab / N tokens) or whole on every rank")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers than the named shape (the result is then not a bench value)")
    ap.add_argument("--workload", default="decode", choices=["decode", "decode-70b", "kernels"],
                    help="decode: the headline 8B-shape decode step (the bench contract) with the kernel rooflines, microbenchmarks and the "
                         "70B tensor-parallel run in the same line; decode-70b: only the 70B shape over --gpus ranks; kernels: only the "
                         "stand-alone kernel timings (the linears at --vectors rows, the attention launches), e.g. under a profiler")
    ap.add_argument("--vectors", type=int, default=BATCH, help="--workload kernels: input rows of the linears")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-microbench", action="store_true", help="skip the quantized-matmul and paged-attention microbenchmark tables")
    ap.add_argument("--no-tp70b", action="store_true", help="skip the 70B-shape run (tensor parallel over the N ranks) that fills the line's tp object")
    ap.add_argument("--tp-steps", type=int, default=32, help="decode steps of the 70B run")
    ap.add_argument("--rank-of", type=int, default=0,
                    help="--workload decode-70b on one GPU: run one rank's share of a tensor-parallel group of this size without the "
                         "exchange (a per-rank compute baseline, e.g. under a profiler)")
    ap.add_argument("--parallelism", default="replicas", choices=["replicas", "tp"],
                    help="N > 1: N independent replicas, each decoding its own batch (weak scaling; the 8B shape fits one GPU), or "
                         "one tensor-parallel model over the ranks (strong scaling)")
    ap.add_argument("--prefill", default="model", choices=["model", "direct"],
                    help="model: the prompt runs through the executable in chunks (the benchmark); direct: K/V rows are written "
                         "straight into the pages (profiling shortcut, not a bench value)")
    ap.add_argument("--prefill-chunk", type=int, default=64, help="tokens per sequence per prefill call")
    ap.add_argument("--no-kernel-timing", action="store_true", help="skip the stand-alone timing of the step's kernels")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.workload == "kernels":
        import torch
        import effect_torch_b200 as et
        torch.cuda.set_device(0)
        rt = et.Runtime(0)
        peaks, peak_kind = measured_peaks()
        line = {"metric": "kernel HBM GB/s vs peak", "unit": "GB/s", "n_gpus": 1, "data": "synthetic",
                "config": {"workload": f"stand-alone kernel timings at {args.vectors} vectors (graph replays over more than L2 of weights / KV)"},
                "roofline_by_projection": projection_rooflines(rt, et, torch, MODEL, args.vectors, peaks, peak_kind)}
        if not args.no_microbench:
            ctx_step = np.full(BATCH, PROMPT + 19)
            line["roofline_attention"] = time_attention(rt, et, torch, BATCH, MODEL["q_heads"], MODEL["kv_heads"], MODEL["head_dim"], ctx_step,
                                                        int(np.ceil((ctx_step + 1) / BLOCK).sum()) * 6 + 256, peaks, peak_kind,
                                                        f"the decode step's launch: {BATCH} sequences at context {PROMPT + 19}")
            ctx_c2 = np.random.default_rng(1).integers(128, 4097, size=64)
            line["attention_microbench"] = time_attention(rt, et, torch, 64, 32, 8, 128, ctx_c2, 65536, peaks, peak_kind,
                                                          "64 sequences, contexts ~U[128, 4096], pool of 65536 pages")
        emit(line)
        return
    if args.workload == "decode-70b":
        import torch
        import torch.distributed as dist
        import effect_torch_b200 as et
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        line = run_tp_70b(args, rank, world, et.Runtime(local), et, torch, dist, steps=args.steps, warmup=args.warmup)
        if rank == 0:
            line["n_gpus"] = world
            emit(line)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    run_gpu_arm(args, rank, world)


if __name__ == "__main__":
    main()
