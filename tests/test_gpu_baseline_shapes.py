"""GPU parity at the sizes the benchmark runs: the Llama-3-8B-shape projections (and the fused gate/up and the head) at 1
to 512 vectors, paged attention at 64 sequences with contexts up to 4096 over shuffled page tables, and a 2-layer decoder
of the 8B width at batch 32. The oracle is run on slices (rows, lanes) so that the CPU side stays in seconds; the inputs
are seeded and identical on both sides. Weights are drawn and quantized on the device (the device quantizer is bit-exact
with the oracle's, tests/test_gpu_quant.py) and the packed rows of the checked slices are read back for the oracle."""
import numpy as np
import pytest
import torch

import effect_torch_b200 as et
import oracle as orc
from tests import helpers
from tests.gpu_util import dev, empty, host, runtime

pytestmark = pytest.mark.gpu
REL_TOL = 2e-3  # north-star tolerance on f16/f32 outputs, as max |err| / max |ref|
THREADS = max(1, min(16, orc.max_threads()))


def device_quantized(codec, rows, columns, seed):
    """[rows, columns] ~ N(0, 0.02) drawn on the device and packed by the device quantizer."""
    rt = runtime()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    bb = 18 if codec == orc.Q4_0 else 34
    packed = torch.empty((rows, columns // 32 * bb), dtype=torch.uint8, device="cuda")
    step = 16384
    for r0 in range(0, rows, step):  # in slabs: the f32 copy of the head would be 2 GB
        r1 = min(rows, r0 + step)
        w = torch.randn((r1 - r0, columns), generator=gen, device="cuda", dtype=torch.float32) * 0.02
        torch.cuda.synchronize()
        rt.quantize_into(codec, w, r1 - r0, columns, packed[r0:r1])
        rt.synchronize()
    return packed


def row_slices(rows, count=128):
    """First, middle and last `count` rows: tile 0, a tile in the middle of the stream-K cut, and the padded tail."""
    mid = (rows // 2 // 128) * 128 + 37
    return [(0, count), (mid, min(rows, mid + count)), (rows - count, rows)]


@pytest.mark.parametrize("codec", [orc.Q4_0, orc.Q8_0], ids=["Q4_0", "Q8_0"])
@pytest.mark.parametrize("rows,columns", [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)])
def test_projection_shapes_match_the_oracle_at_every_vector_count(codec, rows, columns):
    if codec == orc.Q8_0 and rows > 20000:
        pytest.skip("the head is Q4_0 in the benchmark; Q8_0 is covered by the three projection shapes")
    rt = runtime()
    packed = device_quantized(codec, rows, columns, seed=rows + columns + codec)
    qw = et.QWeight(rt, codec, [packed], [rows], columns)
    rng = np.random.default_rng(rows ^ columns)
    slices = row_slices(rows)
    host_rows = [packed[a:b].cpu().numpy() for a, b in slices]
    for vectors in (1, 8, 16, 32, 64, 512):
        x = rng.normal(size=(vectors, columns)).astype(np.float32)
        out = empty((vectors, rows))
        dx = dev(x)
        qw.linear_into(dx, vectors, out)
        got = host(out)
        for (a, b), hp in zip(slices, host_rows):
            expected = orc.qlinear(codec, x, hp, b - a, columns, threads=THREADS)
            assert helpers.rel_err(got[:, a:b], expected) <= REL_TOL, f"{vectors} vectors, rows {a}..{b}"
    qw.close()


@pytest.mark.parametrize("vectors", [4, 16, 32])
def test_fused_gate_up_and_down_at_the_8b_width(vectors):
    """The decode step's two largest launches: gate/up [2 x 14336, 4096] interleaved with the SwiGLU epilogue, then down
    [4096, 14336] with the residual epilogue, on a slice of the FFN rows and of the output rows."""
    rt = runtime()
    d, ffn = 4096, 14336
    pg, pu = device_quantized(orc.Q4_0, ffn, d, 11), device_quantized(orc.Q4_0, ffn, d, 12)
    pd = device_quantized(orc.Q4_0, d, ffn, 13)
    qgu = et.QWeight(rt, orc.Q4_0, [pg, pu], [ffn, ffn], d, interleave8=True)
    qd = et.QWeight(rt, orc.Q4_0, [pd], [d], ffn)
    rng = np.random.default_rng(vectors)
    x = rng.normal(size=(vectors, d)).astype(np.float32)
    act = empty((vectors, ffn))
    qgu.linear_into(dev(x), vectors, act, epilogue=et.EPILOGUE_SWIGLU)
    got_act = host(act)
    for a, b in row_slices(ffn):
        hg, hu = pg[a:b].cpu().numpy(), pu[a:b].cpu().numpy()
        expected = orc.silu_mul(orc.qlinear(orc.Q4_0, x, hg, b - a, d, threads=THREADS), orc.qlinear(orc.Q4_0, x, hu, b - a, d, threads=THREADS))
        assert helpers.rel_err(got_act[:, a:b], expected) <= REL_TOL, f"gate/up rows {a}..{b}"
    residual = rng.normal(size=(vectors, d)).astype(np.float32)
    out = empty((vectors, d))
    qd.linear_into(act, vectors, out, residual=dev(residual), epilogue=et.EPILOGUE_RESIDUAL)
    got = host(out)
    for a, b in row_slices(d):
        expected = residual[:, a:b] + orc.qlinear(orc.Q4_0, got_act, pd[a:b].cpu().numpy(), b - a, ffn, threads=THREADS)
        assert helpers.rel_err(got[:, a:b], expected) <= REL_TOL, f"down rows {a}..{b}"
    qgu.close()
    qd.close()


def shuffled_pool(rt, kv_heads, head_dim, pages, seed):
    """A pool whose free pages come back in a seeded random order: every page is handed to a one-page sequence and the
    sequences are released in shuffled order, so later allocations draw page numbers like a permutation of the pool."""
    pool = et.NativeKvPool(rt, 1, kv_heads, head_dim, pages * 16, 16, et.KV_F16)
    holders = [pool.makeSequence() for _ in range(pages)]
    zeros = torch.zeros((64, kv_heads, 16, head_dim), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    for i in range(0, pages, 64):
        group = holders[i:i + 64]
        rt.kv_append_into(pool, 0, group, len(group), len(group), 16, zeros, zeros, 16)  # allocates one page each; nothing committed
    assert pool.freeBlocks == 0
    for i in np.random.default_rng(seed).permutation(pages):
        holders[int(i)].release()
    assert pool.freeBlocks == pages
    return pool


def test_paged_attention_at_the_microbenchmark_shape_over_shuffled_tables():
    """64 sequences, 32 query / 8 KV heads of 128, f16 pages of 16 tokens, contexts ~U[128, 4096], page tables drawn from a
    shuffled pool; the oracle checks the shortest, the longest and two other lanes."""
    rt = runtime()
    B, Hq, Hkv, D = 64, 32, 8, 128
    rng = np.random.default_rng(1)
    ctx = rng.integers(128, 4097, size=B)
    order = np.argsort(-ctx)  # lanes sorted by length so that the appends below can run batched
    pages = int(np.ceil((ctx + 1) / 16).sum()) + 64
    pool = shuffled_pool(rt, Hkv, D, pages, seed=7)
    seqs = [pool.makeSequence() for _ in range(B)]
    checked = [int(order[0]), int(order[-1]), int(order[B // 3]), int(order[2 * B // 3])]
    kept = {lane: ([], []) for lane in checked}  # K and V rows of the checked lanes, in position order
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    chunk = 64
    sorted_ctx = ctx[order]
    for start in range(0, int(sorted_ctx.max()), chunk):
        active = int((sorted_ctx - start >= chunk).sum())  # lanes that still take a whole chunk
        if active:
            k = torch.randn((active, Hkv, chunk, D), generator=gen, device="cuda", dtype=torch.float32)
            v = torch.randn((active, Hkv, chunk, D), generator=gen, device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            group = [seqs[int(order[i])] for i in range(active)]
            rt.kv_append_into(pool, 0, group, active, active, chunk, k, v, chunk)
            for s in group:
                s.commit(np.arange(chunk, dtype=np.uint32))
            for i in range(active):
                if int(order[i]) in kept:
                    kept[int(order[i])][0].append(k[i].cpu().numpy())
                    kept[int(order[i])][1].append(v[i].cpu().numpy())
    for lane in range(B):  # ragged tails, one lane at a time
        tail = int(ctx[lane]) % chunk
        if tail:
            k = torch.randn((1, Hkv, tail, D), generator=gen, device="cuda", dtype=torch.float32)
            v = torch.randn((1, Hkv, tail, D), generator=gen, device="cuda", dtype=torch.float32)
            torch.cuda.synchronize()
            rt.kv_append_into(pool, 0, [seqs[lane]], 1, 1, tail, k, v, tail)
            seqs[lane].commit(np.arange(tail, dtype=np.uint32))
            if lane in kept:
                kept[lane][0].append(k[0].cpu().numpy())
                kept[lane][1].append(v[0].cpu().numpy())
    assert [s.cursor for s in seqs] == [int(c) for c in ctx]
    tables = [seqs[lane].blocks[0] for lane in checked]
    assert any(np.any(np.diff(t.astype(np.int64)) != 1) for t in tables), "page tables are not shuffled"
    q = rng.normal(size=(B, Hq, D)).astype(np.float32)
    k1 = rng.normal(size=(B, Hkv, D)).astype(np.float32)
    v1 = rng.normal(size=(B, Hkv, D)).astype(np.float32)
    out = empty((B, Hq, D))
    scale = 1.0 / np.sqrt(D)
    rt.kv_attention_decode_into(pool, 0, seqs, B, B, dev(q), dev(k1), dev(v1), Hq, scale, out=out)
    got = host(out)
    for lane in checked:
        n = int(ctx[lane])
        keys = np.concatenate(kept[lane][0], axis=1)      # [Hkv, n, D]
        values = np.concatenate(kept[lane][1], axis=1)
        assert keys.shape[1] == n
        opool = orc.Pool(1, Hkv, D, (n // 16 + 2) * 16, 16, orc.F16)
        oseq = opool.make_sequence()
        for _ in range(n // 16 + 1):
            oseq.push_block(opool.alloc_block())
        rows = np.concatenate([np.arange(16) + int(b) * 16 for b in oseq.blocks])[:n]
        opool.write_rows(0, 0, rows, np.ascontiguousarray(keys.transpose(1, 0, 2).reshape(n, Hkv * D)))
        opool.write_rows(0, 1, rows, np.ascontiguousarray(values.transpose(1, 0, 2).reshape(n, Hkv * D)))
        oseq.set_cursor(n)
        oseq.set_advance(1)
        expected = orc.kv_attention(opool, 0, [oseq], 1, q[lane:lane + 1, :, None, :], k1[lane:lane + 1, :, None, :],
                                    v1[lane:lane + 1, :, None, :], scale, mode=1, threads=THREADS)
        assert helpers.rel_err(got[lane], expected[0, :, 0, :]) <= REL_TOL, f"lane {lane} (context {n})"
    # the same attention through the host-state-free operator over device-resident lane descriptors and tables
    lanes = np.zeros((B, 4), dtype=np.int32)
    flat = []
    for lane in range(B):
        blocks, head = seqs[lane].blocks
        lanes[lane] = (int(ctx[lane]), 1, 0, len(flat) - head)
        flat.extend(int(b) for b in blocks)
    max_pages = int(np.ceil((ctx + 1) / 16).max())
    plan = et.attention_plan(B, Hq, Hkv, D, max_pages, sm_count=rt.capabilities()["sm_count"])
    scratch = torch.empty(max(plan["partial_bytes"], 4), dtype=torch.uint8, device="cuda")
    out2 = empty((B, Hq, D))
    dq = dev(q)
    rt.paged_attention_into(pool, 0, dev(lanes), dev(np.asarray(flat, dtype=np.int32)), B, max_pages, dq, Hq, scale, out2, scratch,
                            plan["partial_bytes"])
    np.testing.assert_array_equal(host(out2), got)


def test_two_layer_decoder_at_the_8b_width_and_batch_32():
    """d_model 4096, 32 query / 8 KV heads of 128, FFN 14336, vocabulary 128256, Q4_0 projections and head, f16 KV, batch
    32: a teacher-forced chunk and three one-token steps against the oracle decoder (logits within 2e-3)."""
    cfg = dict(layers=2, d_model=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256, rms_eps=1e-5, rope_theta=500000.0)
    rt = runtime()
    B, max_tokens = 32, 32 * 64
    gdec = et.Executable(rt, layers=cfg["layers"], d_model=cfg["d_model"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                         head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], rms_eps=cfg["rms_eps"], rope_theta=cfg["rope_theta"],
                         batch=B, max_tokens=max_tokens, block_size=16, kv_dtype=et.KV_F16, exact=False, max_advance=4)
    odec = orc.Decoder(cfg["layers"], cfg["d_model"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                       eps=cfg["rms_eps"], theta=cfg["rope_theta"], batch=B)
    d, qw, kvw, ffn, V = 4096, 4096, 1024, 14336, 128256
    gen = torch.Generator(device="cuda")
    gen.manual_seed(21)

    def put_both(slot, layer, tensor, codec=0, rows=None, cols=None):
        torch.cuda.synchronize()
        gdec.set_weight(slot, layer, tensor, codec=codec, rows=rows, columns=cols)
        if codec:
            odec.set_weight(slot, layer, tensor.cpu().numpy(), codec=codec, rows=rows, columns=cols)
        else:
            odec.set_weight(slot, layer, tensor.cpu().numpy())

    embd = torch.randn((V, d), generator=gen, device="cuda", dtype=torch.float32) * 0.02
    put_both(et.W_TOK_EMBD, 0, embd)
    ones = torch.ones(d, device="cuda", dtype=torch.float32)
    seed = 100
    for l in range(cfg["layers"]):
        put_both(et.W_ATTN_NORM, l, ones)
        put_both(et.W_FFN_NORM, l, ones)
        for slot, (r, c) in ((et.W_Q, (qw, d)), (et.W_K, (kvw, d)), (et.W_V, (kvw, d)), (et.W_O, (d, qw)), (et.W_GATE, (ffn, d)),
                             (et.W_UP, (ffn, d)), (et.W_DOWN, (d, ffn))):
            seed += 1
            put_both(slot, l, device_quantized(orc.Q4_0, r, c, seed), orc.Q4_0, r, c)
    put_both(et.W_OUT_NORM, 0, ones)
    put_both(et.W_HEAD, 0, device_quantized(orc.Q4_0, V, d, 999), orc.Q4_0, V, d)
    del embd
    gdec.finalize()
    odec.set_mode(faithful=False, threads=THREADS)
    gpool = et.NativeKvPool(rt, cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, et.KV_F16)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, orc.F16)
    gseqs = [gpool.makeSequence() for _ in range(B)]
    oseqs = [opool.make_sequence() for _ in range(B)]
    rng = np.random.default_rng(4)
    worst = 0.0
    for advance in (4, 1, 1, 1):
        toks = rng.integers(0, V, size=(B, advance)).astype(np.uint32)
        ol, _ = odec.execute(opool, oseqs, toks)
        gl = gdec.execute(gpool, gseqs, toks)
        err = helpers.rel_err(gl, ol)
        worst = max(worst, err)
        assert err <= REL_TOL, f"advance {advance}: {err:.3e}"
    assert [s.cursor for s in gseqs] == [7] * B
    for gs, os_ in zip(gseqs, oseqs):
        np.testing.assert_array_equal(gs.blocks[0], os_.blocks)
