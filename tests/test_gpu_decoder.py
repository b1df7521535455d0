"""GPU parity of the compiled decoder against the CPU oracle: greedy token ids (exact) and teacher-forced
logits on the tiny f32 model, the quantized tensor-core path within the logits tolerance, and the stateful
transaction rules (padding, rollback, cancellation, device-resident generation)."""
import numpy as np
import pytest

import effect_torch_b200 as et
import oracle as orc
from tests import helpers
from tests.gpu_util import runtime

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-3  # north-star tolerance on logits (max |err| / max |ref|)


def gpu_decoder(cfg, weights, batch, max_tokens, block_size=16, kv_dtype=et.KV_F32, exact=True, max_advance=16, window=None):
    dec = et.Executable(runtime(), layers=cfg["layers"], d_model=cfg["d_model"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                        head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], rms_eps=cfg["rms_eps"],
                        rope_theta=cfg["rope_theta"], batch=batch, max_tokens=max_tokens, block_size=block_size, kv_dtype=kv_dtype,
                        exact=exact, max_advance=max_advance, window=window)
    helpers.load_into(dec, weights)
    dec.finalize()
    return dec


@pytest.fixture(scope="module")
def tiny():
    return helpers.make_weights(helpers.TINY, seed=0)


def test_tiny_model_greedy_tokens_match_the_oracle_exactly(tiny):
    """The reference's CPU-runnable configuration: 4 layers, d_model 256, 4 query x 64, 2 KV heads, FFN 688, vocab 4096,
    f32 weights and KV, 16-token pages; batch 4 prompts of 32 tokens prefetched in chunks of 16, then 64 greedy steps."""
    cfg = helpers.TINY
    rng = np.random.default_rng(0)
    prompts = rng.integers(0, cfg["vocab"], size=(4, 32)).astype(np.uint32)
    max_tokens = 4 * 96
    odec = helpers.oracle_decoder(cfg, tiny, batch=4)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, orc.F32)
    oseqs = [opool.make_sequence() for _ in range(4)]
    gdec = gpu_decoder(cfg, tiny, batch=4, max_tokens=max_tokens)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, et.KV_F32)
    gseqs = [gpool.makeSequence() for _ in range(4)]
    worst = 0.0
    for chunk in (prompts[:, :16], prompts[:, 16:]):
        ol, osamp = odec.execute(opool, oseqs, chunk)
        gl = gdec.execute(gpool, gseqs, chunk)
        worst = max(worst, helpers.rel_err(gl, ol))
    otok = osamp.copy()
    gtok = np.asarray([orc.argmax(r) for r in gl], dtype=np.uint32)
    np.testing.assert_array_equal(gtok, otok)
    first_divergence = None
    for step in range(64):
        ol, onext = odec.execute(opool, oseqs, otok[:, None])
        gnext = gdec.executeSampled(gpool, gseqs, gtok[:, None])
        if first_divergence is None and not np.array_equal(onext, gnext):
            first_divergence = step
        otok, gtok = onext, gnext
    assert first_divergence is None, f"greedy tokens diverged at step {first_divergence}"
    assert worst <= 1e-5
    assert [s.cursor for s in gseqs] == [s.cursor for s in oseqs] == [96] * 4
    for gs, os_ in zip(gseqs, oseqs):
        np.testing.assert_array_equal(gs.blocks[0], os_.blocks)


def test_tiny_model_teacher_forced_logits(tiny):
    # the reference's own answer to argmax instability: compare logits under identical forced tokens
    cfg = helpers.TINY
    rng = np.random.default_rng(1)
    odec = helpers.oracle_decoder(cfg, tiny, batch=2)
    gdec = gpu_decoder(cfg, tiny, batch=2, max_tokens=128)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, orc.F32)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, et.KV_F32)
    oseqs = [opool.make_sequence() for _ in range(2)]
    gseqs = [gpool.makeSequence() for _ in range(2)]
    for advance in (7, 1, 1, 16, 1, 3):
        toks = rng.integers(0, cfg["vocab"], size=(2, advance)).astype(np.uint32)
        ol, _ = odec.execute(opool, oseqs, toks)
        gl = gdec.execute(gpool, gseqs, toks)
        assert helpers.rel_err(gl, ol) <= 1e-5


@pytest.mark.parametrize("codec", [orc.Q4_0, orc.Q8_0])
@pytest.mark.parametrize("kv_dtype,okv,tol", [(et.KV_F16, orc.F16, LOGIT_TOL), (et.KV_F32, orc.F32, LOGIT_TOL), (et.KV_U8, orc.U8, 1e-2)])
def test_quantized_model_on_the_tensor_core_path(codec, kv_dtype, okv, tol):
    """Block-quantized projections on the tiled MMA kernels (and, with an f16 or int8 pool, the flash-decoding kernel)
    against the oracle running the same packed bytes: teacher-forced logits within 2e-3. The int8 tier gets 1e-2: the f16
    linears move a K / V row by about 1e-3, which flips codes of its int8 image by one step (1/127 of the row's maximum),
    so the two sides attend over slightly different caches; on identical cache contents the int8 attention itself holds
    2e-3 (tests/test_gpu_attention.py)."""
    cfg = helpers.TINY_Q
    w = helpers.make_weights(cfg, seed=3, codec=codec)
    rng = np.random.default_rng(2)
    B = 3
    odec = helpers.oracle_decoder(cfg, w, batch=B)
    gdec = gpu_decoder(cfg, w, batch=B, max_tokens=256, kv_dtype=kv_dtype, exact=False, max_advance=8)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 256, 16, okv)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 256, 16, kv_dtype)
    oseqs = [opool.make_sequence() for _ in range(B)]
    gseqs = [gpool.makeSequence() for _ in range(B)]
    for advance in (8, 8, 5, 1, 1, 1, 1):
        toks = rng.integers(0, cfg["vocab"], size=(B, advance)).astype(np.uint32)
        ol, _ = odec.execute(opool, oseqs, toks)
        gl = gdec.execute(gpool, gseqs, toks)
        assert helpers.rel_err(gl, ol) <= tol, f"advance {advance}"
    assert gdec.diagnostics()["launches_per_step"] > 0


K_MIXES = {
    # what the GGUF "medium" recipes produce: v (and down) at more bits than q / k in some layers
    "q4_k_m": dict(wq=orc.Q4_K, wk=orc.Q4_K, wv=orc.Q6_K, wo=orc.Q4_K, gate=orc.Q4_K, up=orc.Q4_K, down=orc.Q6_K, head=orc.Q6_K),
    "q3_k_m": dict(wq=orc.Q3_K, wk=orc.Q3_K, wv=orc.Q5_K, wo=orc.Q4_K, gate=orc.Q3_K, up=orc.Q3_K, down=orc.Q5_K, head=orc.Q6_K),
    "all_different": dict(wq=orc.Q5_K, wk=orc.Q3_K, wv=orc.Q4_K, wo=orc.Q5_K, gate=orc.Q5_K, up=orc.Q5_K, down=orc.Q3_K, head=orc.Q4_K),
}


@pytest.mark.parametrize("mix", sorted(K_MIXES))
def test_k_quant_model_with_mixed_codecs_stays_on_the_tensor_core_path(mix):
    """Projections of different K-quants in one model, q / k / v of a layer included: the fused q/k/v weight holds one
    segment per codec and the step keeps its tiled kernels (one more launch per extra segment and layer than a model of a
    single codec). Teacher-forced logits against the oracle decoding the same packed bytes, within 4e-3: the re-cut rounds
    every effective scale d*sc and minimum dmin*m to f16 once, at load, which is systematic over 32 values (it alone moves
    these logits by 7e-4 when the oracle is run on the rounded weights) and comes on top of the f16 rounding of weights
    and activations that every tiled model has; random code bytes with sub-scales uniform over 0..63 are the worst case."""
    cfg = helpers.TINY_Q
    codecs = K_MIXES[mix]
    w = helpers.make_mixed_weights(cfg, codecs, seed=6)
    rng = np.random.default_rng(7)
    B = 3
    odec = helpers.oracle_decoder(cfg, w, batch=B)
    gdec = gpu_decoder(cfg, w, batch=B, max_tokens=256, kv_dtype=et.KV_F16, exact=False, max_advance=8)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 256, 16, orc.F16)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 256, 16, et.KV_F16)
    oseqs = [opool.make_sequence() for _ in range(B)]
    gseqs = [gpool.makeSequence() for _ in range(B)]
    for advance in (8, 5, 1, 1, 1):
        toks = rng.integers(0, cfg["vocab"], size=(B, advance)).astype(np.uint32)
        ol, _ = odec.execute(opool, oseqs, toks)
        gl = gdec.execute(gpool, gseqs, toks)
        assert helpers.rel_err(gl, ol) <= 2 * LOGIT_TOL, f"advance {advance}"
    uniform = gpu_decoder(cfg, helpers.make_mixed_weights(cfg, {name: orc.Q4_K for name in codecs}, seed=6), batch=B, max_tokens=256,
                          kv_dtype=et.KV_F16, exact=False, max_advance=8)
    upool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 256, 16, et.KV_F16)
    useqs = [upool.makeSequence() for _ in range(B)]
    uniform.execute(upool, useqs, toks)
    segments = len({codecs["wq"], codecs["wk"]}) + (codecs["wv"] != codecs["wk"])
    assert gdec.diagnostics()["launches_per_step"] == uniform.diagnostics()["launches_per_step"] + cfg["layers"] * (segments - 1)


def test_device_resident_generation_equals_stepwise_execution():
    cfg = helpers.TINY_Q
    w = helpers.make_weights(cfg, seed=4, codec=orc.Q4_0)
    B, steps = 4, 40
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg["vocab"], size=(B, 8)).astype(np.uint32)
    first = rng.integers(0, cfg["vocab"], size=B).astype(np.uint32)
    results = []
    for mode in ("stepwise", "resident"):
        dec = gpu_decoder(cfg, w, batch=B, max_tokens=512, kv_dtype=et.KV_F16, exact=False, max_advance=8)
        pool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 512, 16, et.KV_F16)
        seqs = [pool.makeSequence() for _ in range(B)]
        dec.execute(pool, seqs, prompt)
        if mode == "stepwise":
            tok, out = first, []
            for _ in range(steps):
                tok = dec.executeSampled(pool, seqs, tok[:, None])
                out.append(tok)
            results.append(np.stack(out))
        else:
            out, ms = dec.generate_greedy(pool, seqs, first, steps)
            assert ms > 0
            results.append(out)
        assert [s.cursor for s in seqs] == [8 + steps] * B
    np.testing.assert_array_equal(results[0], results[1])


def test_transaction_rollback_padding_and_cancellation(tiny):
    cfg = helpers.TINY
    gdec = gpu_decoder(cfg, tiny, batch=4, max_tokens=32, max_advance=16)
    pool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 32, 16, et.KV_F32)
    a, b = pool.makeSequence(), pool.makeSequence()
    toks = np.arange(32, dtype=np.uint32).reshape(2, 16)
    logits = gdec.execute(pool, [a, b], toks)  # 2 active of 4 lanes
    assert logits.shape == (2, cfg["vocab"]) and (a.cursor, b.cursor) == (16, 16)
    # single-lane run of the same tokens gives the same logits (padding is inert)
    pool1 = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 32, 16, et.KV_F32)
    s1 = pool1.makeSequence()
    np.testing.assert_array_equal(gdec.execute(pool1, [s1], toks[:1])[0], logits[0])
    free_before = pool.freeBlocks
    with pytest.raises(et.BackendError, match="pool exhausted") as e:
        gdec.executeSampled(pool, [a, b], np.asarray([[1], [2]], dtype=np.uint32))
    assert e.value.reason == "execution-failed"
    assert (a.cursor, b.cursor) == (16, 16) and pool.freeBlocks == free_before
    with pytest.raises(et.BackendError, match="^operation aborted$") as e:
        gdec.executeSampled(pool1, [s1], np.asarray([[1]], dtype=np.uint32), cancelled=True)
    assert e.value.reason == "cancelled" and s1.cursor == 16
    with pytest.raises(et.BackendError, match=r"accepts 1\.\.=4 sequences"):
        gdec.execute(pool, [a, b, a, b, a], np.zeros((5, 1), dtype=np.uint32))
    with pytest.raises(et.BackendError, match="duplicate sequence"):
        gdec.execute(pool, [a, a], np.zeros((2, 1), dtype=np.uint32))
    other = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 64, 16, et.KV_F32)
    with pytest.raises(et.BackendError, match="does not match the compiled state schema"):
        gdec.execute(other, [other.makeSequence()], np.zeros((1, 1), dtype=np.uint32))
    with pytest.raises(et.BackendError, match="is outside 0..4096"):
        gdec.execute(pool1, [s1], np.asarray([[5000]], dtype=np.uint32))
    assert s1.cursor == 16  # the failed step rolled back
    b.release()
    with pytest.raises(et.BackendError, match="kv sequence 1 is released"):
        gdec.execute(pool, [a, b], np.zeros((2, 1), dtype=np.uint32))


def test_sliding_window_decoder_matches_the_oracle():
    cfg = dict(helpers.TINY_Q, layers=2)
    w = helpers.make_weights(cfg, seed=6)
    odec = orc.Decoder(cfg["layers"], cfg["d_model"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                       eps=cfg["rms_eps"], theta=cfg["rope_theta"], window=20, batch=1)
    helpers.load_into(odec, w)
    odec.set_mode(False, 4)
    gdec = gpu_decoder(cfg, w, batch=1, max_tokens=48, window=20, max_advance=1)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 48, 16, orc.F32)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 48, 16, et.KV_F32)
    os_, gs = opool.make_sequence(), gpool.makeSequence()
    tok = np.asarray([[3]], dtype=np.uint32)
    for step in range(70):  # cursor runs far past the 48-token pool
        ol, onext = odec.execute(opool, [os_], tok)
        gl = gdec.execute(gpool, [gs], tok)
        assert helpers.rel_err(gl, ol) <= 1e-5, f"step {step}"
        tok = onext[:, None]
    assert gs.cursor == os_.cursor == 70
    np.testing.assert_array_equal(gs.blocks[0], os_.blocks)
    assert gs.blocks[1] == os_.head


@pytest.mark.parametrize("batch", [40, 70])
def test_wide_batches_keep_the_f16_hand_off_path(batch):
    """33..128 sequences per step: activations still travel between kernels in the tensor-core operand layout, with a
    row stride of 64 or 128; teacher-forced logits against the oracle like the narrow case."""
    cfg = helpers.TINY_Q
    w = helpers.make_weights(cfg, seed=9, codec=orc.Q4_0)
    rng = np.random.default_rng(batch)
    max_tokens = batch * 48
    odec = helpers.oracle_decoder(cfg, w, batch=batch)
    gdec = gpu_decoder(cfg, w, batch=batch, max_tokens=max_tokens, kv_dtype=et.KV_F16, exact=False, max_advance=8)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, orc.F16)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], max_tokens, 16, et.KV_F16)
    oseqs = [opool.make_sequence() for _ in range(batch)]
    gseqs = [gpool.makeSequence() for _ in range(batch)]
    for advance in (8, 1, 1, 1):
        toks = rng.integers(0, cfg["vocab"], size=(batch, advance)).astype(np.uint32)
        ol, _ = odec.execute(opool, oseqs, toks)
        gl = gdec.execute(gpool, gseqs, toks)
        assert helpers.rel_err(gl, ol) <= LOGIT_TOL, f"advance {advance}"
    # fewer active sequences than the batch: padded lanes stay out of the result
    toks = rng.integers(0, cfg["vocab"], size=(batch - 5, 1)).astype(np.uint32)
    ol, _ = odec.execute(opool, oseqs[:batch - 5], toks)
    gl = gdec.execute(gpool, gseqs[:batch - 5], toks)
    assert helpers.rel_err(gl, ol) <= LOGIT_TOL


def test_captured_step_plans_fit_the_reserved_partials_at_awkward_capacities():
    """max_tokens = 400 (25 pages), one lane: once the context passes 384 tokens the captured step plans for 32 pages,
    one split more than any table length up to the capacity needs. Logits must stay on the oracle through that range
    (the partials of the extra split have to land inside the decoder's reserve)."""
    cfg = dict(helpers.TINY_Q, layers=2)
    w = helpers.make_weights(cfg, seed=12, codec=orc.Q4_0)
    rng = np.random.default_rng(12)
    odec = helpers.oracle_decoder(cfg, w, batch=1)
    gdec = gpu_decoder(cfg, w, batch=1, max_tokens=400, kv_dtype=et.KV_F16, exact=False, max_advance=16)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 400, 16, orc.F16)
    gpool = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 400, 16, et.KV_F16)
    os_, gs = opool.make_sequence(), gpool.makeSequence()
    for _ in range(23):  # 368 tokens in chunks of 16
        toks = rng.integers(0, cfg["vocab"], size=(1, 16)).astype(np.uint32)
        odec.execute(opool, [os_], toks, want_logits=False, want_sampled=False)
        gdec.execute(gpool, [gs], toks)
    canary = gdec.execute(gpool, [gs], toks[:, :1])  # eager one-token step; later ones replay a captured graph
    odec.execute(opool, [os_], toks[:, :1])
    assert np.isfinite(canary).all()
    for step in range(30):  # cursor 369 .. 399: crosses 384, where the page bucket becomes 32
        toks = rng.integers(0, cfg["vocab"], size=(1, 1)).astype(np.uint32)
        ol, _ = odec.execute(opool, [os_], toks)
        gl = gdec.execute(gpool, [gs], toks)
        assert helpers.rel_err(gl, ol) <= LOGIT_TOL, f"step {step} (cursor {gs.cursor})"
    assert gs.cursor == os_.cursor == 399


def test_a_recreated_pool_never_replays_the_old_pools_graph():
    """A captured step holds the pool's slab addresses. Destroying the pool and creating another one of the same
    schema (which may land at the same host address) must re-capture: the second pool's results equal a fresh run."""
    cfg = dict(helpers.TINY_Q, layers=2)
    w = helpers.make_weights(cfg, seed=13, codec=orc.Q4_0)
    rng = np.random.default_rng(13)
    prompt = rng.integers(0, cfg["vocab"], size=(2, 8)).astype(np.uint32)
    steps = rng.integers(0, cfg["vocab"], size=(6, 2, 1)).astype(np.uint32)
    gdec = gpu_decoder(cfg, w, batch=2, max_tokens=128, kv_dtype=et.KV_F16, exact=False, max_advance=8)

    def run(pool):
        seqs = [pool.makeSequence() for _ in range(2)]
        gdec.execute(pool, seqs, prompt)
        return np.stack([gdec.execute(pool, seqs, t) for t in steps])

    pool_a = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, et.KV_F16)
    first = run(pool_a)
    # occupy pool A's pages with other contents before it goes away, so a replay against stale addresses would show
    pool_a.close()
    filler = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, et.KV_F16)
    pool_b = et.NativeKvPool(runtime(), cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, et.KV_F16)
    second = run(pool_b)
    np.testing.assert_array_equal(second, first)
    del filler


def test_the_operator_by_operator_route_agrees_with_the_fused_decoder():
    """A backend that lowers the specialised decode graph node by node (QuantizedEmbedding, RmsNorm, QuantizedLinear,
    RotaryEmbedding{Cursor}, KvAttention, SwiGLU, Add, LastTokenRow: crates/compiler/src/decode.rs:105-481) calls one C-ABI
    operator per node. That route, the fused decoder and the CPU oracle must tell the same story for a prefill chunk and two
    decode steps of a small quantized model (tensors only change layout between operators here, through torch views)."""
    import torch
    from tests.gpu_util import dev, empty, host

    rt = runtime()
    cfg = helpers.TINY_Q
    codec = orc.Q4_0
    weights = helpers.make_weights(cfg, seed=4, codec=codec)
    weights["tok_embd"] = (orc.quantize(codec, weights["tok_embd"]),) + weights["tok_embd"].shape  # QuantizedEmbedding
    B, max_tokens = 2, 128
    L, d, Hq, Hkv, D, ffn, V = (cfg[k] for k in ("layers", "d_model", "q_heads", "kv_heads", "head_dim", "ffn", "vocab"))
    fused = gpu_decoder(cfg, weights, B, max_tokens, kv_dtype=et.KV_F16, exact=False, max_advance=8)
    odec = helpers.oracle_decoder(cfg, weights, batch=B)
    pool_fused = et.NativeKvPool(rt, L, Hkv, D, max_tokens, 16, et.KV_F16)
    pool_ops = et.NativeKvPool(rt, L, Hkv, D, max_tokens, 16, et.KV_F16)
    opool = orc.Pool(L, Hkv, D, max_tokens, 16, orc.F16)
    seqs_fused = [pool_fused.makeSequence() for _ in range(B)]
    seqs_ops = [pool_ops.makeSequence() for _ in range(B)]
    oseqs = [opool.make_sequence() for _ in range(B)]
    w = {name: [dev(layer[name][0]) if isinstance(layer[name], tuple) else dev(layer[name]) for layer in weights["layers"]]
         for name in helpers.SLOTS}
    embd, head, out_norm = dev(weights["tok_embd"][0]), dev(weights["head"][0]), dev(weights["out_norm"])

    def linear(x, rows_in, weight, n, k):
        out = empty((rows_in, n))
        rt.qlinear_into(codec, x, rows_in, k, weight, n, None, out)
        return out

    def step_by_operators(tokens):
        T = tokens.shape[1]
        R = B * T
        cursors = dev(np.array([s.cursor for s in seqs_ops], dtype=np.int64))
        hidden = empty((R, d))
        rt.qembedding_into(codec, dev(tokens.reshape(-1).astype(np.uint32)), False, R, embd, V, d, hidden)
        for l in range(L):
            normed = empty((R, d))
            rt.rmsnorm_into(hidden, w["attn_norm"][l], cfg["rms_eps"], R, d, normed)
            q, k, v = (linear(normed, R, w[n][l], width, d) for n, width in (("wq", Hq * D), ("wk", Hkv * D), ("wv", Hkv * D)))
            rt.synchronize()
            heads_first = lambda x, h: x.view(B, T, h, D).permute(0, 2, 1, 3).contiguous()  # [B, H, T, D]
            qh, kh, vh = heads_first(q, Hq), heads_first(k, Hkv), heads_first(v, Hkv)
            torch.cuda.synchronize()
            qr, kr = empty((B, Hq, T, D)), empty((B, Hkv, T, D))
            rt.rope_into(qh, cursors, B, cfg["rope_theta"], et.HALF_SPLIT, B, Hq, T, D, qr)
            rt.rope_into(kh, cursors, B, cfg["rope_theta"], et.HALF_SPLIT, B, Hkv, T, D, kr)
            att = empty((B, Hq, T, D))
            rt.kv_attention_into(pool_ops, l, seqs_ops, B, B, T, qr, kr, vh, Hq, T, 1.0 / np.sqrt(D), out=att)
            rt.synchronize()
            att_rows = att.permute(0, 2, 1, 3).contiguous().view(R, Hq * D)
            torch.cuda.synchronize()
            o = linear(att_rows, R, w["wo"][l], d, Hq * D)
            rt.add_into(hidden, o, R * d, hidden)
            rt.rmsnorm_into(hidden, w["ffn_norm"][l], cfg["rms_eps"], R, d, normed)
            gate, up = linear(normed, R, w["gate"][l], ffn, d), linear(normed, R, w["up"][l], ffn, d)
            act = empty((R, ffn))
            rt.swiglu_into(gate, up, R * ffn, act)
            down = linear(act, R, w["down"][l], d, ffn)
            rt.add_into(hidden, down, R * d, hidden)
        normed = empty((R, d))
        rt.rmsnorm_into(hidden, out_norm, cfg["rms_eps"], R, d, normed)
        rt.synchronize()
        last = normed.view(B, T, d)[:, T - 1, :].contiguous()  # LastTokenRow
        torch.cuda.synchronize()
        logits = linear(last, B, head, V, d)
        picked = empty(B, dtype=torch.int32)
        rt.argmax_into(logits, B, V, picked)
        result = host(logits)
        for s, row in zip(seqs_ops, tokens):
            s.commit(row)
        return result, host(picked)

    rng = np.random.default_rng(8)
    for advance in (8, 1, 1):
        tokens = rng.integers(0, V, size=(B, advance)).astype(np.uint32)
        by_ops, picked = step_by_operators(tokens)
        by_decoder = fused.execute(pool_fused, seqs_fused, tokens)
        by_oracle, _ = odec.execute(opool, oseqs, tokens)
        assert helpers.rel_err(by_ops, by_oracle) <= LOGIT_TOL, f"operators vs oracle, advance {advance}"
        assert helpers.rel_err(by_decoder, by_oracle) <= LOGIT_TOL, f"decoder vs oracle, advance {advance}"
        assert helpers.rel_err(by_ops, by_decoder) <= LOGIT_TOL, f"operators vs decoder, advance {advance}"
        np.testing.assert_array_equal(picked, by_ops.argmax(axis=1))
        assert [s.cursor for s in seqs_ops] == [s.cursor for s in seqs_fused]
