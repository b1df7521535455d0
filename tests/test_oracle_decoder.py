"""Decoder-level checks of the CPU oracle, following the reference's own integration recipe
(packages/core/test/Inference.test.ts): cached paged generation equals naive full-recompute generation
token for token, chunked prefill and batching do not change results, failures roll back."""
import numpy as np
import pytest

import oracle as orc
from tests import helpers

CFG = dict(layers=2, d_model=64, q_heads=4, kv_heads=2, head_dim=16, ffn=96, vocab=128, rms_eps=1e-5, rope_theta=10000.0)


def naive_logits(cfg, w, tokens):
    """Full recompute over the whole sequence with dense causal attention; returns last-row logits."""
    T = len(tokens)
    Hq, Hkv, D = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
    h = w["tok_embd"][np.asarray(tokens)]
    for layer in w["layers"]:
        a = orc.rms_norm(h, layer["attn_norm"], cfg["rms_eps"])
        q = orc.linear_rows(a, layer["wq"]).reshape(1, T, Hq, D).transpose(0, 2, 1, 3)
        k = orc.linear_rows(a, layer["wk"]).reshape(1, T, Hkv, D).transpose(0, 2, 1, 3)
        v = orc.linear_rows(a, layer["wv"]).reshape(1, T, Hkv, D).transpose(0, 2, 1, 3)
        q = orc.rotary(np.ascontiguousarray(q), [0], cfg["rope_theta"])
        k = orc.rotary(np.ascontiguousarray(k), [0], cfg["rope_theta"])
        att = orc.sdpa_forward(q, k, np.ascontiguousarray(v), 1 / np.sqrt(D), True)
        att = att.transpose(0, 2, 1, 3).reshape(T, Hq * D)
        h = h + orc.linear_rows(att, layer["wo"])
        f = orc.rms_norm(h, layer["ffn_norm"], cfg["rms_eps"])
        h = h + orc.linear_rows(orc.silu_mul(orc.linear_rows(f, layer["gate"]), orc.linear_rows(f, layer["up"])), layer["down"])
    h = orc.rms_norm(h, w["out_norm"], cfg["rms_eps"])
    return orc.linear_rows(h[-1:], w["head"])[0]


@pytest.fixture(scope="module")
def model():
    w = helpers.make_weights(CFG, seed=11)
    return w


def test_cached_generation_matches_naive_generation_across_block_boundaries(model):
    # Inference.test.ts:280-291 — block size 4 so several page boundaries are crossed
    dec = helpers.oracle_decoder(CFG, model, batch=1)
    pool = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 32, 4, orc.F32)
    seq = pool.make_sequence()
    prompt = [3, 17, 99, 5, 42]
    logits, sampled = dec.execute(pool, [seq], np.asarray([prompt], dtype=np.uint32))
    history = list(prompt)
    for _ in range(9):
        ref = naive_logits(CFG, model, history)
        np.testing.assert_allclose(logits[0], ref, rtol=0, atol=1e-5)
        assert int(sampled[0]) == int(np.argmax(ref))
        history.append(int(sampled[0]))
        logits, sampled = dec.execute(pool, [seq], np.asarray([[history[-1]]], dtype=np.uint32))
    assert seq.cursor == len(history)


def test_chunked_prefill_equals_single_chunk(model):
    # Inference.test.ts:306-316
    dec = helpers.oracle_decoder(CFG, model, batch=1)
    prompt = np.arange(1, 12, dtype=np.uint32)
    pool_a = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 32, 4, orc.F32)
    sa = pool_a.make_sequence()
    la, _ = dec.execute(pool_a, [sa], prompt[None, :])
    pool_b = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 32, 4, orc.F32)
    sb = pool_b.make_sequence()
    for chunk in (prompt[:4], prompt[4:8], prompt[8:]):
        lb, _ = dec.execute(pool_b, [sb], chunk[None, :])
    np.testing.assert_allclose(la, lb, rtol=0, atol=1e-6)
    assert sa.cursor == sb.cursor == 11


def test_batched_equals_per_sequence_and_padding_is_inert(model):
    # Inference.test.ts:590-648
    dec4 = helpers.oracle_decoder(CFG, model, batch=4)
    dec1 = helpers.oracle_decoder(CFG, model, batch=1)
    pool = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 64, 4, orc.F32)
    prompts = [[5, 6, 7], [9, 10, 11], [1, 2, 3]]
    seqs = [pool.make_sequence() for _ in prompts]
    batched, _ = dec4.execute(pool, seqs, np.asarray(prompts, dtype=np.uint32))  # 3 active of 4 lanes
    for i, p in enumerate(prompts):
        solo_pool = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 64, 4, orc.F32)
        s = solo_pool.make_sequence()
        solo, _ = dec1.execute(solo_pool, [s], np.asarray([p], dtype=np.uint32))
        np.testing.assert_array_equal(batched[i], solo[0])
    assert [s.cursor for s in seqs] == [3, 3, 3]
    assert pool.free_blocks == 64 // 4 - 3  # padding lanes returned their (never allocated) blocks


def test_pool_exhaustion_rolls_back(model):
    # Inference.test.ts:693-714
    dec = helpers.oracle_decoder(CFG, model, batch=2)
    pool = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 8, 4, orc.F32)
    a, b = pool.make_sequence(), pool.make_sequence()
    dec.execute(pool, [a, b], np.asarray([[1, 2, 3, 4], [5, 6, 7, 8]], dtype=np.uint32))
    free_before = pool.free_blocks
    with pytest.raises(orc.OracleError, match="pool exhausted"):
        dec.execute(pool, [a, b], np.asarray([[9], [10]], dtype=np.uint32))
    assert (a.cursor, b.cursor) == (4, 4)
    assert pool.free_blocks == free_before
    assert len(a.blocks) == 1 and len(b.blocks) == 1


def test_prefix_cache_shares_whole_blocks(model):
    # Inference.test.ts:375-470
    dec = helpers.oracle_decoder(CFG, model, batch=1)
    pool = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 32, 4, orc.F32)
    prompt = np.arange(20, 31, dtype=np.uint32)  # 11 tokens -> 2 hashed blocks
    first = pool.make_sequence()
    l1, _ = dec.execute(pool, [first], prompt[None, :])
    first.release()
    assert pool.cached_blocks == 2
    second = pool.make_sequence()
    matched = second.prefill_match(prompt)
    assert matched == 8
    l2, _ = dec.execute(pool, [second], prompt[None, matched:])
    np.testing.assert_allclose(l1, l2, rtol=0, atol=1e-6)


def test_sliding_window_evicts_blocks_and_keeps_an_unbounded_cursor(model):
    # Inference.test.ts:1012-1028
    dec = orc.Decoder(CFG["layers"], CFG["d_model"], CFG["q_heads"], CFG["kv_heads"], CFG["head_dim"], CFG["ffn"], CFG["vocab"],
                      window=6, batch=1)
    helpers.load_into(dec, model)
    dec.set_mode(False, 2)
    pool = orc.Pool(CFG["layers"], CFG["kv_heads"], CFG["head_dim"], 12, 4, orc.F32)
    seq = pool.make_sequence()
    tok = 1
    for step in range(30):  # far past the pool's 12-token capacity
        _, sampled = dec.execute(pool, [seq], np.asarray([[tok]], dtype=np.uint32))
        tok = int(sampled[0])
    assert seq.cursor == 30
    assert seq.head > 0 and len(seq.blocks) - seq.head <= 3
