"""Pins the CPU oracle against the golden vectors held by the reference's own tests."""
import numpy as np
import pytest

import oracle as orc
from tests.golden import reference_vectors as gv

U64_MAX = np.iinfo(np.uint64).max


# ---------------------------------------------------------------- codecs
@pytest.mark.parametrize("codec", [gv.Q2_K, gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_k_quant_fixtures_decode_exactly(codec):
    block, _, _ = gv.K_QUANT_FIXTURES[codec]
    assert orc.block_bytes(codec) == block.size
    np.testing.assert_array_equal(orc.decode_block(codec, block), gv.fixture_expected(codec))


@pytest.mark.parametrize("codec", [gv.Q2_K, gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_decoder_rejects_noncanonical_block_lengths(codec):
    block, _, _ = gv.K_QUANT_FIXTURES[codec]
    with pytest.raises(orc.OracleError, match="expected"):
        orc.decode_block(codec, block[:-1])


@pytest.mark.parametrize("case", [gv.linear_prefill_case(), gv.linear_lowered_case()])
@pytest.mark.parametrize("threads", [0, 3])
def test_quantized_linear_golden(case, threads):
    out = orc.qlinear(case["codec"], case["x"], case["packed"], case["rows"], case["columns"], case["bias"], threads=threads)
    np.testing.assert_array_equal(out, case["expected"])


def test_quantized_linear_observes_cancellation():
    case = gv.linear_lowered_case()
    with pytest.raises(orc.OracleError, match="operation aborted"):
        orc.qlinear(case["codec"], case["x"], case["packed"], case["rows"], case["columns"], cancelled=True)


def test_invalid_row_width_is_rejected():
    assert orc.encoded_row_bytes(gv.Q4_K, 255) is None
    assert orc.encoded_row_bytes(gv.Q4_K, 512) == 288
    assert orc.encoded_row_bytes(gv.Q4_0, 4096) == 4096 // 32 * 18
    assert orc.encoded_row_bytes(gv.Q8_0, 4096) == 4096 // 32 * 34
    assert orc.encoded_row_bytes(gv.Q4_0, 48) is None


def test_embedding_decodes_only_selected_rows():
    # quantized.rs:867-897
    block, _, _ = gv.K_QUANT_FIXTURES[gv.Q5_K]
    packed = np.zeros((3, block.size), dtype=np.uint8)
    packed[1] = block
    out = orc.qembedding(gv.Q5_K, [1, 1], packed, 3, 256)
    np.testing.assert_array_equal(out[0], gv.fixture_expected(gv.Q5_K))
    np.testing.assert_array_equal(out[1], gv.fixture_expected(gv.Q5_K))


@pytest.mark.parametrize("index", [-1, 1])
def test_embedding_rejects_negative_and_out_of_range(index):
    # quantized.rs:899-921
    block, _, _ = gv.K_QUANT_FIXTURES[gv.Q2_K]
    with pytest.raises(orc.OracleError, match=r"outside 0\.\.1"):
        orc.qembedding(gv.Q2_K, [index], block.reshape(1, -1), 1, 256)


@pytest.mark.parametrize("codec", [gv.Q2_K, gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_mixed_codec_embedding(codec):
    # crates/runtime-cpu/src/executable.rs:4920-4956
    block, _, _ = gv.K_QUANT_FIXTURES[codec]
    out = orc.qembedding(codec, [0], block.reshape(1, -1), 1, 256)
    np.testing.assert_array_equal(out[0], gv.fixture_expected(codec))


# Q4_0 / Q8_0 are this build's additions (parity unpinned by the reference): self-consistency only.
@pytest.mark.parametrize("codec,step", [(gv.Q4_0, 1 / 8), (gv.Q8_0, 1 / 127)])
def test_block32_codecs_round_trip(codec, step):
    rng = np.random.default_rng(5)
    w = rng.normal(0, 0.02, size=(7, 128)).astype(np.float32)
    packed = orc.quantize(codec, w)
    assert packed.shape == (7, orc.encoded_row_bytes(codec, 128))
    deq = orc.dequantize(codec, packed, 7, 128)
    blocks = w.reshape(7, 4, 32)
    # one quantisation step bounds the error (Q4_0's range is -8..7, so the far side may clamp by a step)
    bound = np.abs(blocks).max(axis=2, keepdims=True) * step * 1.02 + 1e-6
    assert (np.abs(deq.reshape(7, 4, 32) - blocks) <= bound).all()
    # every dequantised value is exactly f32(scale) * integer code
    for r in range(7):
        for b in range(4):
            raw = packed[r, b * orc.block_bytes(codec):(b + 1) * orc.block_bytes(codec)]
            d = np.frombuffer(raw[:2].tobytes(), dtype=np.float16)[0].astype(np.float32)
            if codec == gv.Q4_0:
                codes = np.concatenate([raw[2:] & 0xF, raw[2:] >> 4]).astype(np.int32) - 8
            else:
                codes = raw[2:].view(np.int8).astype(np.int32)
            np.testing.assert_array_equal(deq[r, b * 32:(b + 1) * 32], d * codes.astype(np.float32))


def test_q4_0_known_block():
    # scale 0.5 (f16 0x3800), bytes 0x10..0x1f: low nibbles 0..15, high nibble 1
    block = np.zeros(18, dtype=np.uint8)
    block[0:2] = [0x00, 0x38]
    block[2:18] = np.arange(16) | 0x10
    out = orc.decode_block(gv.Q4_0, block)
    np.testing.assert_array_equal(out[:16], 0.5 * (np.arange(16) - 8))
    np.testing.assert_array_equal(out[16:], np.full(16, 0.5 * (1 - 8)))


def test_q8_0_known_block():
    block = np.zeros(34, dtype=np.uint8)
    block[0:2] = [0x00, 0x3C]  # 1.0
    block[2:34] = np.arange(-16, 16).astype(np.int8).view(np.uint8)
    np.testing.assert_array_equal(orc.decode_block(gv.Q8_0, block), np.arange(-16, 16).astype(np.float32))


# ---------------------------------------------------------------- dense ops
def test_matmul_is_sequential_fma():
    rng = np.random.default_rng(0)
    a = rng.normal(size=(3, 37)).astype(np.float32)
    w = rng.normal(size=(5, 37)).astype(np.float32)
    out = orc.matmul(a, w.T)
    ref = np.empty((3, 5), dtype=np.float32)
    for i in range(3):
        for j in range(5):
            acc = np.float64(0)
            accf = np.float32(0)
            for k in range(37):
                # fma(a,b,c) in f32 == round_f32(exact a*b + c); the exact product fits in f64
                accf = np.float32(np.float64(a[i, k]) * np.float64(w[j, k]) + np.float64(accf))
            ref[i, j] = accf
    np.testing.assert_array_equal(out, ref)
    np.testing.assert_array_equal(orc.linear_rows(a, w, threads=2), ref)


def test_rms_norm_matches_f64_formula():
    rng = np.random.default_rng(1)
    x = rng.normal(size=(4, 256)).astype(np.float32)
    w = rng.normal(size=256).astype(np.float32)
    x64 = x.astype(np.float64)
    ms = np.zeros(4)
    for i in range(256):
        ms += x64[:, i] * x64[:, i]
    scale = 1.0 / np.sqrt(ms / 256 + 1e-5)
    ref = (x64 * scale[:, None] * w.astype(np.float64)).astype(np.float32)
    np.testing.assert_array_equal(orc.rms_norm(x, w, 1e-5), ref)
    np.testing.assert_array_equal(orc.rms_norm(x, None, 1e-5), (x64 * scale[:, None]).astype(np.float32))


def test_rope_both_layouts_golden():
    x, half, inter = gv.rope_case()
    # rotaryEmbedding(x, seqLen 2, theta): positions 0 and 1 along dim -2, offset 0
    np.testing.assert_allclose(orc.rotary(x, [0], 10000.0, orc.HALF_SPLIT).reshape(-1), half, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(orc.rotary(x, [0], 10000.0, orc.INTERLEAVED).reshape(-1), inter, rtol=1e-6, atol=1e-6)


def test_rope_cursor_offsets_are_per_batch_lane():
    rng = np.random.default_rng(2)
    x = rng.normal(size=(3, 2, 1, 8)).astype(np.float32)
    out = orc.rotary(x, [5, 0, 9], 10000.0)
    for b, off in enumerate([5, 0, 9]):
        np.testing.assert_array_equal(out[b], orc.rotary(x[b:b + 1], [off], 10000.0)[0])


def test_silu_is_the_tanh_form():
    x = np.linspace(-6, 6, 41).astype(np.float32)
    u = np.full_like(x, 2.0)
    ref = x * (np.tanh(x / np.float32(2)) / np.float32(2) + np.float32(0.5)) * u
    np.testing.assert_allclose(orc.silu_mul(x, u), ref.astype(np.float32), rtol=1e-6, atol=1e-6)  # tanhf implementations differ in the last ulp


# ---------------------------------------------------------------- attention
def test_gqa_matches_repeated_heads():
    # packages/core/test/Attention.test.ts:188-215
    for hq, hkv in [(4, 2), (16, 1)]:
        q = np.asarray(gv.pattern(hq * 4), dtype=np.float32).reshape(1, hq, 2, 2)
        k = (np.asarray(gv.pattern(hkv * 6)) * 0.7).astype(np.float32).reshape(1, hkv, 3, 2)
        v = (np.asarray(gv.pattern(hkv * 9)) * -0.5).astype(np.float32).reshape(1, hkv, 3, 3)
        rep = hq // hkv
        a = orc.sdpa_forward(q, k, v, 1 / np.sqrt(2), True)
        b = orc.sdpa_forward(q, np.repeat(k, rep, axis=1), np.repeat(v, rep, axis=1), 1 / np.sqrt(2), True)
        np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("mode", [0, 1])
def test_kv_attention_matches_sdpa(mode):
    c = gv.kv_attention_vs_sdpa_case()
    pool = orc.Pool(1, c["kv_heads"], c["head_dim"], c["max_tokens"], c["block_size"], orc.F32)
    seq = pool.make_sequence()
    seq.set_advance(c["advance"])
    out = orc.kv_attention(pool, 0, [seq], 1, c["q"], c["k"], c["v"], c["scale"], mode=mode, threads=2)
    expected = orc.sdpa_forward(c["q"], np.repeat(c["k"], 2, axis=1), np.repeat(c["v"], 2, axis=1), c["scale"], True)
    np.testing.assert_allclose(out, expected, rtol=0, atol=c["tol"])
    np.testing.assert_array_equal(seq.blocks, [0])


def test_kv_attention_modes_are_bit_identical():
    rng = np.random.default_rng(3)
    pool_a = orc.Pool(1, 2, 8, 64, 4, orc.F16)
    pool_b = orc.Pool(1, 2, 8, 64, 4, orc.F16)
    sa, sb = pool_a.make_sequence(), pool_b.make_sequence()
    for step, t in enumerate([5, 1, 1, 3]):
        q = rng.normal(size=(1, 4, t, 8)).astype(np.float32)
        k = rng.normal(size=(1, 2, t, 8)).astype(np.float32)
        v = rng.normal(size=(1, 2, t, 8)).astype(np.float32)
        for s in (sa, sb):
            s.set_advance(t)
        a = orc.kv_attention(pool_a, 0, [sa], 1, q, k, v, 0.35, mode=0)
        b = orc.kv_attention(pool_b, 0, [sb], 1, q, k, v, 0.35, mode=1, threads=3)
        np.testing.assert_array_equal(a, b)
        for s in (sa, sb):
            s.set_cursor(s.cursor + t)


def test_windowed_and_full_attention_known_answers():
    c = gv.WINDOWED_CASE
    pool = orc.Pool(2, c["kv_heads"], c["head_dim"], c["max_tokens"], c["block_size"], orc.F32)
    seq = pool.make_sequence()

    def run(v_values, tokens, expect_error=None):
        t = len(tokens)
        # inputs are [1,H,4,1] exemplar-shaped in the reference; only `advance` rows are live
        q = np.zeros((1, c["q_heads"], 4, 1), dtype=np.float32)
        k = np.zeros((1, c["kv_heads"], 4, 1), dtype=np.float32)
        v = np.asarray(v_values, dtype=np.float32).reshape(1, c["kv_heads"], 4, 1)
        seq.set_advance(t)
        ev = np.full(1, U64_MAX, dtype=np.uint64)
        # the program mixes a windowed and a full layer, so the schema-wide eviction window is None
        local = orc.kv_attention(pool, 0, [seq], 1, q, k, v, 1.0, op_window=c["local_window"], eviction_starts=ev)
        full = orc.kv_attention(pool, 1, [seq], 1, q, k, v, 1.0, eviction_starts=ev)
        seq.note_tokens(tokens)
        seq.set_cursor(seq.cursor + t)
        return local, full

    run(c["first_v"], c["first_tokens"])
    local, full = run(c["second_v"], c["second_tokens"])
    np.testing.assert_allclose(local.reshape(-1)[[0, 4, 8, 12]], c["local_expected"], rtol=1e-6)
    np.testing.assert_allclose(full.reshape(-1)[[0, 4, 8, 12]], c["full_expected"], rtol=1e-6)
    run([0] * 8, c["third_tokens"])
    with pytest.raises(orc.OracleError, match=c["overflow_message"]):
        run([0] * 8, c["overflow_tokens"])


def test_online_rescaling_large_scores():
    # packages/core/test/Attention.test.ts:315-336 — scores span about -124..254
    n = 2 * 40 * 16
    q = (np.asarray(gv.pattern(n)) * 8).astype(np.float32).reshape(1, 2, 40, 16)
    v = (np.asarray(gv.pattern(n)) * -0.5 + 0.2).astype(np.float32).reshape(1, 2, 40, 16)
    out = orc.sdpa_forward(q, q, v, 0.25, True)
    assert np.isfinite(out).all()
    pool = orc.Pool(1, 2, 16, 48, 16, orc.F32)
    seq = pool.make_sequence()
    seq.set_advance(40)
    paged = orc.kv_attention(pool, 0, [seq], 1, q, q, v, 0.25, mode=1)
    np.testing.assert_allclose(paged, out, rtol=1e-4, atol=1e-4)


# ---------------------------------------------------------------- slab tiers
def test_slab_write_read_f16():
    c = gv.SLAB_F16_CASE
    pool = orc.Pool(1, 1, c["width"], c["rows"], 1, orc.F16)
    pool.write_rows(0, 0, c["write_rows"], c["values"])
    np.testing.assert_array_equal(pool.read_rows(0, 0, c["read_rows"]).reshape(-1), c["expected"])


def test_slab_scatter_gather_roundtrip():
    # crates/runtime-cpu/src/napi/mod.rs:4955-4961
    pool = orc.Pool(1, 1, 6, 8, 1, orc.F32)
    src = np.arange(12, dtype=np.float32)
    pool.write_rows(0, 0, [4, 5], src)
    np.testing.assert_array_equal(pool.read_rows(0, 0, [4, 5]).reshape(-1), src)


def test_int8_roundtrip():
    c = gv.INT8_ROUNDTRIP_CASE
    q, s = orc.quantize_int8(c["x"], c["rows"], c["heads"], c["d"])
    back = orc.dequantize_int8(q, s, c["rows"], c["heads"], c["d"])
    assert np.abs(back - np.asarray(c["x"], dtype=np.float32)).max() < c["tol"]


def test_bf16_and_f16_conversions_round_to_nearest_even():
    L = orc.lib()
    assert L.orc_f32_to_bf16.restype is not None
    L.orc_f32_to_bf16.argtypes = [orc.C.c_float]
    L.orc_f32_to_f16.argtypes = [orc.C.c_float]
    L.orc_f32_to_bf16.restype = orc.C.c_uint16
    L.orc_f32_to_f16.restype = orc.C.c_uint16
    # 1 + 2^-8 is exactly halfway between two bf16 values -> ties to even (1.0)
    assert L.orc_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    assert L.orc_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82
    rng = np.random.default_rng(4)
    xs = rng.normal(size=200).astype(np.float32)
    for x in xs:
        assert L.orc_f32_to_f16(float(x)) == int(np.float16(x).view(np.uint16))


def test_state_bytes_formula():
    c = gv.STATE_BYTES_CASE
    assert orc.state_bytes(c["layers"], c["max_tokens"], c["kv_heads"], c["head_dim"], orc.U8) == c["dtype_u8_bytes"]
    assert orc.state_bytes(1, 8, 2, 4, orc.F32) == 512
    assert orc.state_bytes(1, 8, 2, 4, orc.F16) == 256


# ---------------------------------------------------------------- allocator / prefix cache
def _block_store_pool(blocks):
    return orc.Pool(0, 0, 0, blocks * 2, 2, orc.F32)


def test_prefix_cache_take_and_reclaim():
    # crates/runtime-cpu/src/napi/mod.rs:5404-5420
    pool = _block_store_pool(2)
    a = pool.alloc_block()
    b = pool.alloc_block()
    assert (a, b) == (0, 1)
    assert pool.alloc_block() is None
    pool.set_hash(a, 42)
    pool.unref_block(a)
    assert pool.cached_blocks == 1
    assert pool.take_block(42) == a
    assert pool.cached_blocks == 0
    pool.unref_block(a)
    assert pool.alloc_block() == a
    pool.unref_block(a)
    pool.unref_block(b)
    assert pool.free_blocks == 2


def test_note_tokens_hashes_completed_blocks():
    # napi/mod.rs:5422-5448
    pool = _block_store_pool(2)
    seq = pool.make_sequence()
    seq.push_block(pool.alloc_block())
    seq.push_block(pool.alloc_block())
    seq.note_tokens([7, 8, 9])
    first = orc.chain_hash(orc.HASH_SEED, [7, 8])
    second = orc.chain_hash(first, [9, 5])
    assert pool.block_hash(int(seq.blocks[0])) == first
    seq.set_cursor(3)
    seq.note_tokens([5])
    assert pool.block_hash(int(seq.blocks[1])) == second


def test_chain_hash_is_fnv1a_over_le_bytes():
    h = orc.HASH_SEED
    for byte in (7).to_bytes(4, "little") + (0x01020304).to_bytes(4, "little"):
        h = ((h ^ byte) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    assert orc.chain_hash(orc.HASH_SEED, [7, 0x01020304]) == h


def test_prefill_match_reuses_whole_blocks_but_never_the_last_token():
    # napi/mod.rs:3874-3946 (non-recurrent branch): at most (len-1)/block_size blocks are reused
    pool = orc.Pool(1, 1, 1, 8, 2, orc.F32)
    tokens = [10, 11, 12, 13, 14]
    h1 = orc.chain_hash(orc.HASH_SEED, [10, 11])
    h2 = orc.chain_hash(h1, [12, 13])
    for h in (h1, h2):
        b = pool.alloc_block()
        pool.set_hash(b, h)
        pool.unref_block(b)
    seq = pool.make_sequence()
    assert seq.prefill_match(tokens) == 4
    assert seq.last_hash == h2 and len(seq.blocks) == 2
    with pytest.raises(orc.OracleError, match="already holds tokens"):
        seq.prefill_match(tokens)
    other = pool.make_sequence()
    assert other.prefill_match([10, 11, 12, 13]) == 2  # 4 tokens: only (4-1)//2 = 1 block may match
    third = pool.make_sequence()
    assert third.prefill_match([1, 2, 3]) == 0


def test_pool_geometry_rules():
    with pytest.raises(orc.OracleError, match="positive multiple of block size"):
        orc.Pool(1, 1, 1, 10, 4)
    with pytest.raises(orc.OracleError, match="must be positive"):
        orc.Pool(1, 0, 4, 8, 4)
    with pytest.raises(orc.OracleError, match="must be zero when layers is zero"):
        orc.Pool(0, 1, 4, 8, 4)


def test_pool_exhaustion_and_capacity_messages():
    pool = orc.Pool(1, 1, 2, 8, 4, orc.F32)
    a, b = pool.make_sequence(), pool.make_sequence()
    zeros = lambda t: (np.zeros((1, 1, t, 2), np.float32),) * 3
    a.set_advance(4)
    orc.kv_attention(pool, 0, [a], 1, *zeros(4), 1.0)
    a.set_cursor(4)
    b.set_advance(4)
    orc.kv_attention(pool, 0, [b], 1, *zeros(4), 1.0)
    b.set_cursor(4)
    a.set_advance(1)
    with pytest.raises(orc.OracleError, match="pool exhausted"):
        orc.kv_attention(pool, 0, [a], 1, *zeros(1), 1.0)
    b.release()
    assert pool.free_blocks == 1
    a.set_cursor(8)
    a.set_advance(1)
    with pytest.raises(orc.OracleError, match="exceeds pool capacity"):
        orc.kv_attention(pool, 0, [a], 1, *zeros(1), 1.0)


# ---------------------------------------------------------------- sampling / last token row
@pytest.mark.parametrize("logits,expected", gv.GREEDY_CASES)
def test_greedy_prefers_lower_token_on_ties(logits, expected):
    assert orc.argmax(logits) == expected
    assert orc.sample_logits(logits, temperature=0.0, top_k=4, seed=7) == expected


def test_sampler_semantics():
    # crates/runtime/src/sampling.rs:239-302
    assert orc.sample_logits([1.0, 4.0, 3.0], top_k=1, seed=7, counter=3) == 1
    assert orc.sample_logits([2.0, 1.0, 0.0], top_p=0.8, seed=1, counter=0) < 2
    assert orc.sample_logits([0.0] * 4, seed=7, counter=3) == orc.sample_logits([0.0] * 4, seed=7, counter=3)
    assert orc.sample_logits([0.0, 1.0, 2.0], seed=7, counter=3) == orc.sample_logits([0.0, 1.0, 2.0], top_k=3, seed=7, counter=3)
    with pytest.raises(orc.OracleError, match="topK"):
        orc.sample_logits([1.0, 4.0, 2.0, 0.0], top_k=5)
    with pytest.raises(orc.OracleError, match="temperature"):
        orc.sample_logits([1.0], temperature=-1)
    with pytest.raises(orc.OracleError, match="topP"):
        orc.sample_logits([1.0], top_p=0.0)
    with pytest.raises(orc.OracleError, match="not finite"):
        orc.argmax([0.0, float("nan")])
    u = orc.random_unit(7, 3)
    assert 0.0 <= u < 1.0


def test_last_token_row():
    c = gv.LAST_TOKEN_ROW_CASE
    np.testing.assert_array_equal(orc.last_token_row(c["source"], c["advance"]), c["expected"])
    for bad in c["bad_advances"]:
        with pytest.raises(orc.OracleError) as e:
            orc.last_token_row(c["source"], bad)
        assert str(e.value) == c["message"].format(bad)
