"""GPU parity for the paged KV path: page allocation and tables, slab tiers, reference-order attention and
the tensor-core flash-decoding kernel, against the reference's golden vectors and the CPU oracle."""
import numpy as np
import pytest

import effect_torch_b200 as et
import oracle as orc
from tests import helpers
from tests.golden import reference_vectors as gv
from tests.gpu_util import dev, empty, host, runtime

pytestmark = pytest.mark.gpu
REL_TOL = 2e-3  # north-star tolerance on attention outputs for the f16 path


def gpu_attention(pool, layer, seqs, batch, active, advance, q, k, v, scale, op_window=None, pool_window=None):
    out = empty(q.shape)
    runtime().kv_attention_into(pool, layer, seqs, batch, active, advance, dev(q), dev(k), dev(v), q.shape[1], q.shape[2], scale,
                                op_window, pool_window, out)
    return host(out)


def test_kv_attention_matches_dense_causal_attention():
    c = gv.kv_attention_vs_sdpa_case()
    pool = et.NativeKvPool(runtime(), 1, c["kv_heads"], c["head_dim"], c["max_tokens"], c["block_size"], et.KV_F32)
    seq = pool.makeSequence()
    out = gpu_attention(pool, 0, [seq], 1, 1, c["advance"], c["q"], c["k"], c["v"], c["scale"])
    expected = orc.sdpa_forward(c["q"], np.repeat(c["k"], 2, axis=1), np.repeat(c["v"], 2, axis=1), c["scale"], True)
    np.testing.assert_allclose(out, expected, rtol=0, atol=c["tol"])
    blocks, head = seq.blocks
    np.testing.assert_array_equal(blocks, [0])
    assert head == 0 and seq.cursor == 0  # the cursor moves only at commit


def test_windowed_and_full_attention_known_answers():
    c = gv.WINDOWED_CASE
    rt = runtime()
    pool = et.NativeKvPool(rt, 2, c["kv_heads"], c["head_dim"], c["max_tokens"], c["block_size"], et.KV_F32)
    seq = pool.makeSequence()

    def run(v_values, tokens):
        t = len(tokens)
        q = np.zeros((1, c["q_heads"], 4, 1), dtype=np.float32)
        k = np.zeros((1, c["kv_heads"], 4, 1), dtype=np.float32)
        v = np.asarray(v_values, dtype=np.float32).reshape(1, c["kv_heads"], 4, 1)
        local = gpu_attention(pool, 0, [seq], 1, 1, t, q, k, v, 1.0, op_window=c["local_window"])
        full = gpu_attention(pool, 1, [seq], 1, 1, t, q, k, v, 1.0)
        seq.commit(tokens)
        return local, full

    run(c["first_v"], c["first_tokens"])
    local, full = run(c["second_v"], c["second_tokens"])
    np.testing.assert_allclose(local.reshape(-1)[[0, 4, 8, 12]], c["local_expected"], rtol=1e-6)
    np.testing.assert_allclose(full.reshape(-1)[[0, 4, 8, 12]], c["full_expected"], rtol=1e-6)
    run([0] * 8, c["third_tokens"])
    frontier = seq.frontier
    with pytest.raises(et.BackendError, match=c["overflow_message"]) as e:
        run([0] * 8, c["overflow_tokens"])
    assert e.value.reason == "execution-failed"
    seq.rollback(frontier)
    assert seq.cursor == 8


def test_pool_exhaustion_and_capacity_messages_and_rollback():
    rt = runtime()
    pool = et.NativeKvPool(rt, 1, 1, 2, 8, 4, et.KV_F32)
    a, b = pool.makeSequence(), pool.makeSequence()
    z = lambda t: np.zeros((1, 1, t, 2), np.float32)
    gpu_attention(pool, 0, [a], 1, 1, 4, z(4), z(4), z(4), 1.0)
    a.commit([1, 2, 3, 4])
    gpu_attention(pool, 0, [b], 1, 1, 4, z(4), z(4), z(4), 1.0)
    b.commit([5, 6, 7, 8])
    assert pool.freeBlocks == 0
    frontier = a.frontier
    with pytest.raises(et.BackendError, match="pool exhausted"):
        gpu_attention(pool, 0, [a], 1, 1, 1, z(1), z(1), z(1), 1.0)
    a.rollback(frontier)
    assert a.cursor == 4 and a.frontier == 1
    b.release()
    b.release()  # idempotent
    assert pool.freeBlocks == 1 and pool.cachedBlocks == 1  # b's full block was hashed at commit
    with pytest.raises(et.BackendError, match="is released"):
        gpu_attention(pool, 0, [b], 1, 1, 1, z(1), z(1), z(1), 1.0)


def test_pool_geometry_rules():
    rt = runtime()
    with pytest.raises(et.BackendError, match="positive multiple of block size") as e:
        et.NativeKvPool(rt, 1, 1, 1, 10, 4)
    assert e.value.reason == "invalid-argument"
    with pytest.raises(et.BackendError, match="must be positive"):
        et.NativeKvPool(rt, 1, 0, 4, 8, 4)
    with pytest.raises(et.BackendError, match="must be zero when layers is zero"):
        et.NativeKvPool(rt, 0, 1, 4, 8, 4)


@pytest.mark.parametrize("tier,otier", [(et.KV_F32, orc.F32), (et.KV_F16, orc.F16), (et.KV_BF16, orc.BF16), (et.KV_U8, orc.U8)])
def test_tiers_page_tables_and_attention_match_the_oracle(tier, otier):
    """Two sequences, ragged chunks crossing page boundaries, 3 active of 4 lanes: slab contents, page tables and
    outputs must equal the oracle's (values bit-exact; outputs to f64-exp rounding)."""
    rng = np.random.default_rng(8 + tier)
    Hq, Hkv, D, bs = 4, 2, 16, 4
    rt = runtime()
    gp = et.NativeKvPool(rt, 1, Hkv, D, 64, bs, tier)
    op = orc.Pool(1, Hkv, D, 64, bs, otier)
    gseqs = [gp.makeSequence() for _ in range(3)]
    oseqs = [op.make_sequence() for _ in range(3)]
    for t in (5, 1, 3, 1, 4):
        q = rng.normal(size=(4, Hq, t, D)).astype(np.float32)
        k = rng.normal(size=(4, Hkv, t, D)).astype(np.float32)
        v = rng.normal(size=(4, Hkv, t, D)).astype(np.float32)
        for s in oseqs:
            s.set_advance(t)
        expected = orc.kv_attention(op, 0, oseqs + [op.make_sequence()], 3, q, k, v, 0.25, mode=1, threads=2)
        got = gpu_attention(gp, 0, gseqs, 4, 3, t, q, k, v, 0.25)
        np.testing.assert_allclose(got, expected, rtol=1e-6, atol=1e-6)
        assert not got[3].any()  # padded lane stays zero
        toks = rng.integers(0, 100, size=(3, t)).astype(np.uint32)
        for i in range(3):
            gseqs[i].commit(toks[i])
            oseqs[i].note_tokens(toks[i])
            oseqs[i].set_cursor(oseqs[i].cursor + t)
    for gs, os_ in zip(gseqs, oseqs):
        blocks, head = gs.blocks
        np.testing.assert_array_equal(blocks, os_.blocks)
        assert gs.cursor == os_.cursor == 14
        rows = [int(b) * bs + o for b in blocks for o in range(bs)][:14]
        for which in (0, 1):
            np.testing.assert_array_equal(gp.read_rows(0, which, rows).view(np.uint32),
                                          op.read_rows(0, which, rows, dequant=True).view(np.uint32))
    assert gp.freeBlocks == op.free_blocks and gp.cachedBlocks == op.cached_blocks


def test_prefix_cache_and_prefill_match():
    rt = runtime()
    gp = et.NativeKvPool(rt, 1, 1, 2, 16, 2, et.KV_F32)
    op = orc.Pool(1, 1, 2, 16, 2, orc.F32)
    tokens = [10, 11, 12, 13, 14]
    z = lambda t: np.zeros((1, 1, t, 2), np.float32)
    g1, o1 = gp.makeSequence(), op.make_sequence()
    gpu_attention(gp, 0, [g1], 1, 1, 5, z(5), z(5), z(5), 1.0)
    g1.commit(tokens)
    o1.set_advance(5)
    orc.kv_attention(op, 0, [o1], 1, z(5), z(5), z(5), 1.0)
    o1.note_tokens(tokens)
    o1.set_cursor(5)
    g1.release()
    o1.release()
    assert (gp.freeBlocks, gp.cachedBlocks) == (op.free_blocks, op.cached_blocks) == (8, 2)
    g2, o2 = gp.makeSequence(), op.make_sequence()
    assert g2.prefillMatch(tokens) == o2.prefill_match(tokens) == 4
    np.testing.assert_array_equal(g2.blocks[0], o2.blocks)
    with pytest.raises(et.BackendError, match="already holds tokens"):
        g2.prefillMatch(tokens)
    g3 = gp.makeSequence()
    assert g3.prefillMatch([1, 2, 3]) == 0


@pytest.mark.parametrize("tier,otier,tol", [(et.KV_F16, orc.F16, REL_TOL), (et.KV_BF16, orc.BF16, 2e-2), (et.KV_U8, orc.U8, REL_TOL)])
@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (8, 1, 128), (4, 2, 64)])
def test_tensor_core_decode_attention_matches_the_oracle(tier, otier, tol, Hq, Hkv, D):
    """Flash-decoding kernel vs the f64 oracle on ragged contexts (one lane crosses several splits, one is a single
    token, one is padded), with shuffled page tables."""
    rng = np.random.default_rng(Hq * D + tier)
    B, active, bs, max_tokens = 5, 4, 16, 16 * 200
    rt = runtime()
    gp = et.NativeKvPool(rt, 1, Hkv, D, max_tokens, bs, tier)
    op = orc.Pool(1, Hkv, D, max_tokens, bs, otier)
    gseqs = [gp.makeSequence() for _ in range(active)]
    oseqs = [op.make_sequence() for _ in range(active)]
    contexts = [1, 37, 700, 1500]
    # interleave the lanes' page allocations so tables are not contiguous
    filled = [0] * active
    while any(f < c - 1 for f, c in zip(filled, contexts)):
        for i in range(active):
            t = min(48, contexts[i] - 1 - filled[i])
            if t <= 0:
                continue
            k = rng.normal(size=(1, Hkv, t, D)).astype(np.float32)
            v = rng.normal(size=(1, Hkv, t, D)).astype(np.float32)
            rt.kv_append_into(gp, 0, [gseqs[i]], 1, 1, t, dev(k), dev(v), t)
            toks = rng.integers(0, 1000, size=t).astype(np.uint32)
            gseqs[i].commit(toks)
            oseqs[i].set_advance(t)
            orc.kv_attention(op, 0, [oseqs[i]], 1, np.zeros((1, Hq, t, D), np.float32), k, v, 1.0, mode=1)
            oseqs[i].note_tokens(toks)
            oseqs[i].set_cursor(oseqs[i].cursor + t)
            filled[i] += t
    q = rng.normal(size=(B, Hq, 1, D)).astype(np.float32)
    k = rng.normal(size=(B, Hkv, 1, D)).astype(np.float32)
    v = rng.normal(size=(B, Hkv, 1, D)).astype(np.float32)
    scale = 1 / np.sqrt(D)
    for s in oseqs:
        s.set_advance(1)
    expected = orc.kv_attention(op, 0, oseqs + [op.make_sequence()], active, q, k, v, scale, mode=1, threads=8)
    out = empty((B, Hq, D))
    rt.kv_attention_decode_into(gp, 0, gseqs, B, active, dev(q.reshape(B, Hq, D)), dev(k.reshape(B, Hkv, D)), dev(v.reshape(B, Hkv, D)),
                                Hq, scale, out=out)
    got = host(out).reshape(B, Hq, 1, D)
    assert not got[4].any()
    for i in range(active):
        assert helpers.rel_err(got[i], expected[i]) <= tol, f"lane {i} (context {contexts[i]})"
    for gs, os_ in zip(gseqs, oseqs):
        np.testing.assert_array_equal(gs.blocks[0], os_.blocks)


def test_tensor_core_decode_attention_with_a_window():
    rng = np.random.default_rng(21)
    Hq, Hkv, D, bs = 8, 2, 128, 16
    rt = runtime()
    gp = et.NativeKvPool(rt, 1, Hkv, D, 1024, bs, et.KV_F16)
    op = orc.Pool(1, Hkv, D, 1024, bs, orc.F16)
    gs, os_ = gp.makeSequence(), op.make_sequence()
    t = 300
    k = rng.normal(size=(1, Hkv, t, D)).astype(np.float32)
    v = rng.normal(size=(1, Hkv, t, D)).astype(np.float32)
    rt.kv_append_into(gp, 0, [gs], 1, 1, t, dev(k), dev(v), t)
    gs.commit(np.arange(t))
    os_.set_advance(t)
    orc.kv_attention(op, 0, [os_], 1, np.zeros((1, Hq, t, D), np.float32), k, v, 1.0, mode=1)
    os_.set_cursor(t)
    q = rng.normal(size=(1, Hq, 1, D)).astype(np.float32)
    k1 = rng.normal(size=(1, Hkv, 1, D)).astype(np.float32)
    v1 = rng.normal(size=(1, Hkv, 1, D)).astype(np.float32)
    os_.set_advance(1)
    expected = orc.kv_attention(op, 0, [os_], 1, q, k1, v1, 0.1, op_window=100, mode=1)
    out = empty((1, Hq, D))
    rt.kv_attention_decode_into(gp, 0, [gs], 1, 1, dev(q.reshape(1, Hq, D)), dev(k1.reshape(1, Hkv, D)), dev(v1.reshape(1, Hkv, D)),
                                Hq, 0.1, op_window=100, out=out)
    assert helpers.rel_err(host(out).reshape(1, Hq, 1, D), expected) <= REL_TOL
