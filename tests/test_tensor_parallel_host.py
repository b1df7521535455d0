"""Tensor-parallel host logic on CPU: the shard arithmetic against the oracle, and a world_size-2 gloo run of one
projection block (shard, partial linear, residual on rank 0 only, all-reduce) against the unsharded oracle."""
import os
import socket

import numpy as np
import pytest

import oracle as orc
from effect_torch_b200 import tensor_parallel as tp
from tests import helpers
from tests.golden import reference_vectors as gv


def test_local_geometry_and_divisibility_errors():
    cfg = helpers.TINY_Q
    local = tp.local_config(cfg, 2)
    assert (local["q_heads"], local["kv_heads"], local["ffn"], local["d_model"], local["vocab"]) == (2, 1, 384, 256, 2048)
    with pytest.raises(ValueError, match="kv_heads"):
        tp.local_config(cfg, 4)
    with pytest.raises(ValueError, match="multiple of 64"):
        tp.local_config(dict(cfg, ffn=704, kv_heads=2), 2)  # 352 columns per rank


@pytest.mark.parametrize("codec", [gv.Q4_0, gv.Q8_0])
def test_row_and_column_shards_recombine_to_the_full_linear(codec):
    rng = np.random.default_rng(5)
    n, k, world = 96, 256, 2
    w = rng.normal(0, 0.05, size=(n, k)).astype(np.float32)
    packed = orc.quantize(codec, w)
    x = rng.normal(size=(3, k)).astype(np.float32)
    full = orc.qlinear(codec, x, packed, n, k)
    # column-parallel projection: ranks hold row ranges, outputs concatenate
    parts = [orc.qlinear(codec, x, tp.shard_rows(packed, r, world), n // world, k) for r in range(world)]
    np.testing.assert_array_equal(np.concatenate(parts, axis=1), full)
    # row-parallel projection: ranks hold block ranges of every row and the matching slice of x, outputs add
    kk = k // world
    partial = [orc.qlinear(codec, np.ascontiguousarray(x[:, r * kk:(r + 1) * kk]), tp.shard_columns(packed, codec, r, world), n, kk)
               for r in range(world)]
    assert helpers.rel_err(partial[0] + partial[1], full) <= 1e-6
    # the shard's bytes are the blocks of that column range, bit for bit
    np.testing.assert_array_equal(orc.dequantize(codec, tp.shard_columns(packed, codec, 1, world), n, kk),
                                  orc.dequantize(codec, packed, n, k)[:, kk:])


@pytest.mark.parametrize("codec", [gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_k_quant_shards_cut_whole_256_value_blocks(codec):
    rng = np.random.default_rng(8)
    n, k, world = 64, 1024, 2
    packed = helpers.random_k_quant(codec, n, k, rng)
    full = orc.dequantize(codec, packed, n, k)
    kk = k // world
    for r in range(world):
        np.testing.assert_array_equal(orc.dequantize(codec, tp.shard_columns(packed, codec, r, world), n, kk), full[:, r * kk:(r + 1) * kk])
        np.testing.assert_array_equal(orc.dequantize(codec, tp.shard_rows(packed, r, world), n // world, k), full[r * n // world:(r + 1) * n // world])
    with pytest.raises(ValueError, match="not divisible"):
        tp.shard_columns(helpers.random_k_quant(codec, 4, 768, rng), codec, 0, 2)  # three blocks per row


def test_shard_weights_keeps_every_projections_own_codec():
    cfg = helpers.TINY_Q
    codecs = dict(wq=gv.Q4_K, wk=gv.Q4_K, wv=gv.Q6_K, wo=gv.Q4_K, gate=gv.Q4_K, up=gv.Q4_K, down=gv.Q6_K, head=gv.Q6_K)
    cfg = dict(cfg, ffn=1024, q_heads=8)  # a rank's share of the columns of down and wo must be whole 256-value blocks
    weights = helpers.make_mixed_weights(cfg, codecs, seed=3)
    shards = [tp.shard_weights(weights, cfg, r, 2, shard_head=True) for r in range(2)]
    for name in tp.ROW_SPLIT + tp.COLUMN_SPLIT:
        packed, n, k, codec = weights["layers"][1][name]
        axis = 0 if name in tp.ROW_SPLIT else 1
        got = np.concatenate([s["layers"][1][name][0] for s in shards], axis=axis)
        np.testing.assert_array_equal(got, packed)
        assert shards[1]["layers"][1][name][1:] == ((n // 2, k, codec) if axis == 0 else (n, k // 2, codec))
    assert shards[0]["head"][1:] == (cfg["vocab"] // 2, cfg["d_model"], gv.Q6_K)


def test_shard_weights_covers_every_projection():
    cfg = helpers.TINY_Q
    weights = helpers.make_weights(cfg, seed=2, codec=gv.Q4_0)
    shards = [tp.shard_weights(weights, cfg, r, 2) for r in range(2)]
    for name in tp.ROW_SPLIT:
        packed, n, k = weights["layers"][0][name]
        got = np.concatenate([s["layers"][0][name][0] for s in shards], axis=0)
        np.testing.assert_array_equal(got, packed)
        assert shards[0]["layers"][0][name][1:] == (n // 2, k)
    for name in tp.COLUMN_SPLIT:
        packed, n, k = weights["layers"][0][name]
        got = np.concatenate([s["layers"][0][name][0] for s in shards], axis=1)
        np.testing.assert_array_equal(got, packed)
        assert shards[1]["layers"][0][name][1:] == (n, k // 2)
    assert shards[0]["head"] is weights["head"] and shards[1]["tok_embd"] is weights["tok_embd"]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, results):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 0's 128-byte id reaches every rank through the host transport (what the CUDA path does with the NCCL id)
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            ident = torch.arange(128, dtype=torch.uint8)
        dist.broadcast(ident, src=0)
        assert ident.tolist() == list(range(128))
        cfg = helpers.TINY_Q
        codec = gv.Q4_0
        weights = helpers.make_weights(cfg, seed=7, codec=codec)  # same seed on every rank: replicated host state
        local = tp.shard_weights(weights, cfg, rank, world)
        rng = np.random.default_rng(11)
        hidden = rng.normal(size=(4, cfg["d_model"])).astype(np.float32)
        att = rng.normal(size=(4, cfg["q_heads"] * cfg["head_dim"])).astype(np.float32)
        packed, n, k = weights["layers"][0]["wo"]
        expected = hidden + orc.qlinear(codec, att, packed, n, k)
        lp, ln, lk = local["layers"][0]["wo"]
        partial = orc.qlinear(codec, np.ascontiguousarray(att[:, rank * lk:(rank + 1) * lk]), lp, ln, lk)
        mine = torch.from_numpy((hidden + partial) if rank == 0 else partial)  # the residual enters once
        dist.all_reduce(mine)
        results[rank] = helpers.rel_err(mine.numpy(), expected)
        # gate/up are row shards: the ranks' activations concatenate to the full SwiGLU input of down
        g, gn, gk = local["layers"][0]["gate"]
        u, _, _ = local["layers"][0]["up"]
        x = rng.normal(size=(4, cfg["d_model"])).astype(np.float32)
        act_local = orc.silu_mul(orc.qlinear(codec, x, g, gn, gk), orc.qlinear(codec, x, u, gn, gk))
        dp, dn, dk = local["layers"][0]["down"]
        down_partial = torch.from_numpy(orc.qlinear(codec, act_local, dp, dn, dk))
        dist.all_reduce(down_partial)
        fg, fgn, fgk = weights["layers"][0]["gate"]
        fu, _, _ = weights["layers"][0]["up"]
        fd, fdn, fdk = weights["layers"][0]["down"]
        full = orc.qlinear(codec, orc.silu_mul(orc.qlinear(codec, x, fg, fgn, fgk), orc.qlinear(codec, x, fu, fgn, fgk)), fd, fdn, fdk)
        results[world + rank] = helpers.rel_err(down_partial.numpy(), full)
        # step-status exchange: rank 1 reports a failed step (as if its bounded peer wait had run out); rank 0's own call
        # succeeded, yet both ranks must see the step as failed and roll back, and a clean step is clean on both
        results[("agree", rank)] = (tp.all_ranks_ok(rank != 1), tp.all_ranks_ok(True))
        tp.barrier_before_teardown()
    finally:
        dist.destroy_process_group()


def test_two_rank_projection_block_over_gloo_matches_the_unsharded_oracle():
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    numeric = {k: v for k, v in results.items() if isinstance(k, int)}
    assert sorted(numeric.keys()) == [0, 1, 2, 3]
    assert all(err <= 1e-6 for err in numeric.values()), dict(results)
    assert results[("agree", 0)] == (False, True) and results[("agree", 1)] == (False, True)


def test_a_sharded_head_cuts_the_vocabulary_by_rows_and_the_picks_recombine_to_the_full_argmax():
    """Vocabulary-parallel head on the host side: local geometry, the head shard, and the rule the ranks' (best logit, token)
    picks are merged by (largest logit, lowest token on ties) against the full-row argmax of the oracle."""
    cfg = helpers.TINY_Q
    world = 4
    locals_ = [tp.local_config(dict(cfg, kv_heads=4, q_heads=8), world, shard_head=True, rank=r) for r in range(world)]
    assert [c["vocab"] for c in locals_] == [512] * 4 and all(c["vocab_global"] == 2048 for c in locals_)
    assert [c["head_first_row"] for c in locals_] == [0, 512, 1024, 1536]
    assert "vocab_global" not in tp.local_config(cfg, 2)  # replicated head: nothing changes
    with pytest.raises(ValueError, match="vocab"):
        tp.local_config(dict(cfg, vocab=2049), 2, shard_head=True)
    weights = helpers.make_weights(cfg, seed=1, codec=gv.Q4_0)
    shards = [tp.shard_weights(weights, cfg, r, 2, shard_head=True) for r in range(2)]
    packed, n, k = weights["head"]
    for r, shard in enumerate(shards):
        got, rows, cols = shard["head"]
        assert (rows, cols) == (n // 2, k)
        np.testing.assert_array_equal(got, packed[r * n // 2:(r + 1) * n // 2])
    assert tp.shard_weights(weights, cfg, 0, 2)["head"][0] is packed
    # merging picks: ties across ranks go to the lower token
    rng = np.random.default_rng(3)
    logits = rng.normal(size=(5, 2048)).astype(np.float32)
    logits[1, 1700] = logits[1, 40] = logits[1].max() + 1  # the same maximum on rank 0 and rank 3
    per = 2048 // world
    picks = [[(float(row[r * per:(r + 1) * per].max()), r * per + int(row[r * per:(r + 1) * per].argmax())) for r in range(world)] for row in logits]
    merged = [min(p, key=lambda vt: (-vt[0], vt[1]))[1] for p in picks]
    assert merged == [orc.argmax(row) for row in logits] and merged[1] == 40
