"""Shared builders for the parity tests: synthetic Llama-shaped weights fed identically to the CPU
oracle and to the CUDA library."""
from __future__ import annotations

import numpy as np

import oracle as orc

TINY = dict(layers=4, d_model=256, q_heads=4, kv_heads=2, head_dim=64, ffn=688, vocab=4096, rms_eps=1e-5, rope_theta=10000.0)
# a quantizable sibling of the tiny config (every projection width is a multiple of 64)
TINY_Q = dict(layers=3, d_model=256, q_heads=4, kv_heads=2, head_dim=64, ffn=768, vocab=2048, rms_eps=1e-5, rope_theta=10000.0)


def make_weights(cfg, seed=0, codec=0):
    """f32 weights ~N(0, 0.02) drawn in a fixed order (token embedding; per layer attn_norm (ones), wq, wk, wv,
    wo, ffn_norm (ones), gate, up, down; out_norm (ones); head), all in the reference's [N, K] row layout.
    With a block codec, projections and head are quantized by the oracle quantizer; embeddings and norms stay f32."""
    rng = np.random.default_rng(seed)
    d, qw, kvw, ffn, V = cfg["d_model"], cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"], cfg["ffn"], cfg["vocab"]
    normal = lambda *shape: rng.normal(0.0, 0.02, size=shape).astype(np.float32)
    w = {"tok_embd": normal(V, d), "layers": []}
    for _ in range(cfg["layers"]):
        w["layers"].append(dict(attn_norm=np.ones(d, np.float32), wq=normal(qw, d), wk=normal(kvw, d), wv=normal(kvw, d),
                                wo=normal(d, qw), ffn_norm=np.ones(d, np.float32), gate=normal(ffn, d), up=normal(ffn, d),
                                down=normal(d, ffn)))
    w["out_norm"] = np.ones(d, np.float32)
    w["head"] = normal(V, d)
    if codec:
        for layer in w["layers"]:
            for name in ("wq", "wk", "wv", "wo", "gate", "up", "down"):
                layer[name] = (orc.quantize(codec, layer[name]),) + layer[name].shape
        w["head"] = (orc.quantize(codec, w["head"]),) + w["head"].shape
    w["codec"] = codec
    return w


K_SCALE_FIELDS = {orc.Q2_K: [80, 82], orc.Q3_K: [108], orc.Q4_K: [0, 2], orc.Q5_K: [0, 2], orc.Q6_K: [208]}
# block scale that puts decoded values of random code bytes near 0.02 (codes x 6-bit sub-scales span about 500 / 100)
K_SCALE_SIGMA = {orc.Q2_K: 2e-4, orc.Q3_K: 4e-4, orc.Q4_K: 8e-5, orc.Q5_K: 4e-5, orc.Q6_K: 1e-5}


def random_k_quant(codec, rows, columns, rng):
    """Packed K-quant rows from random bytes (every bit pattern of the code and sub-scale bytes is legal) with small finite
    f16 block scales, so that the decoded weights have the magnitude of a model's."""
    bb, bv = orc.block_bytes(codec), orc.block_values(codec)
    blocks = rows * columns // bv
    raw = rng.integers(0, 256, size=(blocks, bb), dtype=np.uint8)
    for off in K_SCALE_FIELDS[codec]:
        scale = rng.normal(0, K_SCALE_SIGMA[codec], size=blocks).astype(np.float16)
        raw[:, off:off + 2] = scale.view(np.uint8).reshape(blocks, 2)
    return raw.reshape(rows, columns // bv * bb)


def make_mixed_weights(cfg, codecs, seed=0):
    """Like make_weights, but every projection carries its own codec: `codecs` maps wq, wk, wv, wo, gate, up, down and head
    to a K-quant. Packed entries are (bytes, rows, columns, codec)."""
    rng = np.random.default_rng(seed)
    d, qw, kvw, ffn, V = cfg["d_model"], cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"], cfg["ffn"], cfg["vocab"]
    shapes = dict(wq=(qw, d), wk=(kvw, d), wv=(kvw, d), wo=(d, qw), gate=(ffn, d), up=(ffn, d), down=(d, ffn))
    packed = lambda name, shape: (random_k_quant(codecs[name], shape[0], shape[1], rng),) + shape + (codecs[name],)
    w = {"tok_embd": rng.normal(0.0, 0.02, size=(V, d)).astype(np.float32), "layers": []}
    for _ in range(cfg["layers"]):
        layer = dict(attn_norm=np.ones(d, np.float32), ffn_norm=np.ones(d, np.float32))
        for name, shape in shapes.items():
            layer[name] = packed(name, shape)
        w["layers"].append(layer)
    w["out_norm"] = np.ones(d, np.float32)
    w["head"] = packed("head", (V, d))
    w["codec"] = 0
    return w


SLOTS = dict(attn_norm=1, wq=2, wk=3, wv=4, wo=5, ffn_norm=6, gate=7, up=8, down=9)


def load_into(target, weights):
    """target: oracle.Decoder or effect_torch_b200.Executable (same set_weight signature)."""
    codec = weights["codec"]

    def put(slot, layer, value):
        if isinstance(value, tuple):
            packed, rows, cols = value[:3]
            target.set_weight(slot, layer, packed, codec=value[3] if len(value) > 3 else codec, rows=rows, columns=cols)
        else:
            target.set_weight(slot, layer, value)

    put(0, 0, weights["tok_embd"])
    for l, layer in enumerate(weights["layers"]):
        for name, slot in SLOTS.items():
            put(slot, l, layer[name])
    put(10, 0, weights["out_norm"])
    put(11, 0, weights["head"])


def oracle_decoder(cfg, weights, batch, window=None):
    dec = orc.Decoder(cfg["layers"], cfg["d_model"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"], cfg["vocab"],
                      eps=cfg["rms_eps"], theta=cfg["rope_theta"], window=window, batch=batch)
    load_into(dec, weights)
    dec.set_mode(faithful=False, threads=max(1, min(8, orc.max_threads())))
    return dec


def rel_err(actual, expected):
    """max |a - e| / max |e| — the relative error the 2e-3 logits/attention tolerance is stated in."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    denom = max(np.abs(expected).max(), 1e-30)
    return float(np.abs(actual - expected).max() / denom)
