"""GGUF tensors streamed into device memory and used in place by the quantized linear."""
import struct

import numpy as np
import pytest
import torch

import oracle as orc
from effect_torch_b200.gguf import GgufFile
from oracle import gguf as og
from tests import helpers
from tests.golden import reference_vectors as gv
from tests.gpu_util import dev, empty, host, runtime

pytestmark = pytest.mark.gpu
QV = [og.metadata_entry("general.quantization_version", 4, struct.pack("<I", 2))]


def test_packed_and_dense_tensors_load_to_the_device_bit_for_bit(tmp_path):
    rng = np.random.default_rng(4)
    rows, cols = 96, 256
    packed = orc.quantize(gv.Q4_0, rng.normal(0, 0.05, size=(rows, cols)).astype(np.float32))
    big = rng.normal(size=(5 << 20,)).astype(np.float32)  # 20 MiB: three staging chunks, the last one partial
    offset_big = (packed.nbytes + 31) // 32 * 32
    data = og.build(QV, [("blk.0.w", [cols, rows], 2, 0, packed.nbytes), ("dense", [big.size], 0, offset_big, big.nbytes)],
                    payloads={"blk.0.w": packed.tobytes(), "dense": big.tobytes()})
    path = tmp_path / "m.gguf"
    path.write_bytes(data)
    f = GgufFile(str(path))
    rt = runtime()
    d_packed = empty((rows, cols // 32 * 18), dtype=torch.uint8)
    f.load_tensor_device(rt, f.index("blk.0.w"), d_packed)
    np.testing.assert_array_equal(host(d_packed), packed)
    d_big = empty((big.size,), dtype=torch.float32)
    f.load_tensor_device(rt, f.index("dense"), d_big)
    np.testing.assert_array_equal(host(d_big), big)
    # the loaded bytes feed the linear directly
    x = rng.normal(size=(3, cols)).astype(np.float32)
    out = empty((3, rows))
    dx = dev(x)
    rt.qlinear_into(gv.Q4_0, dx, 3, cols, d_packed, rows, None, out)
    assert helpers.rel_err(host(out), orc.qlinear(gv.Q4_0, x, packed, rows, cols)) <= 2e-3
    with pytest.raises(Exception, match="destination bytes"):
        f.load_tensor_device(rt, 0, empty((7,), dtype=torch.uint8))


def _llama_file(cfg, weights, path):
    """A synthetic Llama-family GGUF holding `weights` (tests/helpers.make_weights layout, Q4_0 projections)."""
    u32 = lambda v: struct.pack("<I", v)
    meta = QV + [og.metadata_entry("llama.block_count", 4, u32(cfg["layers"])), og.metadata_entry("llama.embedding_length", 4, u32(cfg["d_model"])),
                 og.metadata_entry("llama.attention.head_count", 4, u32(cfg["q_heads"])),
                 og.metadata_entry("llama.attention.head_count_kv", 4, u32(cfg["kv_heads"])),
                 og.metadata_entry("llama.feed_forward_length", 4, u32(cfg["ffn"])),
                 og.metadata_entry("llama.attention.layer_norm_rms_epsilon", 6, struct.pack("<f", cfg["rms_eps"])),
                 og.metadata_entry("llama.rope.freq_base", 6, struct.pack("<f", cfg["rope_theta"]))]
    tensors, payloads, offset = [], {}, 0

    def add(name, value):
        nonlocal offset
        if isinstance(value, tuple):
            packed, rows, cols = value[:3]
            raw, dims, code = packed.tobytes(), [cols, rows], value[3] if len(value) > 3 else weights["codec"]
        else:
            raw, dims, code = np.ascontiguousarray(value, dtype=np.float32).tobytes(), list(reversed(value.shape)), 0
        tensors.append((name, dims, code, offset, len(raw)))
        payloads[name] = raw
        offset = (offset + len(raw) + 31) // 32 * 32

    add("token_embd.weight", weights["tok_embd"])
    stems = dict(attn_norm="attn_norm", wq="attn_q", wk="attn_k", wv="attn_v", wo="attn_output", ffn_norm="ffn_norm", gate="ffn_gate",
                 up="ffn_up", down="ffn_down")
    for l, layer in enumerate(weights["layers"]):
        for ours, theirs in stems.items():
            add(f"blk.{l}.{theirs}.weight", layer[ours])
    add("output_norm.weight", weights["out_norm"])
    add("output.weight", weights["head"])
    path.write_bytes(og.build(meta, tensors, architecture="llama", payloads=payloads))


def test_a_llama_shaped_decoder_loads_from_a_gguf_file(tmp_path):
    import effect_torch_b200 as et
    from effect_torch_b200.gguf import load_llama_decoder

    cfg = helpers.TINY_Q
    weights = helpers.make_weights(cfg, seed=6, codec=gv.Q4_0)
    path = tmp_path / "tiny.gguf"
    _llama_file(cfg, weights, path)
    rt = runtime()
    B = 2
    loaded, geometry = load_llama_decoder(rt, str(path), batch=B, max_tokens=128, kv_dtype=et.KV_F16, max_advance=8)
    assert {k: geometry[k] for k in ("layers", "d_model", "q_heads", "kv_heads", "head_dim", "ffn", "vocab")} == {
        k: cfg[k] for k in ("layers", "d_model", "q_heads", "kv_heads", "head_dim", "ffn", "vocab")}
    direct = et.Executable(rt, layers=cfg["layers"], d_model=cfg["d_model"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                           head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], rms_eps=cfg["rms_eps"], rope_theta=cfg["rope_theta"],
                           batch=B, max_tokens=128, block_size=16, kv_dtype=et.KV_F16, exact=False, max_advance=8)
    helpers.load_into(direct, weights)
    direct.finalize()
    odec = helpers.oracle_decoder(cfg, weights, batch=B)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, orc.F16)
    oseqs = [opool.make_sequence() for _ in range(B)]
    pools = [et.NativeKvPool(rt, cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, et.KV_F16) for _ in range(2)]
    seqs = [[p.makeSequence() for _ in range(B)] for p in pools]
    rng = np.random.default_rng(8)
    for advance in (8, 1, 1):
        toks = rng.integers(0, cfg["vocab"], size=(B, advance)).astype(np.uint32)
        from_file = loaded.execute(pools[0], seqs[0], toks)
        from_memory = direct.execute(pools[1], seqs[1], toks)
        expected, _ = odec.execute(opool, oseqs, toks)
        np.testing.assert_array_equal(from_file, from_memory)  # same bytes, same kernels
        assert helpers.rel_err(from_file, expected) <= 2e-3


def test_a_file_of_mixed_k_quants_loads_onto_the_tiled_kernels(tmp_path):
    """What a "medium" K-quant recipe writes: attn_v and ffn_down at more bits than the other projections. Every tensor keeps
    the codec the file gives it; q/k/v fuse as segments of one tiled weight. Same logits as a decoder fed the same packed
    bytes from memory, and the oracle's within the tolerance of the re-cut K-quants."""
    import effect_torch_b200 as et
    from effect_torch_b200.gguf import load_llama_decoder

    cfg = helpers.TINY_Q
    codecs = dict(wq=gv.Q4_K, wk=gv.Q4_K, wv=gv.Q6_K, wo=gv.Q4_K, gate=gv.Q4_K, up=gv.Q4_K, down=gv.Q6_K, head=gv.Q6_K)
    weights = helpers.make_mixed_weights(cfg, codecs, seed=9)
    path = tmp_path / "tiny_q4_k_m.gguf"
    _llama_file(cfg, weights, path)
    rt = runtime()
    B = 2
    loaded, _ = load_llama_decoder(rt, str(path), batch=B, max_tokens=128, kv_dtype=et.KV_F16, max_advance=8)
    direct = et.Executable(rt, layers=cfg["layers"], d_model=cfg["d_model"], q_heads=cfg["q_heads"], kv_heads=cfg["kv_heads"],
                           head_dim=cfg["head_dim"], ffn=cfg["ffn"], vocab=cfg["vocab"], rms_eps=cfg["rms_eps"], rope_theta=cfg["rope_theta"],
                           batch=B, max_tokens=128, block_size=16, kv_dtype=et.KV_F16, exact=False, max_advance=8)
    helpers.load_into(direct, weights)
    direct.finalize()
    odec = helpers.oracle_decoder(cfg, weights, batch=B)
    opool = orc.Pool(cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, orc.F16)
    oseqs = [opool.make_sequence() for _ in range(B)]
    pools = [et.NativeKvPool(rt, cfg["layers"], cfg["kv_heads"], cfg["head_dim"], 128, 16, et.KV_F16) for _ in range(2)]
    seqs = [[p.makeSequence() for _ in range(B)] for p in pools]
    rng = np.random.default_rng(10)
    for advance in (8, 1, 1):
        toks = rng.integers(0, cfg["vocab"], size=(B, advance)).astype(np.uint32)
        from_file = loaded.execute(pools[0], seqs[0], toks)
        from_memory = direct.execute(pools[1], seqs[1], toks)
        expected, _ = odec.execute(opool, oseqs, toks)
        np.testing.assert_array_equal(from_file, from_memory)
        assert helpers.rel_err(from_file, expected) <= 4e-3
    assert loaded.diagnostics()["launches_per_step"] == direct.diagnostics()["launches_per_step"] > 0
