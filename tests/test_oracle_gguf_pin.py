"""Pins the oracle's block codecs, its weight quantizer and both GGUF parsers against gguf-py (the `gguf` Python package,
the published implementation of the format, version 0.19.0 in this image).

The reference defers the byte formats to upstream GGML (crates/runtime-cpu/src/quantized.rs:6-8) and ships neither Q4_0 /
Q8_0 nor a quantizer, so these checks are what ties the two 32-value codecs of this build to the published definition:
  * quantize: gguf.quants.quantize(Q4_0 / Q8_0) == oracle.quantize, byte for byte;
  * dequantize: gguf.quants.dequantize == oracle.dequantize, bit for bit, for Q4_0, Q8_0 and the five K-quants;
  * files: a Llama-shaped file written by gguf.GGUFWriter is read by the oracle parser and by the library's parser
    (crates/runtime/src/gguf.rs:682-946) with the names, shapes, offsets and bytes that gguf.GGUFReader reports.
No GPU needed."""
import numpy as np
import pytest

gguf = pytest.importorskip("gguf")
from gguf import GGMLQuantizationType as T  # noqa: E402
from gguf import quants  # noqa: E402

import oracle as orc  # noqa: E402
from oracle import gguf as og  # noqa: E402

QUANTIZED = [(orc.Q4_0, T.Q4_0), (orc.Q8_0, T.Q8_0)]
K_QUANTS = [(orc.Q2_K, T.Q2_K), (orc.Q3_K, T.Q3_K), (orc.Q4_K, T.Q4_K), (orc.Q5_K, T.Q5_K), (orc.Q6_K, T.Q6_K)]


def sample_matrices():
    """Seeded matrices that cover ordinary weights, all-zero blocks, ties in magnitude, rounding ties and extremes."""
    rng = np.random.default_rng(2024)
    out = [rng.normal(0.0, 0.02, size=(8, 256)).astype(np.float32), rng.normal(0.0, 1.0, size=(3, 96)).astype(np.float32),
           np.zeros((2, 64), np.float32)]
    ties = np.zeros((4, 32), np.float32)
    ties[0, 3], ties[0, 17] = -1.0, 1.0          # equal magnitudes, opposite signs: the first one sets the scale
    ties[1, :] = np.linspace(-1.0, 1.0, 32)      # both extremes present
    ties[2, :] = 0.5                             # constant block
    ties[3, ::2], ties[3, 1::2] = 0.0625, -0.0625
    out.append(ties)
    half_steps = (np.arange(-16, 16, dtype=np.float32) + 0.5) / 8.0   # values that land on rounding ties for Q4_0
    out.append(np.stack([half_steps, -half_steps, half_steps * 127.0 / 15.5, np.roll(half_steps, 5)]))
    big = rng.normal(0.0, 1.0, size=(2, 64)).astype(np.float32)
    big[0] *= 6.0e4                              # near the top of the f16 scale range
    big[1] *= 1.0e-6                             # scale becomes an f16 subnormal
    out.append(big)
    return out


@pytest.mark.parametrize("codec,kind", QUANTIZED, ids=["Q4_0", "Q8_0"])
def test_quantizer_matches_gguf_py_byte_for_byte(codec, kind):
    for x in sample_matrices():
        expected = quants.quantize(x, kind)
        got = orc.quantize(codec, x)
        assert got.shape == expected.shape
        assert np.array_equal(got, expected), f"{kind.name}: quantizer bytes differ for a {x.shape} sample"


@pytest.mark.parametrize("codec,kind", QUANTIZED, ids=["Q4_0", "Q8_0"])
def test_q4_0_q8_0_dequantize_matches_gguf_py_bit_for_bit(codec, kind):
    rng = np.random.default_rng(7)
    for x in sample_matrices():
        packed = quants.quantize(x, kind)
        expected = quants.dequantize(packed, kind)
        got = orc.dequantize(codec, packed, x.shape[0], x.shape[1])
        assert np.array_equal(got.view(np.uint32), expected.astype(np.float32).view(np.uint32))
    # arbitrary payload bytes under finite f16 scales (not only what a quantizer emits)
    bb = orc.block_bytes(codec)
    raw = rng.integers(0, 256, size=(6, 8 * bb), dtype=np.uint8)
    scales = rng.normal(0.0, 0.05, size=(6, 8)).astype(np.float16)
    raw.reshape(6, 8, bb)[:, :, 0:2] = scales.view(np.uint8).reshape(6, 8, 2)
    expected = quants.dequantize(raw, kind)
    got = orc.dequantize(codec, raw, 6, 8 * 32)
    assert np.array_equal(got.view(np.uint32), expected.astype(np.float32).view(np.uint32))


def finite_f16_fields(raw, bb, offsets, rng):
    """Overwrites the f16 fields of every block with finite values so that NaN payloads cannot hide a mismatch."""
    blocks = raw.reshape(raw.shape[0], -1, bb)
    for off in offsets:
        vals = rng.normal(0.0, 0.05, size=blocks.shape[:2]).astype(np.float16)
        blocks[:, :, off:off + 2] = vals.view(np.uint8).reshape(blocks.shape[0], blocks.shape[1], 2)
    return raw


@pytest.mark.parametrize("codec,kind", K_QUANTS, ids=[k.name for _, k in K_QUANTS])
def test_k_quant_decoders_match_gguf_py_bit_for_bit(codec, kind):
    # f16 field offsets of the block layouts (crates/runtime-cpu/src/quantized.rs:117-261)
    offsets = {orc.Q2_K: (80, 82), orc.Q3_K: (108,), orc.Q4_K: (0, 2), orc.Q5_K: (0, 2), orc.Q6_K: (208,)}[codec]
    rng = np.random.default_rng(100 + codec)
    bb = orc.block_bytes(codec)
    raw = finite_f16_fields(rng.integers(0, 256, size=(5, 3 * bb), dtype=np.uint8), bb, offsets, rng)
    expected = quants.dequantize(raw, kind).astype(np.float32)
    got = orc.dequantize(codec, raw, 5, 3 * 256)
    assert np.array_equal(got.view(np.uint32), expected.view(np.uint32)), f"{kind.name} decoder differs from gguf-py"


# ---- files written by gguf-py ----------------------------------------------------------------------------------------
LLAMA = dict(layers=2, d_model=64, q_heads=4, kv_heads=2, ffn=128, vocab=96)


def write_llama_file(path, codec_kind):
    """A small Llama-shaped file written by gguf.GGUFWriter: f32 embeddings and norms, projections in `codec_kind`."""
    rng = np.random.default_rng(5)
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_block_count(LLAMA["layers"])
    w.add_embedding_length(LLAMA["d_model"])
    w.add_head_count(LLAMA["q_heads"])
    w.add_head_count_kv(LLAMA["kv_heads"])
    w.add_feed_forward_length(LLAMA["ffn"])
    w.add_layer_norm_rms_eps(1e-5)
    w.add_rope_freq_base(10000.0)
    w.add_quantization_version(2)
    payloads = {}

    def dense(name, *shape):
        a = rng.normal(0.0, 0.02, size=shape).astype(np.float32)
        payloads[name] = (a.view(np.uint8).reshape(-1).copy(), 0, shape)
        w.add_tensor(name, a)

    def packed(name, rows, cols):
        a = rng.normal(0.0, 0.02, size=(rows, cols)).astype(np.float32)
        q = quants.quantize(a, codec_kind)
        payloads[name] = (q.reshape(-1).copy(), int(codec_kind), (rows, cols))
        w.add_tensor(name, q, raw_dtype=codec_kind)

    d, kvw = LLAMA["d_model"], LLAMA["d_model"] // LLAMA["q_heads"] * LLAMA["kv_heads"]
    dense("token_embd.weight", LLAMA["vocab"], d)
    for l in range(LLAMA["layers"]):
        dense(f"blk.{l}.attn_norm.weight", d)
        packed(f"blk.{l}.attn_q.weight", d, d)
        packed(f"blk.{l}.attn_k.weight", kvw, d)
        packed(f"blk.{l}.attn_v.weight", kvw, d)
        packed(f"blk.{l}.attn_output.weight", d, d)
        dense(f"blk.{l}.ffn_norm.weight", d)
        packed(f"blk.{l}.ffn_gate.weight", LLAMA["ffn"], d)
        packed(f"blk.{l}.ffn_up.weight", LLAMA["ffn"], d)
        packed(f"blk.{l}.ffn_down.weight", d, LLAMA["ffn"])
    dense("output_norm.weight", d)
    packed("output.weight", LLAMA["vocab"], d)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return payloads


@pytest.mark.parametrize("kind", [T.Q4_0, T.Q8_0], ids=["Q4_0", "Q8_0"])
def test_parsers_read_a_file_written_by_gguf_py(tmp_path, kind):
    import effect_torch_b200 as et
    from effect_torch_b200.gguf import GgufFile, llama_geometry

    path = tmp_path / "llama.gguf"
    payloads = write_llama_file(path, kind)
    reader = gguf.GGUFReader(str(path))
    data = path.read_bytes()
    parsed = og.parse(data)                      # the oracle's restatement of parse_gguf
    lib_file = GgufFile(str(path))               # the C-ABI parser
    try:
        assert parsed["architecture"] == "llama" == lib_file.architecture
        assert len(reader.tensors) == len(parsed["tensors"]) == len(lib_file.tensors) == len(payloads)
        by_name = {t["name"]: t for t in parsed["tensors"]}
        for i, rt_ in enumerate(reader.tensors):
            name = rt_.name
            o, l = by_name[name], lib_file.tensors[lib_file.index(name)]
            want_bytes, want_codec, want_shape = payloads[name]
            # gguf-py reports dimensions least-major first; both parsers report the logical (row-major) shape
            assert tuple(int(d) for d in reversed(rt_.shape)) == tuple(o["logical_shape"]) == l.logical_shape == tuple(want_shape)
            assert int(rt_.tensor_type) == o["codec"] == l.codec == want_codec
            assert int(rt_.data_offset) == o["data_offset"] == l.data_offset
            assert int(rt_.n_bytes) == o["byte_len"] == l.byte_len == want_bytes.size
            got = lib_file.read_tensor(lib_file.index(name))
            assert np.array_equal(got, want_bytes)
            assert np.array_equal(np.frombuffer(data, np.uint8, o["byte_len"], o["data_offset"]), want_bytes)
            assert np.array_equal(np.asarray(rt_.data).view(np.uint8).reshape(-1), want_bytes)
        g = llama_geometry(lib_file)
        assert (g["layers"], g["d_model"], g["q_heads"], g["kv_heads"], g["ffn"], g["vocab"]) == (
            LLAMA["layers"], LLAMA["d_model"], LLAMA["q_heads"], LLAMA["kv_heads"], LLAMA["ffn"], LLAMA["vocab"])
        assert g["head_dim"] == LLAMA["d_model"] // LLAMA["q_heads"] and g["rope_theta"] == 10000.0
        # metadata keys and scalar values agree with gguf-py's reader
        lib_meta = {m["key"]: m for m in lib_file.metadata}
        for key, field in reader.fields.items():
            if key.startswith("GGUF."):
                continue                          # header pseudo-fields of the reader, not metadata entries
            assert key in lib_meta, key
            if len(field.types) == 1 and field.types[0] != gguf.GGUFValueType.STRING:
                assert lib_meta[key]["value"] == pytest.approx(field.parts[field.data[0]][0].item())
        assert isinstance(et.BackendError(9, "x"), Exception)
    finally:
        lib_file.close()


def test_packed_rows_of_a_gguf_py_file_decode_to_gguf_py_values(tmp_path):
    """End of the chain: bytes read through the C-ABI parser, decoded by the oracle, equal gguf-py's own dequantisation."""
    from effect_torch_b200.gguf import GgufFile

    path = tmp_path / "llama.gguf"
    write_llama_file(path, T.Q4_0)
    reader = gguf.GGUFReader(str(path))
    f = GgufFile(str(path))
    try:
        for rt_ in reader.tensors:
            if int(rt_.tensor_type) == 0:
                continue
            info = f.tensors[f.index(rt_.name)]
            rows, cols = info.logical_shape
            ours = orc.dequantize(info.codec, f.read_tensor(f.index(rt_.name)), rows, cols)
            theirs = quants.dequantize(np.asarray(rt_.data), rt_.tensor_type).astype(np.float32).reshape(rows, cols)
            assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32))
    finally:
        f.close()
