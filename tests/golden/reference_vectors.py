"""Golden vectors transcribed (as data) from the reference project's own tests.

Each entry names the reference test that holds it (path relative to the reference
project root). They pin the CPU oracle; the GPU parity tests reuse them as
known-answer cases.
"""
import numpy as np

Q4_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 2, 8, 10, 11, 12, 13, 14


def _q2_bytes():  # crates/runtime-cpu/src/quantized.rs:629-646
    b = np.zeros(84, dtype=np.uint8)
    for i in range(16):
        b[i] = 0x10 | (i % 15 + 1)
    b[16:80] = 0xE4
    b[80:84] = [0x00, 0x3C, 0x00, 0x38]
    return b


def _q3_bytes():  # quantized.rs:651-674
    b = np.zeros(110, dtype=np.uint8)
    b[0:32] = 0xAA
    b[32:96] = 0xE4
    b[96:104] = 0x11
    b[104:108] = 0xAA
    b[108:110] = [0x00, 0x3C]
    return b


def _scale_min_fixture(n, quant_offset, high_offset):  # quantized.rs:679-714
    b = np.zeros(n, dtype=np.uint8)
    b[0:4] = [0x00, 0x3C, 0x00, 0x38]
    b[4:8] = 1
    b[8:12] = 2
    b[12:16] = 0x21
    if high_offset is not None:
        b[high_offset:high_offset + 32] = 0x99
    b[quant_offset:] = 0xE4
    return b


def _q6_bytes():  # quantized.rs:722-741
    b = np.zeros(210, dtype=np.uint8)
    b[0:192] = 0xE4
    for i in range(16):
        b[192 + i] = i + 1
    b[208:210] = [0x00, 0x38]
    return b


# codec -> (block bytes, group width, expected value of each group)   quantized.rs:647-778
K_QUANT_FIXTURES = {
    Q2_K: (_q2_bytes(), 16,
           [-0.5, -0.5, 2.5, 3.5, 9.5, 11.5, 20.5, 23.5, -0.5, -0.5, 10.5, 11.5, 25.5, 27.5, 44.5, 2.5]),
    Q3_K: (_q3_bytes(), 16,
           [-4.0, -4.0, 1.0, 1.0, -2.0, -2.0, 3.0, 3.0, -4.0, -4.0, 1.0, 1.0, -2.0, -2.0, 3.0, 3.0]),
    Q4_K: (_scale_min_fixture(144, 16, None), 32, [3.0, 13.0, 3.0, 13.0, 3.0, 13.0, 3.0, 13.0]),
    Q5_K: (_scale_min_fixture(176, 48, 16), 32, [19.0, 13.0, 3.0, 29.0, 19.0, 13.0, 3.0, 29.0]),
    Q6_K: (_q6_bytes(), 16,
           [-14.0, -28.0, -18.0, -24.0, 35.0, 42.0, 105.0, 120.0, -126.0, -140.0, -66.0, -72.0, 91.0, 98.0, 225.0,
            240.0]),
}


def fixture_expected(codec):
    _, width, groups = K_QUANT_FIXTURES[codec]
    return np.repeat(np.asarray(groups, dtype=np.float32), width)


def linear_prefill_case():
    """quantized.rs:827-865 `linear_decodes_blocks_during_prefill`."""
    block = K_QUANT_FIXTURES[Q4_K][0]
    x = np.zeros(1024, dtype=np.float32)
    x[:576] = 1.0
    packed = np.tile(block, 4).reshape(2, 288)
    bias = np.asarray([0.5, -0.5], dtype=np.float32)
    expected = np.asarray([[4096.5, 4095.5], [512.5, 511.5]], dtype=np.float32)
    return dict(codec=Q4_K, x=x.reshape(2, 512), packed=packed, rows=2, columns=512, bias=bias, expected=expected)


def linear_lowered_case():
    """crates/runtime-cpu/src/executable.rs:4881-4918 `quantized_linear_lowers_and_executes`."""
    block = K_QUANT_FIXTURES[Q4_K][0]
    return dict(codec=Q4_K, x=np.ones((1, 256), dtype=np.float32), packed=np.tile(block, 3).reshape(3, 144), rows=3,
                columns=256, bias=None, expected=np.full((1, 3), 2048.0, dtype=np.float32))


def kv_attention_vs_sdpa_case():
    """crates/runtime-cpu/src/napi/mod.rs:4963-5051 `kv_attention_matches_sdpa` (tolerance 1e-6)."""
    q = np.arange(48, dtype=np.float32).reshape(1, 4, 3, 4)
    k = (np.arange(24, 48, dtype=np.float32) * np.float32(0.01)).reshape(1, 2, 3, 4)
    v = (np.arange(48, 72, dtype=np.float32) * np.float32(0.01)).reshape(1, 2, 3, 4)
    return dict(q=q, k=k, v=v, scale=0.5, kv_heads=2, head_dim=4, block_size=4, max_tokens=8, advance=3, tol=1e-6)


# packages/core/test/Inference.test.ts:206-278 — pool of 8 tokens, block 4, 2 KV heads, head dim 1,
# two attention layers (layer 0 windowed to 2, layer 1 full), zero queries and keys.
WINDOWED_CASE = dict(
    max_tokens=8, block_size=4, kv_heads=2, q_heads=4, head_dim=1,
    first_v=[1, 2, 4, 8, 10, 20, 40, 80], first_tokens=[1, 2, 3, 4],
    second_v=[16, 0, 0, 0, 160, 0, 0, 0], second_tokens=[5],
    local_expected=[12, 12, 120, 120], full_expected=[6.2, 6.2, 62, 62], local_window=2,
    third_tokens=[6, 7, 8], overflow_tokens=[9], overflow_message="capacity",
)

# crates/runtime/src/sampling.rs:222-237 and packages/core/test/Sampling.test.ts:92-148
GREEDY_CASES = [([1.0, 4.0, 4.0, 2.0], 1), ([1.0, 4.0, 4.0, 0.0], 1), ([0.0, 3.0, 1.0, 2.0], 1), ([9.0, 1.0, 2.0, 3.0], 0)]

# crates/runtime-cpu/src/pool.rs:263-285
SLAB_F16_CASE = dict(rows=4, width=3, write_rows=[1, 3], values=[1.0, 2.0, 3.0, 4.0, 5.0, 6.0], read_rows=[3, 0, 1],
                     expected=[4.0, 5.0, 6.0, 0.0, 0.0, 0.0, 1.0, 2.0, 3.0])
INT8_ROUNDTRIP_CASE = dict(x=[0.5, -1.0, 0.25, 2.0, 0.0, -0.5, 1.0, 1.0], rows=2, heads=2, d=2, tol=0.02)

# crates/runtime-cpu/src/napi/mod.rs:4922-4953: u8 KV tier, 1 layer, 8 tokens, 2 heads x 4 — the KV part of
# the 1440-byte total (the remaining 1184 bytes are recurrent state, outside this path).
STATE_BYTES_CASE = dict(layers=1, max_tokens=8, kv_heads=2, head_dim=4, dtype_u8_bytes=256)

# crates/runtime-cpu/src/napi/mod.rs:5227-5274
LAST_TOKEN_ROW_CASE = dict(source=np.arange(12, dtype=np.float32).reshape(1, 3, 4), advance=2, expected=[4.0, 5.0, 6.0, 7.0],
                           bad_advances=[0, 4], message="last token row: token advance must be in 1..=3, got {}")


def rope_case():
    """packages/core/test/Attention.test.ts:338-378 — x [1,2,4], theta 10000, offset 0."""
    x = np.asarray([1, 2, 3, 4, 5, 6, 7, 8], dtype=np.float32).reshape(1, 2, 4)
    s0, c0, s1, c1 = np.sin(1.0), np.cos(1.0), np.sin(0.01), np.cos(0.01)
    half = [1, 2, 3, 4, 5 * c0 - 7 * s0, 6 * c1 - 8 * s1, 7 * c0 + 5 * s0, 8 * c1 + 6 * s1]
    inter = [1, 2, 3, 4, 5 * c0 - 6 * s0, 6 * c0 + 5 * s0, 7 * c1 - 8 * s1, 8 * c1 + 7 * s1]
    return x, np.asarray(half), np.asarray(inter)


def pattern(n):
    """packages/core/test/Attention.test.ts:43 — the deterministic input pattern of the attention tests."""
    return [((i * 7 + 3) % 13 - 6) / 4 for i in range(n)]
