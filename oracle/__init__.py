"""ctypes/numpy front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

The oracle restates the reference CPU backend's arithmetic for the paged-KV decode path
(see ``et_oracle.cpp`` for the per-routine reference citations). Only the test suite, the
smoke check and the benchmark's CPU-baseline leg may import this package; the product
library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libet_oracle.so")

Q4_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 2, 8, 10, 11, 12, 13, 14
CODEC_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q2_K: "Q2_K", Q3_K: "Q3_K", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}
F32, F16, BF16, U8 = 0, 1, 2, 3
HALF_SPLIT, INTERLEAVED = 0, 1
NO_WINDOW = -1


def build(force: bool = False) -> str:
    """Compile the oracle shared library (make -C oracle) if it is missing or stale."""
    src = os.path.join(_HERE, "et_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _declare(_lib)
    return _lib


_p = C.c_void_p
_ll = C.c_longlong
_d = C.c_double
_i = C.c_int
_u64 = C.c_uint64
_u32 = C.c_uint32


def _declare(L):
    def sig(name, res, *args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("orc_block_values", _i, _i)
    sig("orc_block_bytes", _i, _i)
    sig("orc_encoded_row_bytes", _ll, _i, _ll)
    sig("orc_decode_block", _i, _i, _p, _ll, _p)
    sig("orc_dequantize", _i, _i, _p, _ll, _ll, _p)
    sig("orc_quantize_q4_0", None, _p, _ll, _ll, _p)
    sig("orc_quantize_q8_0", None, _p, _ll, _ll, _p)
    sig("orc_qlinear", _i, _i, _p, _ll, _ll, _p, _ll, _p, _p, _p)
    sig("orc_qlinear_mt", _i, _i, _p, _ll, _ll, _p, _ll, _p, _p, _i)
    sig("orc_qembedding", _i, _i, _p, _ll, _p, _ll, _ll, _p, _p)
    sig("orc_matmul_f32", None, _p, _ll, _ll, _p, _ll, _ll, _p, _ll, _ll, _ll)
    sig("orc_linear_rows_f32", None, _p, _ll, _ll, _p, _ll, _p, _i)
    sig("orc_rms_norm", None, _p, _p, _d, _p, _ll, _ll)
    sig("orc_rotary", None, _p, _p, _ll, _d, _d, _i, _p, _ll, _ll, _ll, _ll)
    sig("orc_silu_mul", None, _p, _p, _p, _ll)
    sig("orc_add", None, _p, _p, _p, _ll)
    sig("orc_sdpa_forward", None, _p, _p, _p, _d, _i, _ll, _p, _ll, _ll, _ll, _ll, _ll, _ll, _ll)
    sig("orc_argmax", _ll, _p, _ll)
    sig("orc_random_unit", _d, _u64, _u64)
    sig("orc_sample_logits", _ll, _p, _ll, _d, _ll, _d, _u64, _u64)
    sig("orc_last_token_row", _i, _p, _ll, _ll, _ll, _p)
    sig("orc_quantize_int8", None, _p, _ll, _ll, _ll, _p, _p)
    sig("orc_dequantize_int8", None, _p, _p, _ll, _ll, _ll, _p)
    sig("orc_chain_hash", _u64, _u64, _p, _ll)
    sig("orc_hash_seed", _u64)
    sig("orc_pool_create", _p, _i, _i, _i, _i, _i, _i, C.c_char_p, _i)
    sig("orc_pool_destroy", None, _p)
    sig("orc_pool_capacity", _i, _p)
    sig("orc_pool_free_blocks", _i, _p)
    sig("orc_pool_cached_blocks", _i, _p)
    sig("orc_pool_alloc_block", _ll, _p)
    sig("orc_pool_take_block", _ll, _p, _u64)
    sig("orc_pool_unref_block", None, _p, _u32)
    sig("orc_pool_set_hash", None, _p, _u32, _u64)
    sig("orc_pool_block_hash", _i, _p, _u32, _p)
    sig("orc_pool_refcount", _i, _p, _u32)
    sig("orc_state_bytes", _ll, _ll, _ll, _ll, _ll, _i)
    sig("orc_pool_write_rows_f32", None, _p, _i, _i, _p, _ll, _p)
    sig("orc_pool_read_rows_f32", None, _p, _i, _i, _p, _ll, _p)
    sig("orc_pool_read_rows_dequant", None, _p, _i, _i, _p, _ll, _p)
    sig("orc_seq_create", _p, _p)
    sig("orc_seq_release", None, _p)
    sig("orc_seq_destroy", None, _p)
    sig("orc_seq_cursor", _ll, _p)
    sig("orc_seq_head", _ll, _p)
    sig("orc_seq_last_hash", _u64, _p)
    sig("orc_seq_num_blocks", _ll, _p)
    sig("orc_seq_blocks", None, _p, _p)
    sig("orc_seq_set_advance", None, _p, _ll)
    sig("orc_seq_set_cursor", None, _p, _ll)
    sig("orc_seq_push_block", None, _p, _u32)
    sig("orc_seq_note_tokens", None, _p, _p, _ll)
    sig("orc_seq_prefill_match", _ll, _p, _p, _ll)
    sig("orc_seq_evict", None, _p, _ll)
    sig("orc_kv_attention", _i, _p, _i, _p, _ll, _ll, _p, _p, _p, _ll, _ll, _ll, _ll, _d, _ll, _ll, _p, _p, _i, _i,
        C.c_char_p, _i)
    sig("orc_decoder_create", _p, _i, _i, _i, _i, _i, _i, _i, _d, _d, _i, _ll, _i)
    sig("orc_decoder_destroy", None, _p)
    sig("orc_decoder_set_mode", None, _p, _i, _i)
    sig("orc_decoder_set_weight", _i, _p, _i, _i, _i, _p, _ll, _ll)
    sig("orc_decoder_execute", _i, _p, _p, _p, _ll, _p, _ll, _p, _p, _i, C.c_char_p, _i)
    sig("orc_max_threads", _i)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


class OracleError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


# ------------------------------------------------------------------ codecs
def block_values(codec):
    return lib().orc_block_values(codec)


def block_bytes(codec):
    return lib().orc_block_bytes(codec)


def encoded_row_bytes(codec, columns):
    v = lib().orc_encoded_row_bytes(codec, columns)
    return None if v < 0 else v


def decode_block(codec, block):
    block = _u8(block)
    out = np.empty(block_values(codec) or 1, dtype=np.float32)
    if lib().orc_decode_block(codec, _ptr(block), block.size, _ptr(out)) != 0:
        raise OracleError(-1, f"{CODEC_NAMES.get(codec, codec)} block has {block.size} bytes, expected {block_bytes(codec)}")
    return out


def dequantize(codec, packed, rows, columns):
    packed = _u8(packed)
    out = np.empty((rows, columns), dtype=np.float32)
    if lib().orc_dequantize(codec, _ptr(packed), rows, columns, _ptr(out)) != 0:
        raise OracleError(-1, f"logical row width {columns} is invalid for {CODEC_NAMES.get(codec, codec)}")
    return out


def quantize(codec, x):
    x = _f32(x)
    rows, columns = x.shape
    row_bytes = encoded_row_bytes(codec, columns)
    if row_bytes is None:
        raise OracleError(-1, f"logical row width {columns} is invalid for {CODEC_NAMES.get(codec, codec)}")
    out = np.empty((rows, row_bytes), dtype=np.uint8)
    if codec == Q4_0:
        lib().orc_quantize_q4_0(_ptr(x), rows, columns, _ptr(out))
    elif codec == Q8_0:
        lib().orc_quantize_q8_0(_ptr(x), rows, columns, _ptr(out))
    else:
        raise OracleError(-1, "the oracle only quantizes to Q4_0 and Q8_0")
    return out


def qlinear(codec, x, packed, rows, columns, bias=None, cancelled=False, threads=0):
    """threads == 0: reference-faithful scalar loop; > 0: fair multi-core variant (same results)."""
    x = _f32(x)
    packed = _u8(packed)
    vectors = x.size // columns
    out = np.empty(x.shape[:-1] + (rows,), dtype=np.float32)
    bias_a = None if bias is None else _f32(bias)
    if threads > 0:
        rc = lib().orc_qlinear_mt(codec, _ptr(x), vectors, columns, _ptr(packed), rows, _ptr(bias_a), _ptr(out), threads)
    else:
        flag = C.c_int(1 if cancelled else 0)
        rc = lib().orc_qlinear(codec, _ptr(x), vectors, columns, _ptr(packed), rows, _ptr(bias_a), _ptr(out),
                               C.cast(C.byref(flag), C.c_void_p))
    if rc == 1:
        raise OracleError(1, "operation aborted")
    if rc != 0:
        raise OracleError(rc, f"quantized_linear: logical row width {columns} is invalid")
    return out


def qembedding(codec, indexes, packed, rows, columns):
    idx = np.ascontiguousarray(indexes, dtype=np.int64)
    packed = _u8(packed)
    out = np.empty(idx.shape + (columns,), dtype=np.float32)
    bad = C.c_longlong(0)
    rc = lib().orc_qembedding(codec, _ptr(idx), idx.size, _ptr(packed), rows, columns, _ptr(out), C.cast(C.byref(bad), C.c_void_p))
    if rc == 2:
        raise OracleError(2, f"quantized_embedding: index {bad.value} is outside 0..{rows}")
    if rc != 0:
        raise OracleError(rc, "quantized_embedding: invalid geometry")
    return out


# ------------------------------------------------------------------ dense ops
def matmul(a, b):
    a = _f32(a)
    b = np.asarray(b, dtype=np.float32)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_matmul_f32(_ptr(a), k, 1, C.c_void_p(b.ctypes.data), b.strides[0] // 4, b.strides[1] // 4, _ptr(out), m, n, k)
    return out


def linear_rows(x, w, threads=1):
    x = _f32(x)
    w = _f32(w)
    n, k = w.shape
    m = x.size // k
    out = np.empty(x.shape[:-1] + (n,), dtype=np.float32)
    lib().orc_linear_rows_f32(_ptr(x), m, k, _ptr(w), n, _ptr(out), threads)
    return out


def rms_norm(x, weight, eps):
    x = _f32(x)
    n = x.shape[-1]
    w = None if weight is None else _f32(weight)
    out = np.empty_like(x)
    lib().orc_rms_norm(_ptr(x), _ptr(w), eps, _ptr(out), x.size // n, n)
    return out


def rotary(x, offsets, theta, layout=HALF_SPLIT, sign=1.0):
    x = _f32(x)
    offs = np.ascontiguousarray(offsets, dtype=np.int64).reshape(-1)
    batch = 1 if x.ndim == 2 else x.shape[0]
    rows = int(np.prod(x.shape[:-2])) if x.ndim > 2 else 1
    out = np.empty_like(x)
    lib().orc_rotary(_ptr(x), _ptr(offs), offs.size, theta, sign, layout, _ptr(out), batch, rows, x.shape[-2], x.shape[-1])
    return out


def silu_mul(gate, up):
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().orc_silu_mul(_ptr(gate), _ptr(up), _ptr(out), gate.size)
    return out


def sdpa_forward(q, k, v, scale, causal=True, window=None):
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, hq, tq, d = q.shape
    _, hkv, tk, _ = k.shape
    dv = v.shape[-1]
    out = np.empty((b, hq, tq, dv), dtype=np.float32)
    lib().orc_sdpa_forward(_ptr(q), _ptr(k), _ptr(v), scale, int(causal), -1 if window is None else window, _ptr(out),
                           b, hq, hkv, tq, tk, d, dv)
    return out


def argmax(logits):
    logits = _f32(logits)
    tok = lib().orc_argmax(_ptr(logits), logits.size)
    if tok < 0:
        raise OracleError(7, f"sample: logit {-tok - 1} is not finite")
    return tok


def random_unit(seed, counter):
    return lib().orc_random_unit(seed, counter)


def sample_logits(logits, temperature=1.0, top_k=None, top_p=1.0, seed=0, counter=0):
    logits = _f32(logits)
    tok = lib().orc_sample_logits(_ptr(logits), logits.size, temperature, 0 if top_k is None else top_k, top_p, seed, counter)
    if tok <= -2000000000:
        code = -(tok + 2000000000)
        raise OracleError(code, {1: "sample: logits must be non-empty", 2: "sample: temperature must be finite and non-negative",
                                 3: "sample: topP must be finite and in (0, 1]", 4: "sample: topK must be in [1, n]",
                                 5: "sample: vocabulary exceeds limit 1048576"}[code])
    if tok < 0:
        raise OracleError(7, f"sample: logit {-tok - 1} is not finite")
    return tok


def last_token_row(source, advance):
    source = _f32(source)
    _, steps, width = source.shape
    out = np.empty(width, dtype=np.float32)
    if lib().orc_last_token_row(_ptr(source), steps, width, advance, _ptr(out)) != 0:
        raise OracleError(1, f"last token row: token advance must be in 1..={steps}, got {advance}")
    return out


def quantize_int8(x, rows, heads, d):
    x = _f32(x)
    q = np.empty(rows * heads * d, dtype=np.uint8)
    s = np.empty(rows * heads, dtype=np.float32)
    lib().orc_quantize_int8(_ptr(x), rows, heads, d, _ptr(q), _ptr(s))
    return q, s


def dequantize_int8(q, scales, rows, heads, d):
    q, scales = _u8(q), _f32(scales)
    out = np.empty(rows * heads * d, dtype=np.float32)
    lib().orc_dequantize_int8(_ptr(q), _ptr(scales), rows, heads, d, _ptr(out))
    return out


def chain_hash(previous, tokens):
    t = np.ascontiguousarray(tokens, dtype=np.uint32)
    return lib().orc_chain_hash(previous, _ptr(t), t.size)


HASH_SEED = 0xCBF29CE484222325


def state_bytes(layers, max_tokens, kv_heads, head_dim, dtype):
    return lib().orc_state_bytes(layers, max_tokens, kv_heads, head_dim, dtype)


# ------------------------------------------------------------------ pool / sequences
class Pool:
    def __init__(self, layers, kv_heads, head_dim, max_tokens, block_size=16, dtype=F32):
        err = C.create_string_buffer(256)
        self.h = lib().orc_pool_create(layers, kv_heads, head_dim, max_tokens, block_size, dtype, err, 256)
        if not self.h:
            raise OracleError(-1, err.value.decode())
        self.layers, self.kv_heads, self.head_dim = layers, kv_heads, head_dim
        self.max_tokens, self.block_size, self.dtype = max_tokens, block_size, dtype

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_pool_destroy(self.h)
            self.h = None

    capacity = property(lambda self: lib().orc_pool_capacity(self.h))
    free_blocks = property(lambda self: lib().orc_pool_free_blocks(self.h))
    cached_blocks = property(lambda self: lib().orc_pool_cached_blocks(self.h))

    def alloc_block(self):
        b = lib().orc_pool_alloc_block(self.h)
        return None if b < 0 else b

    def take_block(self, h):
        b = lib().orc_pool_take_block(self.h, h)
        return None if b < 0 else b

    def unref_block(self, b):
        lib().orc_pool_unref_block(self.h, b)

    def set_hash(self, b, h):
        lib().orc_pool_set_hash(self.h, b, h)

    def block_hash(self, b):
        h = C.c_uint64(0)
        return h.value if lib().orc_pool_block_hash(self.h, b, C.cast(C.byref(h), C.c_void_p)) else None

    def refcount(self, b):
        return lib().orc_pool_refcount(self.h, b)

    def write_rows(self, layer, which, rows, src):
        rows = np.ascontiguousarray(rows, dtype=np.uint32)
        src = _f32(src)
        lib().orc_pool_write_rows_f32(self.h, layer, which, _ptr(rows), rows.size, _ptr(src))

    def read_rows(self, layer, which, rows, dequant=False):
        rows = np.ascontiguousarray(rows, dtype=np.uint32)
        out = np.empty((rows.size, self.kv_heads * self.head_dim), dtype=np.float32)
        fn = lib().orc_pool_read_rows_dequant if dequant else lib().orc_pool_read_rows_f32
        fn(self.h, layer, which, _ptr(rows), rows.size, _ptr(out))
        return out

    def make_sequence(self):
        return Sequence(self)


class Sequence:
    def __init__(self, pool):
        self.pool = pool
        self.h = lib().orc_seq_create(pool.h)

    def __del__(self):
        if getattr(self, "h", None) and getattr(self.pool, "h", None):
            lib().orc_seq_destroy(self.h)
        self.h = None

    cursor = property(lambda self: lib().orc_seq_cursor(self.h))
    head = property(lambda self: lib().orc_seq_head(self.h))
    last_hash = property(lambda self: lib().orc_seq_last_hash(self.h))

    @property
    def blocks(self):
        n = lib().orc_seq_num_blocks(self.h)
        out = np.empty(n, dtype=np.uint32)
        if n:
            lib().orc_seq_blocks(self.h, _ptr(out))
        return out

    def release(self):
        lib().orc_seq_release(self.h)

    def set_advance(self, a):
        lib().orc_seq_set_advance(self.h, a)

    def set_cursor(self, c):
        lib().orc_seq_set_cursor(self.h, c)

    def push_block(self, b):
        lib().orc_seq_push_block(self.h, b)

    def note_tokens(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        lib().orc_seq_note_tokens(self.h, _ptr(t), t.size)

    def prefill_match(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        r = lib().orc_seq_prefill_match(self.h, _ptr(t), t.size)
        if r == -1:
            raise OracleError(-1, "kv sequence is released")
        if r == -2:
            raise OracleError(-2, "prefill match: sequence already holds tokens")
        return r

    def evict(self, start):
        lib().orc_seq_evict(self.h, start)


def _seq_array(seqs):
    arr = (C.c_void_p * len(seqs))(*[s.h for s in seqs])
    return arr


def kv_attention(pool, layer, seqs, active, q, k, v, scale, op_window=None, pool_window=None, eviction_starts=None,
                 mode=0, threads=1):
    """Scatter + attend for one KvAttention node. q [B,Hq,T,D], k/v [B,Hkv,T,D]; returns out [B,Hq,T,D]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, hq, t, d = q.shape
    hkv = k.shape[1]
    out = np.empty_like(q)
    ev = eviction_starts if eviction_starts is not None else np.full(b, np.iinfo(np.uint64).max, dtype=np.uint64)
    err = C.create_string_buffer(256)
    arr = _seq_array(seqs)
    rc = lib().orc_kv_attention(pool.h, layer, C.cast(arr, C.c_void_p), b, active, _ptr(q), _ptr(k), _ptr(v), hq, hkv, t, d,
                                scale, -1 if op_window is None else op_window, -1 if pool_window is None else pool_window,
                                _ptr(out), _ptr(ev), mode, threads, err, 256)
    if rc != 0:
        raise OracleError(rc, err.value.decode())
    return out


# ------------------------------------------------------------------ decoder
W_TOK_EMBD, W_ATTN_NORM, W_Q, W_K, W_V, W_O, W_FFN_NORM, W_GATE, W_UP, W_DOWN, W_OUT_NORM, W_HEAD = range(12)


class Decoder:
    """Llama-shaped decoder over the oracle ops, with the reference's stateful transaction."""

    def __init__(self, layers, d_model, q_heads, kv_heads, head_dim, ffn, vocab, eps=1e-5, theta=10000.0,
                 rope_layout=HALF_SPLIT, window=None, batch=1):
        self.h = lib().orc_decoder_create(layers, d_model, q_heads, kv_heads, head_dim, ffn, vocab, eps, theta, rope_layout,
                                          -1 if window is None else window, batch)
        self.vocab, self.batch = vocab, batch
        self._keep = []

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_decoder_destroy(self.h)
            self.h = None

    def set_mode(self, faithful=True, threads=1):
        lib().orc_decoder_set_mode(self.h, int(faithful), threads)

    def set_weight(self, which, layer, array, codec=0, rows=0, columns=0):
        if codec == 0:
            array = _f32(array)
            if array.ndim == 2:
                rows, columns = array.shape
            else:
                rows, columns = 1, array.size
        else:
            array = _u8(array)
        self._keep.append(array)
        lib().orc_decoder_set_weight(self.h, which, layer, codec, _ptr(array), rows, columns)

    def execute(self, pool, seqs, tokens, want_logits=True, want_sampled=True, layer_limit=0):
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        active, advance = tokens.shape
        logits = np.empty((active, self.vocab), dtype=np.float32) if want_logits else None
        sampled = np.empty(active, dtype=np.uint32) if want_sampled else None
        err = C.create_string_buffer(256)
        arr = _seq_array(seqs)
        rc = lib().orc_decoder_execute(self.h, pool.h, C.cast(arr, C.c_void_p), active, _ptr(tokens), advance, _ptr(logits),
                                       _ptr(sampled), layer_limit, err, 256)
        if rc != 0:
            raise OracleError(rc, err.value.decode())
        return logits, sampled


def max_threads():
    return lib().orc_max_threads()
