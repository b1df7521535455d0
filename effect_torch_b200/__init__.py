"""effect-torch B200 backend: thin Python harness over the C-ABI CUDA library (libetcuda.so).

Class and method names follow the reference's napi surface
(packages/backend-cpu/src/internal/native-addon.ts): NativeKvPool{capacity, freeBlocks,
cachedBlocks, makeSequence}, NativeKvSequence{cursor, release, prefillMatch}, and an Executable
with execute / executeSampled. All compute happens in the library; PyTorch is used only to own
device memory and for torch.distributed plumbing. There is no fallback path: importing the ops
without the built library, or calling them without a CUDA device, raises.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import DecoderConfig

# status classes (include/et_cuda.h) -> BackendError.reason (packages/core/src/Runtime.ts:129-143)
REASONS = {
    1: "backend-unavailable", 2: "unsupported-operation", 3: "invalid-handle", 4: "compilation-failed",
    5: "execution-failed", 6: "transfer-failed", 7: "cancelled", 8: "closed-runtime", 9: "invalid-argument",
}
Q4_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, F32_CODEC = 2, 8, 10, 11, 12, 13, 14, 0
KV_F32, KV_F16, KV_BF16, KV_U8 = 0, 1, 2, 3
HALF_SPLIT, INTERLEAVED_PAIRS = 0, 1
EPILOGUE_NONE, EPILOGUE_RESIDUAL, EPILOGUE_SWIGLU = 0, 1, 2
NO_WINDOW = -1
(W_TOK_EMBD, W_ATTN_NORM, W_Q, W_K, W_V, W_O, W_FFN_NORM, W_GATE, W_UP, W_DOWN, W_OUT_NORM, W_HEAD) = range(12)


class BackendError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status
        self.reason = REASONS.get(status, "execution-failed")


def _check(status: int):
    if status != 0:
        raise BackendError(status, _lib.load().etc_last_error_message().decode())


def _ptr(t):
    """Device/host address of a torch tensor, numpy array or raw int."""
    if t is None:
        return None
    if isinstance(t, int):
        return C.c_void_p(t)
    if isinstance(t, np.ndarray):
        return C.c_void_p(t.ctypes.data)
    return C.c_void_p(t.data_ptr())


def device_count() -> int:
    n = C.c_int(0)
    _check(_lib.load().etc_device_count(C.byref(n)))
    return n.value


def is_available() -> bool:
    """isAvailable() of the addon: the library loads and a CUDA device exists."""
    try:
        return device_count() > 0
    except (ImportError, OSError):
        return False


def encoded_row_bytes(codec: int, columns: int) -> int:
    out = C.c_int64(0)
    _check(_lib.load().etc_encoded_row_bytes(codec, columns, C.byref(out)))
    return out.value


def pool_state_bytes(layers, max_tokens, kv_heads, head_dim, dtype) -> int:
    out = C.c_int64(0)
    _check(_lib.load().etc_pool_state_bytes(layers, max_tokens, kv_heads, head_dim, dtype, C.byref(out)))
    return out.value


def attention_plan(batch, q_heads, kv_heads, head_dim, attended_pages, sm_count=148) -> dict:
    """Split plan of the flash-decoding kernel for tables of `attended_pages` pages (host arithmetic, no device)."""
    splits, pps, nbytes = C.c_int(0), C.c_int(0), C.c_size_t(0)
    _check(_lib.load().etc_kv_attention_plan(batch, q_heads, kv_heads, head_dim, attended_pages, sm_count, C.byref(splits),
                                             C.byref(pps), C.byref(nbytes)))
    return dict(splits=splits.value, pages_per_split=pps.value, partial_bytes=nbytes.value)


def decoder_attention_reserve(cfg: DecoderConfig, max_advance=1, sm_count=148) -> dict:
    """Longest block table a decoder stages per lane and the split-partial bytes it sets aside at finalize."""
    blocks, nbytes = C.c_int(0), C.c_size_t(0)
    _check(_lib.load().etc_decoder_attention_reserve(C.byref(cfg), max_advance, sm_count, C.byref(blocks), C.byref(nbytes)))
    return dict(max_blocks=blocks.value, partial_bytes=nbytes.value)


class Runtime:
    """One device + stream (makeRuntime()). Tensors passed to ops must live on this device."""

    def __init__(self, device: int = 0):
        self.L = _lib.load()
        h = C.c_void_p()
        _check(self.L.etc_runtime_create(device, C.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.L.etc_runtime_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self) -> int:
        s = C.c_void_p()
        _check(self.L.etc_runtime_stream(self.h, C.byref(s)))
        return s.value or 0

    def synchronize(self):
        _check(self.L.etc_runtime_synchronize(self.h))

    @property
    def launch_count(self) -> int:
        n = C.c_uint64(0)
        _check(self.L.etc_runtime_launch_count(self.h, C.byref(n)))
        return n.value

    def capabilities(self) -> dict:
        """dtypes and features like Capabilities (crates/runtime/src/backend.rs:181-206), plus the device's identity."""
        caps = _lib.Capabilities()
        _check(self.L.etc_runtime_capabilities(self.h, C.byref(caps)))
        names = ["f32", "f64", "f16", "bf16", "u8", "u32", "i64"]
        features = ["compilation", "async-execution", "unified-memory"]
        return dict(dtypes=[n for i, n in enumerate(names) if caps.dtype_mask >> i & 1],
                    features=[n for i, n in enumerate(features) if caps.feature_mask >> i & 1],
                    device=caps.device_ordinal, sm_count=caps.sm_count, compute_capability=(caps.compute_major, caps.compute_minor),
                    device_memory_bytes=caps.device_memory_bytes, device_name=caps.device_name.decode())

    @property
    def memory_bytes(self) -> int:
        n = C.c_uint64(0)
        _check(self.L.etc_runtime_memory_bytes(self.h, C.byref(n)))
        return n.value

    # ---- ops on device tensors (torch tensors or raw device addresses) -------------------
    def dequantize_into(self, codec, packed, rows, columns, out):
        _check(self.L.etc_dequantize_into(self.h, codec, _ptr(packed), rows, columns, _ptr(out)))

    def quantize_into(self, codec, x, rows, columns, packed):
        _check(self.L.etc_quantize_into(self.h, codec, _ptr(x), rows, columns, _ptr(packed)))

    def qlinear_into(self, codec, x, vectors, columns, weight, rows, bias, out, cancelled=None):
        flag = None if cancelled is None else C.cast(C.pointer(C.c_int(int(cancelled))), C.c_void_p)
        _check(self.L.etc_qlinear_into(self.h, codec, _ptr(x), vectors, columns, _ptr(weight), rows, _ptr(bias), _ptr(out), flag))

    def qembedding_into(self, codec, indexes, index_is_i64, count, weight, rows, columns, out):
        _check(self.L.etc_qembedding_into(self.h, codec, _ptr(indexes), 1 if index_is_i64 else 0, count, _ptr(weight), rows,
                                          columns, _ptr(out)))

    def linear_f32_into(self, x, m, k, w, n, bias, out):
        _check(self.L.etc_linear_f32_into(self.h, _ptr(x), m, k, _ptr(w), n, _ptr(bias), _ptr(out)))

    def rmsnorm_into(self, x, weight, eps, rows, n, out):
        _check(self.L.etc_rmsnorm_into(self.h, _ptr(x), _ptr(weight), eps, rows, n, _ptr(out)))

    def rope_into(self, x, offsets, n_offsets, theta, layout, batch, heads, steps, head_dim, out):
        _check(self.L.etc_rope_into(self.h, _ptr(x), _ptr(offsets), n_offsets, theta, layout, batch, heads, steps, head_dim, _ptr(out)))

    def swiglu_into(self, gate, up, n, out):
        _check(self.L.etc_swiglu_into(self.h, _ptr(gate), _ptr(up), n, _ptr(out)))

    def add_into(self, a, b, n, out):
        _check(self.L.etc_add_into(self.h, _ptr(a), _ptr(b), n, _ptr(out)))

    def argmax_into(self, logits, rows, vocab, tokens):
        _check(self.L.etc_argmax_into(self.h, _ptr(logits), rows, vocab, _ptr(tokens)))

    def sample_row(self, logits, vocab, temperature=1.0, top_k=None, top_p=1.0, seed=0, counter=0) -> int:
        out = C.c_uint32(0)
        _check(self.L.etc_sample_row(self.h, _ptr(logits), vocab, temperature, 0 if top_k is None else top_k, top_p, seed, counter,
                                     C.byref(out)))
        return out.value

    def sample_rows_into(self, logits, rows, vocab, tokens, temperature=1.0, top_k=None, top_p=1.0, seed=0, counter=0, seeds=None,
                         counters=None):
        """One token per row into the device tensor `tokens` (uint32); per-row (seed, counter) as device u64 tensors, or the scalars."""
        _check(self.L.etc_sample_rows_into(self.h, _ptr(logits), rows, vocab, temperature, 0 if top_k is None else top_k, top_p, seed,
                                           counter, _ptr(seeds), _ptr(counters), _ptr(tokens)))

    def kv_attention_into(self, pool, layer, seqs, batch, active, advance, q, k, v, q_heads, tokens, scale, op_window=None,
                          pool_window=None, out=None):
        arr = (C.c_void_p * max(len(seqs), 1))(*[s.h for s in seqs])
        _check(self.L.etc_kv_attention_into(self.h, pool.h, layer, arr, batch, active, advance, _ptr(q), _ptr(k), _ptr(v), q_heads,
                                            tokens, scale, NO_WINDOW if op_window is None else op_window,
                                            NO_WINDOW if pool_window is None else pool_window, _ptr(out)))


    def kv_append_into(self, pool, layer, seqs, batch, active, advance, k, v, tokens, pool_window=None):
        arr = (C.c_void_p * max(len(seqs), 1))(*[s.h for s in seqs])
        _check(self.L.etc_kv_append_into(self.h, pool.h, layer, arr, batch, active, advance, _ptr(k), _ptr(v), tokens,
                                         NO_WINDOW if pool_window is None else pool_window))

    def kv_attention_decode_into(self, pool, layer, seqs, batch, active, q, k, v, q_heads, scale, op_window=None,
                                 pool_window=None, out=None):
        arr = (C.c_void_p * max(len(seqs), 1))(*[s.h for s in seqs])
        _check(self.L.etc_kv_attention_decode_into(self.h, pool.h, layer, arr, batch, active, _ptr(q), _ptr(k), _ptr(v), q_heads,
                                                   scale, NO_WINDOW if op_window is None else op_window,
                                                   NO_WINDOW if pool_window is None else pool_window, _ptr(out)))

    def peer_allreduce_into(self, rank, world, regions, capacity, buffer, hidden, count, partial, two_shot=False, wait_cycles=0):
        """hidden[:count] += sum over ranks of their partial sums, exchanged through `buffer` of every rank's region
        (device pointers, own rank local); asynchronous. A peer that never arrives turns into BackendError(ETC_EXECUTION) at the next synchronize."""
        arr = (C.c_void_p * world)(*[_ptr(r) for r in regions])
        _check(self.L.etc_peer_allreduce_into(self.h, rank, world, arr, capacity, buffer, _ptr(partial), _ptr(hidden), count,
                                              int(two_shot), wait_cycles))

    def paged_attention_into(self, pool, layer, lanes, tables, batch, max_pages, q, q_heads, scale, out, scratch, scratch_bytes,
                             op_window=None):
        """Flash-decoding over device-resident lane descriptors [batch, 4] i32 and block tables (asynchronous, capturable)."""
        _check(self.L.etc_paged_attention_into(self.h, pool.h, layer, _ptr(lanes), _ptr(tables), batch, max_pages, _ptr(q), q_heads,
                                               scale, NO_WINDOW if op_window is None else op_window, _ptr(out), _ptr(scratch),
                                               scratch_bytes))


def peer_region_bytes(capacity: int, world: int) -> int:
    """Bytes of one rank's exchange region for peer all-reduces of up to `capacity` floats among `world` ranks."""
    return int(_lib.load().etc_peer_region_bytes(capacity, world))


class QWeight:
    """A retained block-quantized matrix in the tensor-core tiling (constantWeights)."""

    def __init__(self, rt: Runtime, codec: int, parts, part_rows, columns: int, interleave8: bool = False, on_device: bool = True):
        self.rt = rt
        n = len(parts)
        ptrs = (C.c_void_p * n)(*[_ptr(p) for p in parts])
        rows = (C.c_int64 * n)(*part_rows)
        h = C.c_void_p()
        _check(rt.L.etc_qweight_create(rt.h, codec, ptrs, rows, n, columns, int(interleave8), int(on_device), C.byref(h)))
        self.h = h
        self.rows = sum(part_rows)
        self.columns = columns
        self.interleave8 = interleave8

    def close(self):
        if getattr(self, "h", None) and getattr(self.rt, "h", None):
            self.rt.L.etc_qweight_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def scratch_bytes(self, vectors: int) -> int:
        out = C.c_size_t(0)
        _check(self.rt.L.etc_qlinear_tiled_scratch_bytes(self.h, vectors, C.byref(out)))
        return out.value

    @property
    def device_bytes(self) -> int:
        b = C.c_uint64(0)
        _check(self.rt.L.etc_qweight_shape(self.h, None, None, None, C.byref(b)))
        return b.value

    def linear_into(self, x, vectors, out, bias=None, residual=None, epilogue=EPILOGUE_NONE, scratch=None, scratch_bytes=0):
        _check(self.rt.L.etc_qlinear_tiled_into(self.rt.h, self.h, _ptr(x), vectors, _ptr(bias), _ptr(residual), epilogue,
                                                _ptr(out), _ptr(scratch), scratch_bytes))

    def linear_static_into(self, x, vectors, out, bias=None, residual=None, epilogue=EPILOGUE_NONE):
        """The same linear with its scratch in the library's fixed device array: the call allocates nothing."""
        _check(self.rt.L.etc_qlinear_tiled_static_into(self.rt.h, self.h, _ptr(x), vectors, _ptr(bias), _ptr(residual),
                                                       epilogue, _ptr(out)))

    def static_scratch_max_bytes(self) -> int:
        out = C.c_size_t(0)
        _check(self.rt.L.etc_qlinear_tiled_static_max_bytes(C.byref(out)))
        return out.value


def tensor_parallel_id() -> bytes:
    """128 bytes made by rank 0 and handed to every rank's `Executable.set_tensor_parallel`."""
    buf = (C.c_uint8 * 128)()
    _check(_lib.load().etc_tp_unique_id(buf))
    return bytes(buf)


class NativeKvPool:
    """native-addon.ts:193-207."""

    def __init__(self, rt: Runtime, layers, kv_heads, head_dim, max_tokens, block_size=16, dtype=KV_F32):
        self.rt = rt
        h = C.c_void_p()
        _check(rt.L.etc_pool_create(rt.h, layers, kv_heads, head_dim, max_tokens, block_size, dtype, C.byref(h)))
        self.h = h
        self.layers, self.kv_heads, self.head_dim = layers, kv_heads, head_dim
        self.max_tokens, self.block_size, self.dtype = max_tokens, block_size, dtype

    def close(self):
        if getattr(self, "h", None) and getattr(self.rt, "h", None):
            self.rt.L.etc_pool_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stats(self):
        a, b, c = C.c_uint32(0), C.c_uint32(0), C.c_uint32(0)
        _check(self.rt.L.etc_pool_stats(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    capacity = property(lambda self: self._stats()[0])
    freeBlocks = property(lambda self: self._stats()[1])
    cachedBlocks = property(lambda self: self._stats()[2])

    def makeSequence(self) -> "NativeKvSequence":
        return NativeKvSequence(self)

    def read_rows(self, layer: int, which: int, rows) -> np.ndarray:
        rows = np.ascontiguousarray(rows, dtype=np.uint32)
        out = np.empty((rows.size, self.kv_heads * self.head_dim), dtype=np.float32)
        _check(self.rt.L.etc_pool_read_rows(self.h, layer, which, _ptr(rows), rows.size, _ptr(out)))
        return out


class NativeKvSequence:
    """native-addon.ts:216-220."""

    def __init__(self, pool: NativeKvPool):
        self.pool = pool
        h = C.c_void_p()
        _check(pool.rt.L.etc_seq_create(pool.h, C.byref(h)))
        self.h = h

    def __del__(self):
        try:
            if getattr(self, "h", None) and getattr(self.pool, "h", None):
                self.pool.rt.L.etc_seq_destroy(self.h)
        except Exception:
            pass
        self.h = None

    @property
    def cursor(self) -> int:
        c = C.c_uint32(0)
        _check(self.pool.rt.L.etc_seq_cursor(self.h, C.byref(c)))
        return c.value

    def release(self):
        _check(self.pool.rt.L.etc_seq_release(self.h))

    def prefillMatch(self, tokens) -> int:
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = C.c_uint32(0)
        _check(self.pool.rt.L.etc_seq_prefill_match(self.h, _ptr(t), t.size, C.byref(out)))
        return out.value

    @property
    def blocks(self):
        n, head = C.c_int64(0), C.c_int64(0)
        _check(self.pool.rt.L.etc_seq_blocks(self.h, None, 0, C.byref(n), C.byref(head)))
        buf = np.zeros(max(n.value, 1), dtype=np.uint32)
        _check(self.pool.rt.L.etc_seq_blocks(self.h, _ptr(buf), n.value, C.byref(n), C.byref(head)))
        return buf[:n.value].copy(), head.value

    @property
    def frontier(self) -> int:
        f = C.c_int64(0)
        _check(self.pool.rt.L.etc_seq_frontier(self.h, C.byref(f)))
        return f.value

    def commit(self, tokens, eviction_start: int = 0):
        t = np.ascontiguousarray(tokens, dtype=np.uint32)
        _check(self.pool.rt.L.etc_seq_commit(self.h, _ptr(t), t.size, eviction_start))

    def rollback(self, frontier: int):
        _check(self.pool.rt.L.etc_seq_rollback(self.h, frontier))


class Executable:
    """The compiled stateful decoder (compile + Executable of native-addon.ts:43-56, 252-257)."""

    def __init__(self, rt: Runtime, *, layers, d_model, q_heads, kv_heads, head_dim, ffn, vocab, rms_eps=1e-5, rope_theta=10000.0,
                 rope_layout=HALF_SPLIT, window=None, batch=1, max_tokens=256, block_size=16, kv_dtype=KV_F32, exact=False,
                 max_advance=1, vocab_global=None, head_first_row=0):
        self.rt = rt
        self.cfg = DecoderConfig(layers, d_model, q_heads, kv_heads, head_dim, ffn, vocab, rms_eps, rope_theta, rope_layout,
                                 NO_WINDOW if window is None else window, batch, max_tokens, block_size, kv_dtype, int(exact))
        h = C.c_void_p()
        _check(rt.L.etc_decoder_create(rt.h, C.byref(self.cfg), C.byref(h)))
        self.h = h
        _check(rt.L.etc_decoder_set_max_advance(self.h, max_advance))
        if vocab_global is not None:  # vocabulary-parallel head: `vocab` rows of it from `head_first_row` on
            _check(rt.L.etc_decoder_set_head_shard(self.h, vocab_global, head_first_row))
        self.vocab, self.batch = vocab, batch

    def close(self):
        if getattr(self, "h", None) and getattr(self.rt, "h", None):
            self.rt.L.etc_decoder_destroy(self.h)
        self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_weight(self, slot, layer, array, codec=F32_CODEC, rows=None, columns=None):
        """Host numpy array (uploaded and retained) or a device torch tensor."""
        if isinstance(array, np.ndarray):
            a = np.ascontiguousarray(array, dtype=np.float32 if codec == F32_CODEC else np.uint8)
            if codec == F32_CODEC and rows is None:
                rows, columns = (a.shape if a.ndim == 2 else (1, a.size))
            _check(self.rt.L.etc_decoder_set_weight(self.h, slot, layer, codec, _ptr(a), rows, columns))
        else:
            if codec == F32_CODEC and rows is None:
                rows, columns = (tuple(array.shape) if array.dim() == 2 else (1, array.numel()))
            _check(self.rt.L.etc_decoder_set_weight_device(self.h, slot, layer, codec, _ptr(array), rows, columns))

    def finalize(self):
        _check(self.rt.L.etc_decoder_finalize(self.h))

    def set_tensor_parallel(self, rank: int, world: int, unique_id: bytes | None):
        """Joins this rank's decoder (built with local geometry and weight shards) to the tensor-parallel group.
        Every rank calls this with the id rank 0 made with `tensor_parallel_id()`; it returns when all have joined."""
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id) if unique_id is not None else None
        _check(self.rt.L.etc_decoder_set_tensor_parallel(self.h, rank, world, buf))

    def peer_exchange_handle(self) -> bytes:
        """64-byte CUDA IPC handle of this rank's all-reduce exchange region (after finalize and set_tensor_parallel)."""
        buf = (C.c_uint8 * 64)()
        _check(self.rt.L.etc_decoder_tp_peer_export(self.h, buf))
        return bytes(buf)

    def use_peer_allreduce(self, handles: list):
        """Switches the all-reduces to the one-shot kernel over peer memory; `handles[r]` is rank r's exchange handle."""
        table = (C.c_uint8 * (64 * len(handles))).from_buffer_copy(b"".join(handles))
        _check(self.rt.L.etc_decoder_tp_peer_import(self.h, table))

    def peer_region(self):
        """(device pointer, bytes) of this rank's exchange region, for hosts that map the regions themselves."""
        ptr, size = C.c_void_p(), C.c_size_t(0)
        _check(self.rt.L.etc_decoder_tp_region(self.h, C.byref(ptr), C.byref(size)))
        return ptr.value, size.value

    def attach_peer_regions(self, regions: list):
        """regions[r]: rank r's region as a device tensor / pointer valid in this process (own slot ignored)."""
        arr = (C.c_void_p * len(regions))(*[_ptr(r) for r in regions])
        _check(self.rt.L.etc_decoder_tp_peer_attach(self.h, arr))

    def set_wait_limit(self, cycles: int):
        """Bound of the waits for a peer inside the step's kernels, in SM clock cycles."""
        _check(self.rt.L.etc_decoder_set_wait_limit(self.h, cycles))

    @staticmethod
    def _seq_array(seqs):
        return (C.c_void_p * max(len(seqs), 1))(*[s.h for s in seqs])

    def execute(self, pool, seqs, tokens, cancelled: bool = False) -> np.ndarray:
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        active, advance = tokens.shape
        logits = np.empty((active, self.vocab), dtype=np.float32)
        flag = C.c_int(int(cancelled))
        _check(self.rt.L.etc_decoder_execute(self.h, pool.h, self._seq_array(seqs), active, _ptr(tokens), advance, _ptr(logits),
                                             C.cast(C.byref(flag), C.c_void_p)))
        return logits

    def executeSampled(self, pool, seqs, tokens, cancelled: bool = False) -> np.ndarray:
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        active, advance = tokens.shape
        out = np.empty(active, dtype=np.uint32)
        flag = C.c_int(int(cancelled))
        _check(self.rt.L.etc_decoder_execute_sampled(self.h, pool.h, self._seq_array(seqs), active, _ptr(tokens), advance, _ptr(out),
                                                     C.cast(C.byref(flag), C.c_void_p)))
        return out

    def generate_greedy(self, pool, seqs, first_tokens, steps: int):
        first = np.ascontiguousarray(first_tokens, dtype=np.uint32).reshape(-1)
        active = first.size
        out = np.empty((steps, active), dtype=np.uint32)
        ms = C.c_float(0.0)
        _check(self.rt.L.etc_decoder_generate_greedy(self.h, pool.h, self._seq_array(seqs), active, _ptr(first), steps, _ptr(out),
                                                     C.byref(ms)))
        return out, ms.value

    def diagnostics(self):
        n, wb, sb = C.c_int(0), C.c_uint64(0), C.c_uint64(0)
        _check(self.rt.L.etc_decoder_diagnostics(self.h, C.byref(n), C.byref(wb), C.byref(sb)))
        return dict(launches_per_step=n.value, weight_bytes=wb.value, workspace_bytes=sb.value)
