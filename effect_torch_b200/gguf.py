"""GGUF files through the C ABI: inspect the catalog (inspectGguf) and load tensors to host or device memory (loadGguf),
packages/backend-cpu/src/internal/native-addon.ts:316-325."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from . import BackendError, _check, _ptr  # noqa: F401  (BackendError re-exported for callers)

VALUE_KINDS = {0: "u8", 1: "i8", 2: "u16", 3: "i16", 4: "u32", 5: "i32", 6: "f32", 7: "bool", 8: "string", 10: "u64", 11: "i64", 12: "f64"}
FORMAT_NAMES = {0: "F32", 2: "Q4_0", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}
_SIGNED_BITS = {1: 8, 3: 16, 5: 32, 11: 64}


@dataclass
class TensorInfo:
    name: str
    codec: int
    format: str
    logical_shape: tuple
    physical_shape: tuple
    data_offset: int
    byte_len: int


class GgufFile:
    def __init__(self, path: str, cancelled: bool = False):
        self.L = _lib.load()
        flag = C.c_int(int(cancelled))
        h = C.c_void_p()
        _check(self.L.etc_gguf_open(path.encode(), C.cast(C.byref(flag), C.c_void_p), C.byref(h)))
        self.h = h
        arch, nm, nt = C.c_char_p(), C.c_int64(0), C.c_int64(0)
        _check(self.L.etc_gguf_summary(self.h, C.byref(arch), C.byref(nm), C.byref(nt)))
        self.architecture = arch.value.decode()
        self.metadata = [self._metadata(i) for i in range(nm.value)]
        self.tensors = [self._tensor(i) for i in range(nt.value)]

    def close(self):
        if getattr(self, "h", None):
            self.L.etc_gguf_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _metadata(self, i):
        key, s = C.c_char_p(), C.c_char_p()
        vt, et_, n, bits, real = C.c_int(0), C.c_int(0), C.c_int64(0), C.c_uint64(0), C.c_double(0.0)
        _check(self.L.etc_gguf_metadata(self.h, i, C.byref(key), C.byref(vt), C.byref(et_), C.byref(n), C.byref(bits), C.byref(real), C.byref(s)))
        kind = vt.value if vt.value != 9 else et_.value

        def scalar():
            if kind in (6, 12):
                return real.value
            if kind == 8:
                return s.value.decode()
            if kind == 7:
                return bool(bits.value)
            if kind in _SIGNED_BITS:
                v = bits.value
                return v - (1 << 64) if v >> 63 else v
            return bits.value

        entry = {"key": key.value.decode(), "kind": VALUE_KINDS[kind], "array": vt.value == 9}
        if vt.value == 9:
            entry["count"] = n.value
            entry["first"] = scalar() if n.value else None
        else:
            entry["value"] = scalar()
        return entry

    def _tensor(self, i):
        name = C.c_char_p()
        codec, rank = C.c_int(0), C.c_int(0)
        logical, physical = (C.c_int64 * 4)(), (C.c_int64 * 4)()
        off, nbytes = C.c_uint64(0), C.c_uint64(0)
        _check(self.L.etc_gguf_tensor(self.h, i, C.byref(name), C.byref(codec), C.byref(rank), logical, physical, C.byref(off), C.byref(nbytes)))
        prank = rank.value if codec.value == 0 else 2
        return TensorInfo(name.value.decode(), codec.value, FORMAT_NAMES[codec.value], tuple(logical[:rank.value]), tuple(physical[:prank]),
                          off.value, nbytes.value)

    def index(self, name: str) -> int:
        out = C.c_int64(0)
        _check(self.L.etc_gguf_find_tensor(self.h, name.encode(), C.byref(out)))
        return out.value

    def read_tensor(self, index: int, out: np.ndarray | None = None, cancelled: bool = False) -> np.ndarray:
        """Payload bytes of one tensor in a caller-owned (or new) uint8 array of exactly byte_len bytes."""
        info = self.tensors[index]
        if out is None:
            out = np.empty(info.byte_len, dtype=np.uint8)
        flag = C.c_int(int(cancelled))
        _check(self.L.etc_gguf_read_tensor_into(self.h, index, _ptr(out), out.nbytes, C.cast(C.byref(flag), C.c_void_p)))
        return out

    def load_tensor_device(self, rt, index: int, device_tensor, cancelled: bool = False):
        """Streams the payload into a device buffer (a torch uint8/float32 tensor of exactly byte_len bytes)."""
        flag = C.c_int(int(cancelled))
        nbytes = device_tensor.numel() * device_tensor.element_size()
        _check(self.L.etc_gguf_load_tensor_device(rt.h, self.h, index, _ptr(device_tensor), nbytes, C.cast(C.byref(flag), C.c_void_p)))
        return device_tensor


# ---- a Llama-shaped decoder straight from a GGUF file ---------------------------------------------------------------
LLAMA_TENSORS = {  # GGUF tensor name pattern -> weight slot of the decoder (include/et_cuda.h etc_weight_slot)
    "attn_norm": 1, "attn_q": 2, "attn_k": 3, "attn_v": 4, "attn_output": 5, "ffn_norm": 6, "ffn_gate": 7, "ffn_up": 8, "ffn_down": 9,
}


def llama_geometry(f: GgufFile) -> dict:
    """Decoder geometry from the `<arch>.*` metadata keys of a Llama-family file and the embedding tensor's shape."""
    meta = {m["key"]: m.get("value") for m in f.metadata if not m["array"]}
    arch = f.architecture

    def need(key):
        if f"{arch}.{key}" not in meta:
            raise BackendError(9, f"gguf: metadata key {arch}.{key} is missing")
        return meta[f"{arch}.{key}"]

    d_model, q_heads = int(need("embedding_length")), int(need("attention.head_count"))
    embd = f.tensors[f.index("token_embd.weight")]
    return dict(layers=int(need("block_count")), d_model=d_model, q_heads=q_heads,
                kv_heads=int(meta.get(f"{arch}.attention.head_count_kv", q_heads)),
                head_dim=int(meta.get(f"{arch}.attention.key_length", d_model // q_heads)), ffn=int(need("feed_forward_length")),
                vocab=int(embd.logical_shape[0]), rms_eps=float(meta.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)),
                rope_theta=float(meta.get(f"{arch}.rope.freq_base", 10000.0)))


def load_llama_decoder(rt, path: str, *, batch: int, max_tokens: int, block_size: int = 16, kv_dtype=None, exact: bool = False,
                       max_advance: int = 1, rope_layout=None, window=None):
    """Builds an `Executable` whose weights are streamed from `path` into device memory (packed tensors stay packed and are
    re-tiled on the device at finalize). Tensors: token_embd, blk.N.{attn_norm, attn_q, attn_k, attn_v, attn_output,
    ffn_norm, ffn_gate, ffn_up, ffn_down}, output_norm, output (falls back to token_embd when the head is tied).
    Returns (executable, geometry)."""
    import torch

    from . import HALF_SPLIT, KV_F16, W_HEAD, W_OUT_NORM, W_TOK_EMBD, Executable

    f = GgufFile(path)
    try:
        g = llama_geometry(f)
        dec = Executable(rt, layers=g["layers"], d_model=g["d_model"], q_heads=g["q_heads"], kv_heads=g["kv_heads"], head_dim=g["head_dim"],
                         ffn=g["ffn"], vocab=g["vocab"], rms_eps=g["rms_eps"], rope_theta=g["rope_theta"],
                         rope_layout=HALF_SPLIT if rope_layout is None else rope_layout, window=window, batch=batch, max_tokens=max_tokens,
                         block_size=block_size, kv_dtype=KV_F16 if kv_dtype is None else kv_dtype, exact=exact, max_advance=max_advance)
        names = {t.name: i for i, t in enumerate(f.tensors)}

        def bind(slot, layer, name):
            if name not in names:
                raise BackendError(9, f'gguf: tensor "{name}" is missing')
            info = f.tensors[names[name]]
            if info.codec == 0:
                buf = torch.empty(info.byte_len // 4, dtype=torch.float32, device=f"cuda:{rt.device}")
            else:
                buf = torch.empty(info.byte_len, dtype=torch.uint8, device=f"cuda:{rt.device}")
            torch.cuda.synchronize()
            f.load_tensor_device(rt, names[name], buf)
            if len(info.logical_shape) == 1:
                dec.set_weight(slot, layer, buf, codec=0, rows=1, columns=info.logical_shape[0])
            else:
                rows = int(np.prod(info.logical_shape[:-1]))
                dec.set_weight(slot, layer, buf, codec=info.codec, rows=rows, columns=info.logical_shape[-1])

        bind(W_TOK_EMBD, 0, "token_embd.weight")
        for layer in range(g["layers"]):
            for stem, slot in LLAMA_TENSORS.items():
                bind(slot, layer, f"blk.{layer}.{stem}.weight")
        bind(W_OUT_NORM, 0, "output_norm.weight")
        bind(W_HEAD, 0, "output.weight" if "output.weight" in names else "token_embd.weight")
        dec.finalize()
        return dec, g
    finally:
        f.close()
