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
