"""Test infrastructure: CPU restatement of the reference's GGUF v3 header parser (crates/runtime/src/gguf.rs:682-946),
in plain Python over a bytes object, and a writer for synthetic files. Only tests may import this module.

Pinned against the reference's own tests (gguf.rs:1117-1480): the physical shapes of its mixed F32/K-quant file, the
accept/reject matrix and the message substrings those tests assert. Type codes 2 (Q4_0) and 8 (Q8_0) are this build's
addition (32-value blocks); the reference rejects them like every code outside {0, 10..14}."""
from __future__ import annotations

import struct

JS_SAFE = 9007199254740991
MAX_HEADER = 64 << 20
LIMITS = dict(metadata=4096, tensor=65536, key=65535, name=64, string=16 << 20, array=1048576)
BLOCK = {2: (32, 18), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
NAMES = {0: "F32", 2: "Q4_0", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}
SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    pass


def _invalid(message):
    return GgufError("gguf: " + message)


class _Reader:
    def __init__(self, data: bytes):
        self.data, self.pos, self.file_len = data, 0, len(data)

    def take(self, n):  # HeaderReader::read_exact (:366-392)
        end = self.pos + n
        if end > self.file_len:
            raise _invalid("unexpected end of file in header")
        if end > MAX_HEADER:
            raise _invalid(f"header exceeds the {MAX_HEADER}-byte resource limit")
        out = self.data[self.pos:end]
        self.pos = end
        return out

    def scalar(self, fmt):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def count(self, value, what, minimum, maximum):  # HeaderReader::count (:462-487)
        if value > maximum:
            raise _invalid(f"{what} count {value} exceeds the resource limit {maximum}")
        remaining = max(0, min(self.file_len, MAX_HEADER) - self.pos)
        if minimum > 0 and value > remaining // minimum:
            raise _invalid(f"{what} count {value} exceeds the remaining file")
        return value

    def string(self, what, maximum):  # HeaderReader::read_string (:492-503)
        n = self.count(self.scalar("<Q"), what, 1, maximum)
        raw = self.take(n)
        try:
            return raw.decode("utf-8")
        except UnicodeDecodeError:
            raise _invalid(f"{what} is not valid UTF-8")


def _value(r, kind, in_array=False):  # read_metadata_value (:618-646), read_array (:536-616)
    if kind in SCALARS:
        v = r.scalar(SCALARS[kind])
        if kind == 10 and v > JS_SAFE:
            raise _invalid(f"metadata u64{' array' if in_array else ''} value {v} is outside the JavaScript safe integer range")
        if kind == 11 and abs(v) > JS_SAFE:
            raise _invalid(f"metadata i64{' array' if in_array else ''} value {v} is outside the JavaScript safe integer range")
        return v
    if kind == 7:
        b = r.scalar("<B")
        if b > 1:
            raise _invalid(f"invalid boolean metadata byte {b}")
        return bool(b)
    if kind == 8:
        return r.string("metadata array string" if in_array else "metadata string", LIMITS["string"])
    if kind == 9 and not in_array:
        element = r.scalar("<I")
        if element == 9:
            raise _invalid("nested metadata arrays are not supported by this parser")
        n = r.scalar("<Q")
        minimum = {0: 1, 1: 1, 7: 1, 2: 2, 3: 2, 4: 4, 5: 4, 6: 4, 8: 8, 10: 8, 11: 8, 12: 8}.get(element)
        if minimum is None:
            raise _invalid(f"unsupported metadata array element type {element}")
        n = r.count(n, "metadata array", minimum, LIMITS["array"])
        return ("array", element, [_value(r, element, True) for _ in range(n)])
    raise _invalid(f"unsupported metadata value type {kind}")


def parse(data: bytes) -> dict:
    """parse_gguf (:682-946) over an in-memory file. Returns architecture, metadata [(key, kind, value)], tensors
    [dict(name, codec, logical_shape, physical_shape, data_offset, byte_len)]."""
    r = _Reader(data)
    if r.take(4) != b"GGUF":
        raise _invalid("invalid magic")
    version = r.scalar("<I")
    if version != 3:
        raise _invalid(f"unsupported version {version}; expected version 3")
    tensor_count, metadata_count = r.scalar("<Q"), r.scalar("<Q")
    metadata_count = r.count(metadata_count, "metadata", 13, LIMITS["metadata"])
    tensor_count = r.count(tensor_count, "tensor", 32, LIMITS["tensor"])
    metadata, keys = [], set()
    for _ in range(metadata_count):
        key = r.string("metadata key", LIMITS["key"])
        if not key:
            raise _invalid("metadata key must not be empty")
        if key in keys:
            raise _invalid(f'duplicate metadata key "{key}"')
        keys.add(key)
        kind = r.scalar("<I")
        metadata.append((key, kind, _value(r, kind)))
    table = {k: (kind, v) for k, kind, v in metadata}
    if "general.architecture" not in table:
        raise _invalid("missing general.architecture metadata")
    kind, arch = table["general.architecture"]
    if kind != 8:
        raise _invalid("general.architecture metadata must be a string")
    if not arch:
        raise _invalid("general.architecture metadata must not be empty")
    alignment = 32
    if "general.alignment" in table:
        kind, alignment = table["general.alignment"]
        if kind != 4:
            raise _invalid("general.alignment metadata must be u32")
    if alignment == 0 or alignment & (alignment - 1):
        raise _invalid(f"general.alignment must be a positive power of two, got {alignment}")
    raws, names, quantized = [], set(), False
    for _ in range(tensor_count):
        name = r.string("tensor name", LIMITS["name"])
        if not name:
            raise _invalid("tensor name must not be empty")
        if name in names:
            raise _invalid(f'duplicate tensor name "{name}"')
        names.add(name)
        rank = r.scalar("<I")
        if not 1 <= rank <= 4:
            raise _invalid(f'tensor "{name}" rank must be in 1..=4, got {rank}')
        dims = []
        for _ in range(rank):
            d = r.scalar("<Q")
            if d == 0 or d > JS_SAFE:
                raise _invalid(f'tensor "{name}" has invalid dimension {d}')
            dims.append(d)
        code = r.scalar("<I")
        if code not in NAMES:
            raise _invalid(f"unsupported GGML tensor type code {code}")
        quantized |= code != 0
        offset = r.scalar("<Q")
        if offset % alignment:
            raise _invalid(f'tensor "{name}" offset {offset} is not aligned to {alignment}')
        raws.append((name, dims, code, offset))
    if quantized:
        if "general.quantization_version" not in table:
            raise _invalid("missing general.quantization_version metadata for quantized tensors")
        kind, qv = table["general.quantization_version"]
        if kind != 4:
            raise _invalid("general.quantization_version metadata must be u32")
        if qv != 2:
            raise _invalid(f"unsupported general.quantization_version {qv}; expected 2")
    data_start = (r.pos + alignment - 1) // alignment * alignment
    if data_start > r.file_len:
        raise _invalid("aligned tensor-data section starts beyond the file")
    tensors = []
    for name, dims, code, offset in raws:
        logical = list(reversed(dims))
        if code == 0:
            n = 1
            for d in logical:
                n *= d
            physical, byte_len = list(logical), n * 4
        else:
            bv, bb = BLOCK[code]
            if dims[0] % bv:
                raise _invalid(f'tensor "{name}" least-major dimension {dims[0]} is not divisible by {bv} for {NAMES[code]}')
            rows = 1
            for d in dims[1:]:
                rows *= d
            physical, byte_len = [rows, dims[0] // bv * bb], rows * (dims[0] // bv * bb)
        if byte_len >= 1 << 64:
            raise _invalid(f'tensor "{name}" byte length overflows')
        start = data_start + offset
        end = start + byte_len
        if end > r.file_len:
            raise _invalid(f'tensor "{name}" range [{start}, {end}) exceeds file size {r.file_len}')
        tensors.append(dict(name=name, codec=code, logical_shape=logical, physical_shape=physical, data_offset=start, byte_len=byte_len))
    ordered = sorted(tensors, key=lambda t: t["data_offset"])
    for a, b in zip(ordered, ordered[1:]):
        if b["data_offset"] < a["data_offset"] + a["byte_len"]:
            raise _invalid(f'tensor ranges for "{a["name"]}" and "{b["name"]}" overlap')
    return dict(architecture=arch, metadata=metadata, tensors=tensors)


# ---- writer for synthetic files (mirrors the builder in the reference's tests, gguf.rs:1034-1103) -------------------
def _string(s: str) -> bytes:
    raw = s.encode()
    return struct.pack("<Q", len(raw)) + raw


def metadata_entry(key: str, kind: int, payload: bytes) -> bytes:
    return _string(key) + struct.pack("<I", kind) + payload


def string_value(s: str) -> bytes:
    return _string(s)


def array_value(kind: int, count: int, payload: bytes) -> bytes:
    return struct.pack("<IQ", kind, count) + payload


def build(extra_metadata, tensors, alignment=32, architecture="test", payloads=None, version=3, magic=b"GGUF") -> bytes:
    """extra_metadata: list of metadata_entry() byte strings; tensors: list of (name, dims (least-major first), code,
    relative offset, byte length). The data section is zero-filled unless `payloads` maps names to bytes."""
    entries = [metadata_entry("general.architecture", 8, string_value(architecture)),
               metadata_entry("general.alignment", 4, struct.pack("<I", alignment))] + list(extra_metadata)
    out = bytearray(magic + struct.pack("<IQQ", version, len(tensors), len(entries)))
    for e in entries:
        out += e
    for name, dims, code, offset, _ in tensors:
        out += _string(name) + struct.pack("<I", len(dims))
        for d in dims:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", code, offset)
    aligned = (len(out) + alignment - 1) // alignment * alignment if alignment else len(out)
    out += bytes(aligned - len(out))
    length = max([offset + nbytes for _, _, _, offset, nbytes in tensors], default=0)
    data = bytearray(length)
    for name, _, _, offset, nbytes in tensors:
        if payloads and name in payloads:
            data[offset:offset + nbytes] = payloads[name]
    return bytes(out + data)
