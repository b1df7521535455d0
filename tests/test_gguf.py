"""GGUF catalog parser and tensor reader of the C ABI against the oracle restatement, over the reference's own
accept/reject matrix (crates/runtime/src/gguf.rs:1117-1480) rebuilt with a synthetic writer. No GPU needed."""
import struct

import numpy as np
import pytest

import effect_torch_b200 as et
from effect_torch_b200.gguf import GgufFile
from oracle import gguf as og

QV = [og.metadata_entry("general.quantization_version", 4, struct.pack("<I", 2))]
WEIGHT = ("weight", [256], 10, 0, 84)


def both(tmp_path, data: bytes):
    """Parses `data` with the oracle and the library; returns (oracle result or error text, library file or error)."""
    path = tmp_path / "model.gguf"
    path.write_bytes(data)
    try:
        expected = og.parse(data)
    except og.GgufError as e:
        expected = str(e)
    try:
        got = GgufFile(str(path))
    except et.BackendError as e:
        got = e
    return expected, got


def assert_rejected(tmp_path, data, fragment):
    expected, got = both(tmp_path, data)
    assert isinstance(expected, str) and fragment in expected, expected
    assert isinstance(got, et.BackendError), "the library accepted a file the oracle rejects"
    assert str(got) == expected  # same message text
    assert got.reason == "invalid-argument"


def test_f32_and_every_block_codec_shape(tmp_path):
    # the reference's mixed file (gguf.rs:1119-1182) plus this build's two 32-value codecs
    tensors = [("a", [3, 2], 0, 0, 24), ("b", [256, 2], 10, 32, 168), ("c", [256, 2], 11, 224, 220), ("d", [512, 2], 12, 448, 576),
               ("e", [256, 2], 13, 1024, 352), ("f", [256, 2], 14, 1376, 420), ("g", [64, 3], 2, 1824, 108), ("h", [32, 2, 2], 8, 1952, 136)]
    expected, got = both(tmp_path, og.build(QV, tensors))
    assert got.architecture == expected["architecture"] == "test"
    assert [list(t.physical_shape) for t in got.tensors[:6]] == [[2, 3], [2, 84], [2, 110], [2, 288], [2, 176], [2, 210]]
    for t, e in zip(got.tensors, expected["tensors"]):
        assert (t.name, t.codec, list(t.logical_shape), list(t.physical_shape), t.data_offset, t.byte_len) == (
            e["name"], e["codec"], e["logical_shape"], e["physical_shape"], e["data_offset"], e["byte_len"])
    assert got.tensors[6].format == "Q4_0" and list(got.tensors[6].physical_shape) == [3, 36]
    assert list(got.tensors[7].logical_shape) == [2, 2, 32] and list(got.tensors[7].physical_shape) == [4, 34]
    assert got.index("e") == 4
    with pytest.raises(et.BackendError, match="no tensor named"):
        got.index("missing")


def test_every_metadata_scalar_and_array_type(tmp_path):
    entries = [
        og.metadata_entry("u8", 0, struct.pack("<B", 200)), og.metadata_entry("i8", 1, struct.pack("<b", -5)),
        og.metadata_entry("u16", 2, struct.pack("<H", 60000)), og.metadata_entry("i16", 3, struct.pack("<h", -300)),
        og.metadata_entry("u32", 4, struct.pack("<I", 4000000000)), og.metadata_entry("i32", 5, struct.pack("<i", -70000)),
        og.metadata_entry("f32", 6, struct.pack("<f", 1.5)), og.metadata_entry("bool", 7, b"\x01"),
        og.metadata_entry("string", 8, og.string_value("héllo")), og.metadata_entry("u64", 10, struct.pack("<Q", 2 ** 53 - 1)),
        og.metadata_entry("i64", 11, struct.pack("<q", -(2 ** 53 - 1))), og.metadata_entry("f64", 12, struct.pack("<d", -2.25)),
        og.metadata_entry("array.u16", 9, og.array_value(2, 3, struct.pack("<3H", 7, 8, 9))),
        og.metadata_entry("array.string", 9, og.array_value(8, 2, og.string_value("x") + og.string_value("yz"))),
        og.metadata_entry("array.empty", 9, og.array_value(6, 0, b"")),
    ]
    expected, got = both(tmp_path, og.build(entries, [("t", [4], 0, 0, 16)]))
    assert len(got.metadata) == len(entries) + 2 == len(expected["metadata"])
    by_key = {m["key"]: m for m in got.metadata}
    for key, kind, value in expected["metadata"]:
        m = by_key[key]
        if kind == 9:
            _, element, values = value
            assert m["array"] and m["count"] == len(values) and m["kind"] == {2: "u16", 8: "string", 6: "f32"}[element]
            assert m["first"] == (values[0] if values else None)
        else:
            assert not m["array"] and m["value"] == value, key


REJECTS = [
    ("bad magic", lambda: b"X" + og.build(QV, [WEIGHT])[1:], "invalid magic"),
    ("bad version", lambda: og.build(QV, [WEIGHT], version=2), "unsupported version 2; expected version 3"),
    ("duplicate key", lambda: og.build([og.metadata_entry("general.architecture", 8, og.string_value("other"))], [WEIGHT]), "duplicate metadata key"),
    ("unsafe u64", lambda: og.build([og.metadata_entry("unsafe", 10, struct.pack("<Q", 2 ** 64 - 1))], [WEIGHT]), "JavaScript safe integer"),
    ("alignment 3", lambda: og.build(QV, [WEIGHT], alignment=3), "positive power of two"),
    ("duplicate tensor", lambda: og.build(QV, [WEIGHT, WEIGHT]), "duplicate tensor name"),
    ("overlap", lambda: og.build(QV, [WEIGHT, ("other", [256], 10, 32, 84)]), "overlap"),
    ("partial block", lambda: og.build(QV, [("weight", [255], 10, 0, 84)]), "not divisible by 256 for Q2_K"),
    ("partial q4_0 block", lambda: og.build(QV, [("weight", [48], 2, 0, 36)]), "not divisible by 32 for Q4_0"),
    ("type code 1", lambda: og.build(QV, [("weight", [256], 1, 0, 84)]), "unsupported GGML tensor type code 1"),
    ("zero dimension", lambda: og.build(QV, [("weight", [0], 10, 0, 84)]), "invalid dimension 0"),
    ("truncated", lambda: og.build(QV, [WEIGHT])[:-1], "exceeds file size"),
    ("rank 5", lambda: og.build(QV, [("weight", [2, 2, 2, 2, 2], 0, 0, 128)]), "rank must be in 1..=4, got 5"),
    ("unaligned offset", lambda: og.build(QV, [("weight", [4], 0, 8, 16)]), "is not aligned to 32"),
    ("missing quantization version", lambda: og.build([], [WEIGHT]), "missing general.quantization_version"),
    ("quantization version type", lambda: og.build([og.metadata_entry("general.quantization_version", 5, struct.pack("<i", 2))], [WEIGHT]), "must be u32"),
    ("quantization version 3", lambda: og.build([og.metadata_entry("general.quantization_version", 4, struct.pack("<I", 3))], [WEIGHT]), "expected 2"),
    ("nested array", lambda: og.build([og.metadata_entry("n", 9, og.array_value(9, 1, b""))], [("t", [4], 0, 0, 16)]), "nested metadata arrays"),
    ("bad bool", lambda: og.build([og.metadata_entry("b", 7, b"\x02")], [("t", [4], 0, 0, 16)]), "invalid boolean metadata byte 2"),
    ("bad utf8", lambda: og.build([og.metadata_entry("s", 8, struct.pack("<Q", 2) + b"\xc3\x28")], [("t", [4], 0, 0, 16)]), "not valid UTF-8"),
    ("empty architecture", lambda: og.build([], [("t", [4], 0, 0, 16)], architecture=""), "must not be empty"),
    ("long tensor name", lambda: og.build([], [("n" * 65, [4], 0, 0, 16)]), "resource limit 64"),
]


@pytest.mark.parametrize("label,make,fragment", REJECTS, ids=[r[0] for r in REJECTS])
def test_malformed_files_are_rejected_with_the_reference_messages(tmp_path, label, make, fragment):
    assert_rejected(tmp_path, make(), fragment)


def test_counts_over_resource_limits_are_rejected_before_allocation(tmp_path):
    header = b"GGUF" + struct.pack("<IQQ", 3, 0, 4097)
    assert_rejected(tmp_path, header, "resource limit")
    key_length = b"GGUF" + struct.pack("<IQQ", 3, 0, 1) + struct.pack("<Q", 65536) + bytes(64)
    assert_rejected(tmp_path, key_length, "resource limit")
    huge_count = b"GGUF" + struct.pack("<IQQ", 3, 60000, 0) + bytes(64)
    assert_rejected(tmp_path, huge_count, "exceeds the remaining file")


def test_f32_needs_no_quantization_version_and_cancellation_stops_before_io(tmp_path):
    expected, got = both(tmp_path, og.build([], [("t", [4], 0, 0, 16)]))
    assert len(got.tensors) == 1 and got.tensors[0].format == "F32"
    with pytest.raises(et.BackendError, match="gguf: operation aborted") as info:
        GgufFile(str(tmp_path / "model.gguf"), cancelled=True)
    assert info.value.reason == "cancelled"
    with pytest.raises(et.BackendError, match="I/O failed") as info:
        GgufFile(str(tmp_path / "absent.gguf"))
    assert info.value.reason == "transfer-failed"


def test_tensor_payload_fills_a_caller_buffer_exactly(tmp_path):
    rng = np.random.default_rng(0)
    a = rng.integers(0, 256, size=24, dtype=np.uint8).tobytes()
    b = rng.integers(0, 256, size=3 * 36, dtype=np.uint8).tobytes()
    data = og.build(QV, [("a", [3, 2], 0, 0, 24), ("b", [64, 3], 2, 32, 108)], payloads={"a": a, "b": b})
    _, got = both(tmp_path, data)
    assert got.read_tensor(0).tobytes() == a
    assert got.read_tensor(1).tobytes() == b
    with pytest.raises(et.BackendError, match='tensor "b" requires 108 destination bytes, got 7'):
        got.read_tensor(1, out=np.empty(7, dtype=np.uint8))
    with pytest.raises(et.BackendError, match="operation aborted"):
        got.read_tensor(1, cancelled=True)
