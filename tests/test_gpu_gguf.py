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
