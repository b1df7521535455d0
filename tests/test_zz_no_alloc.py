"""The allocation-free tiled linear (scratch in the library's fixed device array) against the existing entry point.

Collected last (file name) so that it also runs after every other GPU test has used the runtime's workspace."""
import numpy as np
import pytest
import torch

import effect_torch_b200 as et
import oracle as orc
from tests.golden import reference_vectors as gv
from tests.gpu_util import dev, empty, host, runtime

pytestmark = pytest.mark.gpu


def _weight(codec, rows, columns, seed):
    rng = np.random.default_rng(seed)
    w = rng.normal(0, 0.02, size=(rows, columns)).astype(np.float32)
    return orc.quantize(codec, w)


@pytest.mark.parametrize("codec", [gv.Q4_0, gv.Q8_0])
@pytest.mark.parametrize("rows,columns,vectors", [(512, 4096, 32), (384, 1024, 7), (512, 2048, 300)])
def test_static_scratch_linear_equals_the_existing_entry_point_twice_in_a_row(codec, rows, columns, vectors):
    rt = runtime()
    packed = _weight(codec, rows, columns, rows + vectors)
    qw = et.QWeight(rt, codec, [dev(packed)], [rows], columns)
    assert qw.scratch_bytes(vectors) <= qw.static_scratch_max_bytes()
    rng = np.random.default_rng(vectors)
    for call in range(3):  # calls in a row share the array: a later one must not see an earlier one's leftovers
        x = rng.normal(size=(vectors, columns)).astype(np.float32)
        bias = rng.normal(size=rows).astype(np.float32)
        dx, dbias = dev(x), dev(bias)  # held until the results are read: the runtime's stream is not torch's
        expected, got = empty((vectors, rows)), empty((vectors, rows))
        qw.linear_into(dx, vectors, expected, bias=dbias)
        rt.synchronize()
        torch.cuda.synchronize()
        free_before, tracked_before = torch.cuda.mem_get_info()[0], rt.memory_bytes
        qw.linear_static_into(dx, vectors, got, bias=dbias)
        rt.synchronize()
        if call > 0:  # the first call may still load kernel code; from the second on, device memory must not move at all
            assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free linear changed the free device memory"
            assert rt.memory_bytes == tracked_before
        np.testing.assert_array_equal(host(got), host(expected), err_msg=f"call {call}")


def test_static_scratch_linear_cuts_a_long_call_into_slices_that_fit():
    """A call whose one-pass plan needs more than the fixed array runs 256 vectors at a time; the slices' split plans may
    differ from the one-pass plan, so the result is held to the linear's tolerance, not to bit equality."""
    rt = runtime()
    rows, columns, vectors = 1024, 2048, 700
    packed = _weight(gv.Q4_0, rows, columns, 5)
    qw = et.QWeight(rt, gv.Q4_0, [dev(packed)], [rows], columns)
    assert qw.scratch_bytes(vectors) > qw.static_scratch_max_bytes() >= qw.scratch_bytes(256)
    x = np.random.default_rng(9).normal(size=(vectors, columns)).astype(np.float32)
    dx, got = dev(x), empty((vectors, rows))
    qw.linear_static_into(dx, vectors, got)
    expected = orc.qlinear(gv.Q4_0, x, packed, rows, columns, threads=8)
    err = np.abs(host(got) - expected).max() / np.abs(expected).max()
    assert err <= 2e-3


def test_static_scratch_linear_with_epilogues():
    rt = runtime()
    d, ffn, vectors = 512, 384, 32
    pg, pu = _weight(gv.Q4_0, ffn, d, 1), _weight(gv.Q4_0, ffn, d, 2)
    qgu = et.QWeight(rt, gv.Q4_0, [dev(pg), dev(pu)], [ffn, ffn], d, interleave8=True)
    x = np.random.default_rng(3).normal(size=(vectors, d)).astype(np.float32)
    dx = dev(x)
    expected, got = empty((vectors, ffn)), empty((vectors, ffn))
    qgu.linear_into(dx, vectors, expected, epilogue=et.EPILOGUE_SWIGLU)
    qgu.linear_static_into(dx, vectors, got, epilogue=et.EPILOGUE_SWIGLU)
    np.testing.assert_array_equal(host(got), host(expected))
    with pytest.raises(et.BackendError, match="residual"):
        qgu.linear_static_into(dx, vectors, got, epilogue=et.EPILOGUE_RESIDUAL)


def test_static_scratch_linear_rejects_calls_beyond_its_maximum():
    rt = runtime()
    rows, columns = 8192, 4096
    raw = torch.zeros((rows, columns // 32 * 18), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    qw = et.QWeight(rt, gv.Q4_0, [raw], [rows], columns)
    limit = qw.static_scratch_max_bytes()
    assert limit == 16 << 20
    too_many = next((v for v in (256, 512, 1024, 4096) if qw.scratch_bytes(v) > limit), None)
    assert too_many is not None, "no probe size exceeds the static scratch"
    x, out = empty((too_many, columns)), empty((too_many, rows))
    with pytest.raises(et.BackendError, match="static scratch holds"):
        qw.linear_static_into(x, too_many, out)
