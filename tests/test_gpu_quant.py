"""GPU parity for block-quantized weights: dequantise/quantise bit-exact with the oracle, linear and
embedding against the reference's golden vectors and against the oracle on seeded inputs."""
import numpy as np
import pytest
import torch

import effect_torch_b200 as et
import oracle as orc
from tests import helpers
from tests.golden import reference_vectors as gv
from tests.gpu_util import dev, empty, host, runtime

pytestmark = pytest.mark.gpu

ALL_CODECS = [gv.Q4_0, gv.Q8_0, gv.Q2_K, gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K]
SCALE_FIELDS = {gv.Q4_0: [0], gv.Q8_0: [0], gv.Q2_K: [80, 82], gv.Q3_K: [108], gv.Q4_K: [0, 2], gv.Q5_K: [0, 2], gv.Q6_K: [208]}
REL_TOL = 2e-3  # north-star tolerance on f16/f32 linear outputs, as max |err| / max |ref|


def random_packed(codec, rows, columns, seed):
    """Random packed bytes with finite f16 scale fields (every bit pattern of the code bytes is legal)."""
    rng = np.random.default_rng(seed)
    bb, bv = orc.block_bytes(codec), orc.block_values(codec)
    blocks = rows * columns // bv
    raw = rng.integers(0, 256, size=(blocks, bb), dtype=np.uint8)
    for off in SCALE_FIELDS[codec]:
        scale = rng.normal(0, 0.01, size=blocks).astype(np.float16)
        raw[:, off:off + 2] = scale.view(np.uint8).reshape(blocks, 2)
    return raw.reshape(rows, columns // bv * bb)


@pytest.mark.parametrize("codec", [gv.Q2_K, gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_k_quant_fixtures_decode_exactly_on_gpu(codec):
    block, _, _ = gv.K_QUANT_FIXTURES[codec]
    out = empty((1, 256))
    runtime().dequantize_into(codec, dev(block.reshape(1, -1)), 1, 256, out)
    np.testing.assert_array_equal(host(out)[0], gv.fixture_expected(codec))


@pytest.mark.parametrize("codec", ALL_CODECS)
def test_dequantize_is_bit_exact_with_the_oracle(codec):
    rows, columns = 37, 1024
    packed = random_packed(codec, rows, columns, seed=codec)
    out = empty((rows, columns))
    runtime().dequantize_into(codec, dev(packed), rows, columns, out)
    expected = orc.dequantize(codec, packed, rows, columns)
    np.testing.assert_array_equal(host(out).view(np.uint32), expected.view(np.uint32))


@pytest.mark.parametrize("codec", [gv.Q4_0, gv.Q8_0])
def test_quantizer_is_bit_exact_with_the_oracle(codec):
    rng = np.random.default_rng(2)
    w = rng.normal(0, 0.02, size=(64, 512)).astype(np.float32)
    w[0, :32] = 0.0                       # all-zero block
    w[1, :32] = 0.01                      # every magnitude ties
    w[2, :32] = np.linspace(-1, 1, 32)    # extreme at the first element
    w[3, :32] = np.linspace(1, -1, 32)
    packed = empty((64, orc.encoded_row_bytes(codec, 512)), dtype=torch.uint8)
    runtime().quantize_into(codec, dev(w), 64, 512, packed)
    np.testing.assert_array_equal(host(packed), orc.quantize(codec, w))


@pytest.mark.parametrize("case", [gv.linear_prefill_case(), gv.linear_lowered_case()])
def test_quantized_linear_golden_vectors(case):
    x = case["x"]
    out = empty((x.shape[0], case["rows"]))
    bias = None if case["bias"] is None else dev(case["bias"])
    runtime().qlinear_into(case["codec"], dev(x), x.shape[0], case["columns"], dev(case["packed"]), case["rows"], bias, out)
    np.testing.assert_array_equal(host(out), case["expected"])


@pytest.mark.parametrize("codec", ALL_CODECS)
@pytest.mark.parametrize("vectors", [1, 3, 11])
def test_generic_linear_matches_the_oracle(codec, vectors):
    rng = np.random.default_rng(100 + codec)
    rows, columns = 96, 1024
    packed = random_packed(codec, rows, columns, seed=50 + codec)
    x = rng.normal(size=(vectors, columns)).astype(np.float32)
    bias = rng.normal(size=rows).astype(np.float32)
    out = empty((vectors, rows))
    runtime().qlinear_into(codec, dev(x), vectors, columns, dev(packed), rows, dev(bias), out)
    expected = orc.qlinear(codec, x, packed, rows, columns, bias, threads=4)
    assert helpers.rel_err(host(out), expected) <= REL_TOL


def test_linear_rejects_bad_geometry_and_observes_cancellation():
    rt = runtime()
    x, w, out = empty((1, 256)), empty((1, 144), dtype=torch.uint8), empty((1, 1))
    with pytest.raises(et.BackendError, match="logical row width 255 is invalid for Q4_K"):
        rt.qlinear_into(gv.Q4_K, x, 1, 255, w, 1, None, out)
    with pytest.raises(et.BackendError, match="^operation aborted$") as e:
        rt.qlinear_into(gv.Q4_K, x, 1, 256, w, 1, None, out, cancelled=True)
    assert e.value.reason == "cancelled"


@pytest.mark.parametrize("i64", [False, True])
def test_embedding_selected_rows_both_index_types(i64):
    block, _, _ = gv.K_QUANT_FIXTURES[gv.Q5_K]
    packed = np.zeros((3, block.size), dtype=np.uint8)
    packed[1] = block
    idx = dev(np.asarray([1, 1], dtype=np.int64 if i64 else np.uint32))
    out = empty((2, 256))
    runtime().qembedding_into(gv.Q5_K, idx, i64, 2, dev(packed), 3, 256, out)
    got = host(out)
    np.testing.assert_array_equal(got[0], gv.fixture_expected(gv.Q5_K))
    np.testing.assert_array_equal(got[1], gv.fixture_expected(gv.Q5_K))


@pytest.mark.parametrize("index", [-1, 1])
def test_embedding_reports_out_of_range_indexes(index):
    block, _, _ = gv.K_QUANT_FIXTURES[gv.Q2_K]
    out = empty((1, 256))
    runtime().qembedding_into(gv.Q2_K, dev(np.asarray([index], dtype=np.int64)), True, 1, dev(block.reshape(1, -1)), 1, 256, out)
    with pytest.raises(et.BackendError, match=r"outside 0\.\.1") as e:
        runtime().synchronize()
    assert e.value.reason == "execution-failed"
    runtime().synchronize()  # the status word was cleared: the runtime stays usable


@pytest.mark.parametrize("codec", [gv.Q4_0, gv.Q8_0])
def test_tiling_preserves_every_weight(codec):
    """x = identity picks out single weights: the tensor-core tiling must hold the same dequantised values
    (to f16 rounding of scale*code, the operand precision of the MMA path)."""
    rng = np.random.default_rng(7)
    rows, columns = 48, 128
    w = rng.normal(0, 0.02, size=(rows, columns)).astype(np.float32)
    packed = orc.quantize(codec, w)
    deq = orc.dequantize(codec, packed, rows, columns)
    qw = et.QWeight(runtime(), codec, [dev(packed)], [rows], columns)
    eye = dev(np.eye(columns, dtype=np.float32))
    out = empty((columns, rows))
    qw.linear_into(eye, columns, out)
    got = host(out).T
    np.testing.assert_allclose(got, deq, rtol=2.0 ** -10, atol=1e-9)


@pytest.mark.parametrize("codec", [gv.Q4_0, gv.Q8_0])
@pytest.mark.parametrize("rows,columns", [(256, 512), (200, 1024), (1024, 4096)])
@pytest.mark.parametrize("vectors", [1, 5, 8, 9, 16, 32, 40, 64, 100, 300])
def test_tiled_linear_matches_the_oracle(codec, rows, columns, vectors):
    rng = np.random.default_rng(rows + columns + vectors)
    w = rng.normal(0, 0.02, size=(rows, columns)).astype(np.float32)
    packed = orc.quantize(codec, w)
    x = rng.normal(size=(vectors, columns)).astype(np.float32)
    qw = et.QWeight(runtime(), codec, [dev(packed)], [rows], columns)
    out = empty((vectors, rows))
    qw.linear_into(dev(x), vectors, out)
    expected = orc.qlinear(codec, x, packed, rows, columns, threads=8)
    assert helpers.rel_err(host(out), expected) <= REL_TOL


@pytest.mark.parametrize("codec", [gv.Q4_0, gv.Q8_0])
@pytest.mark.parametrize("vectors", [4, 32])
def test_tiled_linear_epilogues(codec, vectors):
    rng = np.random.default_rng(9)
    d, ffn = 512, 384
    gate = rng.normal(0, 0.05, size=(ffn, d)).astype(np.float32)
    up = rng.normal(0, 0.05, size=(ffn, d)).astype(np.float32)
    down = rng.normal(0, 0.05, size=(d, ffn)).astype(np.float32)
    pg, pu, pd = orc.quantize(codec, gate), orc.quantize(codec, up), orc.quantize(codec, down)
    x = rng.normal(size=(vectors, d)).astype(np.float32)
    residual = rng.normal(size=(vectors, d)).astype(np.float32)
    bias = rng.normal(size=d).astype(np.float32)
    rt = runtime()
    # fused gate/up with the SwiGLU epilogue
    qgu = et.QWeight(rt, codec, [dev(pg), dev(pu)], [ffn, ffn], d, interleave8=True)
    act = empty((vectors, ffn))
    qgu.linear_into(dev(x), vectors, act, epilogue=et.EPILOGUE_SWIGLU)
    expected_act = orc.silu_mul(orc.qlinear(codec, x, pg, ffn, d, threads=4), orc.qlinear(codec, x, pu, ffn, d, threads=4))
    assert helpers.rel_err(host(act), expected_act) <= REL_TOL
    # down projection with bias and the residual epilogue
    qd = et.QWeight(rt, codec, [dev(pd)], [d], ffn)
    out = empty((vectors, d))
    qd.linear_into(dev(expected_act), vectors, out, bias=dev(bias), residual=dev(residual), epilogue=et.EPILOGUE_RESIDUAL)
    expected = residual + orc.qlinear(codec, expected_act, pd, d, ffn, bias, threads=4)
    assert helpers.rel_err(host(out), expected) <= REL_TOL
    # concatenated q/k/v parts
    qkv = et.QWeight(rt, codec, [dev(pg), dev(pu)], [ffn, ffn], d)
    both = empty((vectors, 2 * ffn))
    qkv.linear_into(dev(x), vectors, both)
    expected_both = np.concatenate([orc.qlinear(codec, x, pg, ffn, d, threads=4), orc.qlinear(codec, x, pu, ffn, d, threads=4)], axis=1)
    assert helpers.rel_err(host(both), expected_both) <= REL_TOL


@pytest.mark.parametrize("codec,ffn,d,vectors", [(gv.Q4_0, 9728, 512, 20), (gv.Q4_0, 14336, 1024, 33), (gv.Q8_0, 9600, 256, 32)])
def test_single_split_launch_with_more_tiles_than_sms(codec, ffn, d, vectors):
    """More 128-row tiles than SMs and not a multiple of them (152, 224 and 150 tiles on 148 SMs), one split: the SwiGLU
    epilogue over interleaved gate/up rows and bias + residual over plain rows, each run twice and bit-identical."""
    rng = np.random.default_rng(ffn + d)
    gate = rng.normal(0, 0.05, size=(ffn, d)).astype(np.float32)
    up = rng.normal(0, 0.05, size=(ffn, d)).astype(np.float32)
    pg, pu = orc.quantize(codec, gate), orc.quantize(codec, up)
    x = rng.normal(size=(vectors, d)).astype(np.float32)
    rt = runtime()
    qgu = et.QWeight(rt, codec, [dev(pg), dev(pu)], [ffn, ffn], d, interleave8=True)
    expected_act = orc.silu_mul(orc.qlinear(codec, x, pg, ffn, d, threads=8), orc.qlinear(codec, x, pu, ffn, d, threads=8))
    runs = []
    for _ in range(2):
        act = empty((vectors, ffn))
        qgu.linear_into(dev(x), vectors, act, epilogue=et.EPILOGUE_SWIGLU)
        runs.append(host(act))
        assert helpers.rel_err(runs[-1], expected_act) <= REL_TOL
    np.testing.assert_array_equal(runs[0], runs[1])
    plain = et.QWeight(rt, codec, [dev(pg), dev(pu)], [ffn, ffn], d)
    bias = rng.normal(size=2 * ffn).astype(np.float32)
    residual = rng.normal(size=(vectors, 2 * ffn)).astype(np.float32)
    expected = residual + np.concatenate([orc.qlinear(codec, x, pg, ffn, d, bias[:ffn], threads=8),
                                          orc.qlinear(codec, x, pu, ffn, d, bias[ffn:], threads=8)], axis=1)
    runs = []
    for _ in range(2):
        out = empty((vectors, 2 * ffn))
        plain.linear_into(dev(x), vectors, out, bias=dev(bias), residual=dev(residual), epilogue=et.EPILOGUE_RESIDUAL)
        runs.append(host(out))
        assert helpers.rel_err(runs[-1], expected) <= REL_TOL
    np.testing.assert_array_equal(runs[0], runs[1])


@pytest.mark.parametrize("codec", [gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_k_quant_tiling_preserves_every_weight(codec):
    """The 256-value K-quant blocks are re-cut into 32-value blocks at load (effective scales rounded to f16): x = identity
    picks out single weights, which must equal the reference decode to the f16 precision of the MMA operands."""
    rows, columns = 40, 512
    packed = random_packed(codec, rows, columns, seed=11)
    deq = orc.dequantize(codec, packed, rows, columns)
    qw = et.QWeight(runtime(), codec, [dev(packed)], [rows], columns)
    out = empty((columns, rows))
    qw.linear_into(dev(np.eye(columns, dtype=np.float32)), columns, out)
    scale = np.abs(deq).max()
    np.testing.assert_allclose(host(out).T, deq, rtol=2.0 ** -9, atol=scale * 2.0 ** -10)


@pytest.mark.parametrize("codec", [gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
@pytest.mark.parametrize("rows,columns", [(256, 512), (200, 1024), (1024, 4096)])
@pytest.mark.parametrize("vectors", [1, 8, 17, 32, 64, 300])
def test_k_quant_tiled_linear_matches_the_oracle(codec, rows, columns, vectors):
    rng = np.random.default_rng(rows + columns + vectors)
    packed = random_packed(codec, rows, columns, seed=rows + vectors)
    x = rng.normal(size=(vectors, columns)).astype(np.float32)
    qw = et.QWeight(runtime(), codec, [dev(packed)], [rows], columns)
    out = empty((vectors, rows))
    qw.linear_into(dev(x), vectors, out)
    expected = orc.qlinear(codec, x, packed, rows, columns, threads=8)
    assert helpers.rel_err(host(out), expected) <= REL_TOL


@pytest.mark.parametrize("codec", [gv.Q3_K, gv.Q4_K, gv.Q5_K, gv.Q6_K])
def test_k_quant_fused_gate_up_and_residual_epilogues(codec):
    rng = np.random.default_rng(21)
    d, ffn, vectors = 512, 256, 20
    pg, pu, pd = random_packed(codec, ffn, d, 1), random_packed(codec, ffn, d, 2), random_packed(codec, d, ffn, 3)
    x = rng.normal(size=(vectors, d)).astype(np.float32)
    residual = rng.normal(size=(vectors, d)).astype(np.float32)
    rt = runtime()
    qgu = et.QWeight(rt, codec, [dev(pg), dev(pu)], [ffn, ffn], d, interleave8=True)
    act = empty((vectors, ffn))
    qgu.linear_into(dev(x), vectors, act, epilogue=et.EPILOGUE_SWIGLU)
    expected_act = orc.silu_mul(orc.qlinear(codec, x, pg, ffn, d, threads=4), orc.qlinear(codec, x, pu, ffn, d, threads=4))
    assert helpers.rel_err(host(act), expected_act) <= REL_TOL
    qd = et.QWeight(rt, codec, [dev(pd)], [d], ffn)
    out = empty((vectors, d))
    unit_act = (expected_act / np.abs(expected_act).max()).astype(np.float32)  # random code bytes make huge activations: keep f16 range
    qd.linear_into(dev(unit_act), vectors, out, residual=dev(residual), epilogue=et.EPILOGUE_RESIDUAL)
    expected = residual + orc.qlinear(codec, unit_act, pd, d, ffn, threads=4)
    assert helpers.rel_err(host(out), expected) <= REL_TOL


def test_tiled_weight_rejects_unsupported_geometry():
    rt = runtime()
    raw = empty((16, 18 * 3), dtype=torch.uint8)
    with pytest.raises(et.BackendError, match="multiple of 64"):
        et.QWeight(rt, gv.Q4_0, [raw], [16], 96)
    with pytest.raises(et.BackendError, match="Q4_0, Q8_0, Q3_K, Q4_K, Q5_K and Q6_K"):
        et.QWeight(rt, gv.Q2_K, [empty((16, 84), dtype=torch.uint8)], [16], 256)
    with pytest.raises(et.BackendError, match="multiple of 256"):
        et.QWeight(rt, gv.Q4_K, [raw], [16], 128)
