"""GPU parity for the dense / elementwise ops of the decode graph against the CPU oracle."""
import numpy as np
import pytest
import torch

import effect_torch_b200 as et
import oracle as orc
from tests.golden import reference_vectors as gv
from tests.gpu_util import dev, empty, host, runtime

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,k,n", [(1, 256, 256), (4, 688, 256), (4, 256, 4096), (9, 37, 65)])
def test_dense_linear_is_bit_exact(m, k, n):
    # every output is one sequential fma chain over k, like crates/runtime-cpu/src/matmul.rs:209-230
    rng = np.random.default_rng(m * 1000 + k + n)
    x = rng.normal(size=(m, k)).astype(np.float32)
    w = rng.normal(0, 0.02, size=(n, k)).astype(np.float32)
    out = empty((m, n))
    runtime().linear_f32_into(dev(x), m, k, dev(w), n, None, out)
    np.testing.assert_array_equal(host(out), orc.linear_rows(x, w, threads=4))


@pytest.mark.parametrize("n", [256, 4096, 1000])
def test_rmsnorm_matches_the_oracle(n):
    rng = np.random.default_rng(n)
    x = rng.normal(size=(5, n)).astype(np.float32)
    w = rng.normal(1.0, 0.1, size=n).astype(np.float32)
    out = empty((5, n))
    runtime().rmsnorm_into(dev(x), dev(w), 1e-5, 5, n, out)
    # f64 tree reduction vs the reference's sequential f64 sum: identical after rounding to f32 except at
    # exact rounding boundaries
    np.testing.assert_array_max_ulp(host(out), orc.rms_norm(x, w, 1e-5), maxulp=1)
    runtime().rmsnorm_into(dev(x), None, 1e-5, 5, n, out)
    np.testing.assert_array_max_ulp(host(out), orc.rms_norm(x, None, 1e-5), maxulp=1)


@pytest.mark.parametrize("layout", [et.HALF_SPLIT, et.INTERLEAVED_PAIRS])
def test_rope_matches_the_oracle_and_the_golden_vector(layout):
    x, half, inter = gv.rope_case()
    out = empty(x.shape)
    rt = runtime()
    rt.rope_into(dev(x), dev(np.zeros(1, np.int64)), 1, 10000.0, layout, 1, 1, 2, 4, out)
    np.testing.assert_allclose(host(out).reshape(-1), half if layout == et.HALF_SPLIT else inter, rtol=1e-6, atol=1e-6)
    rng = np.random.default_rng(3)
    xb = rng.normal(size=(3, 4, 5, 64)).astype(np.float32)
    offsets = np.asarray([0, 17, 4000], dtype=np.int64)
    outb = empty(xb.shape)
    rt.rope_into(dev(xb), dev(offsets), 3, 500000.0, layout, 3, 4, 5, 64, outb)
    expected = orc.rotary(xb, offsets, 500000.0, layout)
    # f64 sin/cos differ from the host libm by an ulp of f64 at most: equal in f32 up to boundary cases
    np.testing.assert_allclose(host(outb), expected, rtol=3e-7, atol=1e-7)


def test_swiglu_and_add_match_the_oracle():
    rng = np.random.default_rng(4)
    g = rng.normal(0, 3, size=5000).astype(np.float32)
    u = rng.normal(size=5000).astype(np.float32)
    out = empty(5000)
    runtime().swiglu_into(dev(g), dev(u), 5000, out)
    np.testing.assert_allclose(host(out), orc.silu_mul(g, u), rtol=2e-6, atol=1e-7)
    runtime().add_into(dev(g), dev(u), 5000, out)
    np.testing.assert_array_equal(host(out), g + u)


@pytest.mark.parametrize("logits,expected", gv.GREEDY_CASES)
def test_greedy_argmax_prefers_the_lower_token(logits, expected):
    tokens = empty(1, dtype=torch.int32)
    runtime().argmax_into(dev(np.asarray([logits], dtype=np.float32)), 1, len(logits), tokens)
    assert int(host(tokens)[0]) == expected


def test_argmax_large_rows_and_non_finite_logits():
    rng = np.random.default_rng(5)
    logits = rng.normal(size=(4, 128256)).astype(np.float32)
    logits[1, 77] = logits[1].max() + 1
    logits[1, 90000] = logits[1, 77]  # tie: the lower index wins
    tokens = empty(4, dtype=torch.int32)
    rt = runtime()
    rt.argmax_into(dev(logits), 4, 128256, tokens)
    np.testing.assert_array_equal(host(tokens), [orc.argmax(r) for r in logits])
    assert int(host(tokens)[1]) == 77
    logits[2, 5] = np.nan
    rt.argmax_into(dev(logits), 4, 128256, tokens)
    with pytest.raises(et.BackendError, match="sample: logit 5 is not finite"):
        rt.synchronize()


def test_sample_row_replays_the_reference_stream():
    rng = np.random.default_rng(6)
    logits = rng.normal(size=512).astype(np.float32)
    d = dev(logits)
    rt = runtime()
    for kwargs in (dict(temperature=0.0), dict(temperature=1.0, seed=7, counter=3), dict(temperature=0.7, top_k=5, seed=1, counter=9),
                   dict(temperature=1.3, top_p=0.8, seed=1234, counter=0), dict(temperature=1.0, top_k=40, top_p=0.5, seed=3, counter=2)):
        assert rt.sample_row(d, 512, **kwargs) == orc.sample_logits(logits, **kwargs)
    with pytest.raises(et.BackendError, match="topK"):
        rt.sample_row(d, 512, top_k=513)


@pytest.mark.parametrize("vocab", [1, 33, 4096, 128256])
def test_device_sampling_agrees_with_the_reference_rule_on_many_draws(vocab):
    """Every mode of sample_logits over batches of rows with per-row (seed, counter) keys: unfiltered (token-order walk),
    top-k, top-p, both; peaked and flat rows; ties (repeated values must be ordered by token)."""
    rt = runtime()
    rng = np.random.default_rng(vocab)
    rows = 24
    logits = (rng.normal(size=(rows, vocab)) * rng.uniform(0.2, 6.0, size=(rows, 1))).astype(np.float32)
    logits[3] = np.round(logits[3])  # many exact ties
    logits[4] = 0.25                 # one value everywhere: order is by token alone
    d = dev(logits)
    seeds = rng.integers(0, 2**63, size=rows, dtype=np.uint64)
    counters = rng.integers(0, 1000, size=rows, dtype=np.uint64)
    d_seeds, d_counters = dev(seeds), dev(counters)
    tokens = empty(rows, dtype=torch.int32)
    modes = [dict(temperature=1.0), dict(temperature=0.6), dict(temperature=0.0)]
    if vocab > 1:
        k = min(vocab - 1, 50)
        modes += [dict(temperature=0.8, top_k=k), dict(temperature=1.0, top_p=0.9), dict(temperature=1.5, top_p=0.3),
                  dict(temperature=0.9, top_k=k, top_p=0.7), dict(temperature=1.0, top_k=1), dict(temperature=2.0, top_k=vocab)]
    for mode in modes:
        rt.sample_rows_into(d, rows, vocab, tokens, seeds=d_seeds, counters=d_counters, **mode)
        got = host(tokens)
        want = [orc.sample_logits(logits[r], seed=int(seeds[r]), counter=int(counters[r]), **mode) for r in range(rows)]
        np.testing.assert_array_equal(got, want, err_msg=str(mode))


def test_device_sampling_reports_bad_arguments_and_non_finite_logits_like_the_reference():
    rt = runtime()
    logits = np.zeros((2, 64), dtype=np.float32)
    d, tokens = dev(logits), empty(2, dtype=torch.int32)
    for kwargs, message in ((dict(temperature=-1.0), "temperature must be finite and non-negative"), (dict(top_p=0.0), "topP"),
                            (dict(top_p=1.5), "topP"), (dict(top_k=65), "topK"), (dict(temperature=float("nan")), "temperature")):
        with pytest.raises(et.BackendError, match=message):
            rt.sample_rows_into(d, 2, 64, tokens, **kwargs)
    logits[1, 9] = np.inf
    rt.sample_rows_into(dev(logits), 2, 64, tokens, temperature=1.0, top_p=0.9)
    with pytest.raises(et.BackendError, match="sample: logit 9 is not finite"):
        rt.synchronize()
