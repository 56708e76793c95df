"""The sampler oracle: pinned arithmetic against the plain restatement."""
import numpy as np

from oracle import sampling_oracle as so


def test_pinned_exp_and_log_are_accurate():
    rng = np.random.default_rng(0)
    x = -np.abs(rng.standard_normal(20000).astype(np.float32)) * 20
    ref = np.exp(x.astype(np.float64))
    ok = ref > 1e-37
    assert np.max(np.abs(so.exp_f32(x)[ok] - ref[ok]) / ref[ok]) < 2e-7
    assert np.all(so.exp_f32(np.array([-88.0, -1e10], np.float32)) == 0)
    u = rng.random(20000, dtype=np.float32).clip(so.TINY, None)
    assert np.max(np.abs(so.log_f32(u) - np.log(u.astype(np.float64)))) < 1e-6


def test_filter_of_the_reference_example_row():
    """The only fixed input the reference holds (sampling.py:49).  With top_p 0.9 the
    three lowest logits (-3, -2, -1) fall outside the nucleus."""
    row = np.array([[-2, -1, 0, 0.8, 0, 0.1, 0.3, 0.4, 0.5, 0.6, 0.7, -3]], np.float32)
    want = row.copy()
    want[0, [0, 1, 11]] -= np.float32(1e10)
    assert np.array_equal(so.nucleaus_filter_plain(row), want)
    assert np.array_equal(so.nucleaus_filter(row)[0], want)


def test_blocked_cumsum_matches_sequential_within_rounding():
    v = np.random.default_rng(2).random(50400, dtype=np.float32)
    v /= v.sum()
    cum, tot = so.blocked_cumsum(v)
    assert np.max(np.abs(cum - np.cumsum(v.astype(np.float64)))) < 1e-5
    assert abs(tot - 1.0) < 1e-5 and np.all(np.diff(cum) >= -1e-6)


def test_pinned_sampler_agrees_with_plain_sampler():
    rng = np.random.default_rng(3)
    for i in range(24):
        v = [512, 50400][i % 2]
        lg = (rng.standard_normal((2, v)) * rng.choice([0.5, 2.0, 6.0])).astype(np.float32)
        un = rng.random((2, v), dtype=np.float32).clip(so.TINY, None)
        a = so.nucleaus_sample(un, lg, 0.9, 0.8)
        b = so.nucleaus_sample_plain(un, lg, 0.9, 0.8)
        assert np.array_equal(a, b)


def test_top_p_zero_is_argmax_with_highest_index_on_ties():
    lg = np.zeros((1, 64), np.float32)
    lg[0, [5, 9, 40]] = 3.0
    un = np.random.default_rng(4).random((1, 64), dtype=np.float32).clip(so.TINY, None)
    assert so.nucleaus_sample(un, lg, 0.0, 1.0)[0] == 40
    assert so.nucleaus_sample_plain(un, lg, 0.0, 1.0)[0] == 40
    from oracle.gptj_oracle import greedy_sampler
    assert greedy_sampler(None, lg, None)[0][0] == 40
