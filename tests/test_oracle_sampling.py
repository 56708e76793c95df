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


def test_batched_kept_counts_are_the_filters_removed_sets():
    rng = np.random.default_rng(11)
    lg = (rng.standard_normal((6, 50400)) * 2.0).astype(np.float32)
    for tp in (0.5, 0.9):
        assert np.array_equal(50400 - so.kept_count(lg, tp), so.nucleaus_filter(lg, tp)[1].sum(-1))
        removed_plain = (so.nucleaus_filter_plain(lg, tp) != lg).sum(-1)
        assert np.array_equal(50400 - so.kept_count_plain(lg, tp), removed_plain)


def test_pinned_cut_against_plain_fp32_and_exact_cuts_over_ten_thousand_rows():
    """Where the nucleus ends (sampling.py:13,29) is decided by an fp32 cumulative sum in the reference;
    its association order belongs to XLA.  Over 10 080 rows of 50 400 logits (three logit scales, three
    top_p) the pinned fixed-point rule is compared with (a) the plain restatement (NumPy's sequential fp32
    cumsum) and (b) the same rule in float64.  The pinned rule must coincide with the float64 cut; the
    fp32 cut may differ from both by a few entries at the boundary, whose total probability is tiny."""
    rng = np.random.default_rng(7)
    rows = mism_plain = mism_exact = 0
    worst_entries, worst_mass = 0, 0.0
    for scale in (0.5, 2.0, 6.0):
        for tp in (0.5, 0.9, 0.99):
            for _ in range(4):
                lg = (rng.standard_normal((280, 50400)) * scale).astype(np.float32)
                plain, pinned = so.kept_count_plain(lg, tp), so.kept_count(lg, tp)
                s = -np.sort(-lg.astype(np.float64), axis=-1)
                e = np.exp(s - s[:, :1])
                cum = np.cumsum(e / e.sum(-1, keepdims=True), axis=-1)
                exact = 1 + np.sum(cum[:, :-1] <= float(np.float32(tp)), axis=-1)
                r = np.arange(len(lg))
                rows += len(lg)
                mism_plain += int((plain != pinned).sum())
                mism_exact += int((exact != pinned).sum())
                worst_entries = max(worst_entries, int(np.abs(plain - pinned).max()))
                worst_mass = max(worst_mass, float(np.abs(cum[r, plain - 1] - cum[r, pinned - 1]).max()))
    print(f"rows {rows}: pinned != plain fp32 on {mism_plain} rows (at most {worst_entries} entries, "
          f"probability mass {worst_mass:.2e}); pinned != float64 on {mism_exact} rows")
    assert rows >= 10000
    assert mism_exact <= rows // 1000
    assert worst_entries <= 32 and worst_mass <= 5e-4


def test_top_k_mask_follows_the_reference_arithmetic():
    """sampling.py:15-26 by hand on the reference's own demo row (:49): with top_k = 3 the entries 0.8, 0.7, 0.6
    (indices 3, 10, 9) stay; every other entry i loses 1e10 * i -- so index 0 loses nothing to this branch --
    and the top-p rule (computed from the unmasked row) then removes indices 0, 1 and 11 as without top_k."""
    row = np.array([[-2, -1, 0, 0.8, 0, 0.1, 0.3, 0.4, 0.5, 0.6, 0.7, -3]], np.float32)
    want = row.copy()
    for i in (1, 2, 4, 5, 6, 7, 8, 11):
        want[0, i] = np.float32(want[0, i] - np.float32(1e10) * np.float32(i))
    for i in (0, 1, 11):
        want[0, i] = np.float32(want[0, i] - np.float32(1e10))
    for f in (lambda r: so.nucleaus_filter(r, 0.9, 3)[0], lambda r: so.nucleaus_filter_plain(r, 0.9, 3)):
        assert np.array_equal(f(row), want)
    # equal logits: the higher index sorts first (argsort()[::-1]), so with top_k = 2 of three equal heads the
    # lowest index of the three is the one beyond the first two
    tie = np.array([[0.0, 1.0, 1.0, 1.0]], np.float32)
    got = so.nucleaus_filter(tie, 1.0, 2)[0]
    assert np.array_equal(got, np.array([[0.0, np.float32(1.0 - 1e10), 1.0, 1.0]], np.float32))   # index 0 loses 0
    assert np.array_equal(so.nucleaus_filter(tie, 1.0, 4)[0], tie)        # top_k >= vocab masks nothing
    u = np.full((1, 4), 0.5, np.float32)
    assert so.nucleaus_sample(u, tie, 1.0, 1.0, 1)[0] == 3                # only the highest index of the tie is left
