"""Restatement of the reference's sampler (mesh_transformer/sampling.py:6-44).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the
reference holds no expected output for its sampler (sampling.py:47-50 only
prints the filter of one 12-element row).

Two layers:

* ``nucleaus_filter_plain`` / ``nucleaus_sample_plain`` follow the reference
  line by line with NumPy's own exp/log/cumsum.
* ``nucleaus_filter`` / ``nucleaus_sample`` are the same algorithm with every
  floating-point operation pinned down, so that a GPU kernel can reproduce the
  sampled token ids bit for bit given identical logits and uniforms.  What is
  pinned is exactly what the reference leaves to XLA (jax 0.2.12, not part of
  the reference tree): the exp / log polynomials, and the rounding of the
  softmax denominator and of the cumulative sum.

  - exp and log are fixed polynomials evaluated with individually rounded fp32
    multiplies and adds (no fused multiply-add);
  - the softmax numerators e_i = exp(l_i - max) are turned into fixed-point
    weights q_i = floor(e_i * 2^40); all sums of weights are exact integers
    (they do not depend on the order of addition), and the reference's test
    "cumulative probability of the entries sorted before this one > top_p" is
    evaluated exactly:  sum_{k before j} q_k  >  floor(top_p * sum_k q_k).
    Because the sums are exact, the entries removed are a suffix of the sorted
    order, which a selection on the sort key finds without sorting.

  ``blocked_cumsum`` (a fixed-association fp32 cumulative sum) is kept as a
  checked helper; the pinned filter no longer uses it.

The sort order is the reference's: ``jnp.sort(x)[::-1]`` / ``jnp.argsort(x)[::-1]``
(stable ascending, reversed), i.e. descending by value and, among equal
values, the HIGHER index first; -0.0 and +0.0 compare equal.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
RUNS = 1024
TINY = np.finfo(np.float32).tiny


# ----------------------------------------------------------------------------
# plain restatement
# ----------------------------------------------------------------------------
def _sorted_desc(logits):
    """sampling.py:11-12 for one row."""
    keys = np.where(logits == 0, F32(0), logits).astype(F32)
    order = np.argsort(keys, kind="stable")[::-1]
    return logits[order], order


def top_k_mask(order, top_k):
    """sampling.py:15-26: every token whose rank in the descending order is >= top_k gets the mask
    1e10 * (its own index) -- ``where(range >= top_k, sorted_indices, 0)`` scattered back to token order --
    so token 0 is never masked by this branch.  Returns the fp32 mask [V]."""
    v = order.shape[0]
    idx = np.zeros(v, np.int64)
    idx[order] = np.where(np.arange(v) >= int(top_k), order, 0)
    return (F32(1e10) * idx.astype(F32)).astype(F32)


def nucleaus_filter_plain(logits, top_p=0.9, top_k=None):
    """sampling.py:10-38; logits [rows, V] float32.  The cumulative probabilities come from the unmasked logits
    also when top_k is given (:13 precedes :15)."""
    logits = np.asarray(logits, F32)
    out = logits.copy()
    for r in range(logits.shape[0]):
        s, order = _sorted_desc(logits[r])
        e = np.exp(s - s.max())
        cum = np.cumsum(e / e.sum(dtype=F32), dtype=F32)
        remove_sorted = cum > F32(top_p)
        remove_sorted = np.concatenate(([False], remove_sorted))[:-1]
        remove = np.zeros(logits.shape[1], bool)
        remove[order] = remove_sorted                      # sort_key_val(sorted_indices, ...) scatters back
        row = logits[r]
        if top_k is not None:
            row = (row - top_k_mask(order, np.asarray(top_k).reshape(-1)[r % np.asarray(top_k).size])).astype(F32)
        out[r] = row - F32(1e10) * remove
    return out


def gumbel_plain(u):
    return -np.log(-np.log(np.asarray(u, F32)))


def nucleaus_sample_plain(uniforms, logits, top_p=0.9, temp=1.0, top_k=None):
    """sampling.py:41-44 + :6-7; categorical = argmax(logits/temp + Gumbel)."""
    filt = nucleaus_filter_plain(logits, top_p, top_k)
    score = (filt / F32(temp)).astype(F32) + gumbel_plain(uniforms)
    return np.argmax(score, axis=-1).astype(np.uint32)


# ----------------------------------------------------------------------------
# pinned arithmetic
# ----------------------------------------------------------------------------
_LOG2E = F32(1.4426950408889634)
_LN2_HI = F32(0.693145751953125)          # 0x3f317200: few mantissa bits, n * LN2_HI is exact
_LN2_LO = F32(1.42860682030941723212e-6)
_EXP_C = [F32(c) for c in (1.9875691500e-4, 1.3981999507e-3, 8.3334519073e-3,
                           4.1665795894e-2, 1.6666665459e-1, 5.0000001201e-1)]


def exp_f32(x):
    """exp for x <= 0, fp32, every multiply/add rounded on its own; 0 below -87."""
    x = np.asarray(x, F32)
    xs = np.maximum(x, F32(-87.0))
    n = np.rint(xs * _LOG2E).astype(F32)
    r = (xs - n * _LN2_HI).astype(F32)
    r = (r - n * _LN2_LO).astype(F32)
    p = _EXP_C[0]
    for c in _EXP_C[1:]:
        p = (p * r).astype(F32) + c
    r2 = (r * r).astype(F32)
    y = ((p * r2).astype(F32) + r).astype(F32) + F32(1.0)
    scale = ((n.astype(np.int32) + 127) << 23).astype(np.int32).view(F32)
    out = (y * scale).astype(F32)
    return np.where(x < F32(-87.0), F32(0.0), out).astype(F32)


_SQRT_HALF = F32(0.70710678118654752440)
_LOG_C = [F32(c) for c in (7.0376836292e-2, -1.1514610310e-1, 1.1676998740e-1, -1.2420140846e-1,
                           1.4249322787e-1, -1.6668057665e-1, 2.0000714765e-1, -2.4999993993e-1,
                           3.3333331174e-1)]


def log_f32(x):
    """Natural log for positive normal fp32, individually rounded operations."""
    x = np.asarray(x, F32)
    bits = x.view(np.int32)
    e = ((bits >> 23) & 0xFF).astype(np.int32) - 126
    m = ((bits & 0x007FFFFF) | 0x3F000000).view(F32)        # mantissa scaled into [0.5, 1)
    small = m < _SQRT_HALF
    e = np.where(small, e - 1, e).astype(F32)
    f = np.where(small, (m + m).astype(F32), m).astype(F32) - F32(1.0)
    z = (f * f).astype(F32)
    p = _LOG_C[0]
    for c in _LOG_C[1:]:
        p = (p * f).astype(F32) + c
    y = ((p * f).astype(F32) * z).astype(F32)
    y = (y + (e * F32(-2.12194440e-4)).astype(F32)).astype(F32)
    y = (y - (F32(0.5) * z).astype(F32)).astype(F32)
    return ((f + y).astype(F32) + (e * F32(0.693359375)).astype(F32)).astype(F32)


def _hillis_steele(x):
    """Inclusive scan along the last axis (length 32), x[i] += x[i - off] for off = 1, 2, 4, 8, 16."""
    x = x.astype(F32).copy()
    for off in (1, 2, 4, 8, 16):
        y = x.copy()
        y[..., off:] = (x[..., off:] + x[..., :-off]).astype(F32)
        x = y
    return x


def blocked_cumsum(v):
    """Cumulative sum and total of a 1-D fp32 array in the pinned association order."""
    v = np.asarray(v, F32)
    n = v.shape[0]
    per = -(-n // RUNS)
    pad = np.zeros(RUNS * per, F32)
    pad[:n] = v
    runs = pad.reshape(RUNS, per)
    local = np.zeros_like(runs)
    acc = np.zeros(RUNS, F32)
    for j in range(per):                                    # sequential inside each run
        acc = (acc + runs[:, j]).astype(F32)
        local[:, j] = acc
    tot = local[:, -1].reshape(32, 32)                      # [group, lane]
    inc = _hillis_steele(tot)
    exc = np.concatenate([np.zeros((32, 1), F32), inc[:, :-1]], axis=1)
    ginc = _hillis_steele(inc[:, -1][None, :])[0]            # scan of the 32 group totals
    gexc = np.concatenate([[F32(0)], ginc[:-1]]).astype(F32)
    prefix = (gexc[:, None] + exc).astype(F32).reshape(RUNS)
    cum = np.zeros_like(runs)
    acc = prefix.copy()
    for j in range(per):
        acc = (acc + runs[:, j]).astype(F32)
        cum[:, j] = acc
    return cum.reshape(-1)[:n], F32(ginc[-1])


WEIGHT_BITS = 40


def fixed_point_weights(e):
    """q = floor(e * 2^40) as uint64 for fp32 e in [0, 1] (exact: a power-of-two scaling, then truncation)."""
    return np.floor(np.asarray(e, F32).astype(np.float64) * 2.0 ** WEIGHT_BITS).astype(np.uint64)


def weight_threshold(top_p, total):
    """floor(top_p * total) for the exact value of the fp32 ``top_p`` and the integer ``total``;
    negative top_p counts as 0; None means "nothing can exceed it" (top_p is NaN)."""
    from fractions import Fraction
    tp = float(F32(top_p))
    if np.isnan(tp):
        return None
    if np.isinf(tp):
        return None if tp > 0 else 0
    if tp <= 0:
        return 0
    fr = Fraction(tp) * int(total)
    return fr.numerator // fr.denominator


def nucleaus_filter(logits, top_p=0.9, top_k=None):
    """sampling.py:10-38 with pinned arithmetic; returns (filtered, removed by the top-p rule).  ``top_k`` (None,
    a scalar or one value per row) adds the reference's top-k mask, which needs no arithmetic to be pinned."""
    logits = np.asarray(logits, F32)
    out = logits.copy()
    removed = np.zeros(logits.shape, bool)
    for r in range(logits.shape[0]):
        s, order = _sorted_desc(logits[r])
        q = fixed_point_weights(exp_f32((s - s[0]).astype(F32)))
        before = np.cumsum(q, dtype=np.uint64) - q           # weight sorted before each entry (< 2^56: exact)
        thr = weight_threshold(top_p, int(q.sum(dtype=np.uint64)))
        if thr is None or thr >= 2 ** 63:
            remove_sorted = np.zeros(q.shape, bool)
        else:
            remove_sorted = before > np.uint64(thr)          # the head (before == 0) always stays
        removed[r, order] = remove_sorted
        row = logits[r]
        if top_k is not None:
            row = (row - top_k_mask(order, np.asarray(top_k).reshape(-1)[r % np.asarray(top_k).size])).astype(F32)
        out[r] = (row - F32(1e10) * removed[r].astype(F32)).astype(F32)
    return out, removed


def gumbel(u):
    """-log(-log(u)) as jax.random.gumbel does, u in [tiny, 1)."""
    t = (-log_f32(u)).astype(F32)
    return (-log_f32(t)).astype(F32)


def nucleaus_sample(uniforms, logits, top_p=0.9, temp=1.0, top_k=None):
    """Token ids [rows] uint32: argmax(filtered / temp + Gumbel(uniforms)), first index on ties."""
    logits = np.asarray(logits, F32)
    uniforms = np.asarray(uniforms, F32)
    top_p = np.broadcast_to(np.asarray(top_p, F32), (logits.shape[0],))
    temp = np.broadcast_to(np.asarray(temp, F32), (logits.shape[0],))
    toks = np.zeros(logits.shape[0], np.uint32)
    for r in range(logits.shape[0]):
        k_r = None if top_k is None else np.asarray(top_k).reshape(-1)[r % np.asarray(top_k).size]
        filt, _ = nucleaus_filter(logits[r:r + 1], top_p[r], k_r)
        score = ((filt[0] / temp[r]).astype(F32) + gumbel(uniforms[r])).astype(F32)
        toks[r] = np.argmax(score)
    return toks


def nucleus_sampler(uniforms_row, logits, _aux, top_p=0.9, temp=1.0):
    """Adapter with the reference's sampler signature (key, logits, aux, **opts)
    where the "key" is the row of pre-drawn uniforms for this step."""
    tok = nucleaus_sample(np.asarray(uniforms_row, F32)[None, :], logits, top_p, temp)
    return tok, None


# ----------------------------------------------------------------------------
# batched "how many sorted entries stay" for both definitions (the removed entries are a suffix of
# the sorted order under either, so the count fixes the removed set)
# ----------------------------------------------------------------------------
def kept_count_plain(logits, top_p=0.9):
    """Entries kept per row by ``nucleaus_filter_plain`` (rows, V) -> int64 [rows]."""
    s = -np.sort(-np.asarray(logits, F32), axis=-1)
    e = np.exp(s - s[:, :1])
    cum = np.cumsum(e / e.sum(axis=-1, keepdims=True, dtype=F32), axis=-1, dtype=F32)
    return 1 + np.sum(cum[:, :-1] <= F32(top_p), axis=-1)   # entry j stays iff cum[j-1] <= top_p (cum is monotone)


def kept_count(logits, top_p=0.9):
    """Entries kept per row by the pinned ``nucleaus_filter``."""
    s = -np.sort(-np.asarray(logits, F32), axis=-1)
    q = fixed_point_weights(exp_f32((s - s[:, :1]).astype(F32)))
    before = np.cumsum(q, axis=-1, dtype=np.uint64) - q
    out = np.zeros(s.shape[0], np.int64)
    for r in range(s.shape[0]):
        thr = weight_threshold(top_p, int(q[r].sum(dtype=np.uint64)))
        out[r] = s.shape[1] if (thr is None or thr >= 2 ** 63) else int(np.sum(before[r] <= np.uint64(thr)))
    return out
