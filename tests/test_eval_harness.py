"""lm-eval adaptor arithmetic: the host module against the restated reference rules."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "mesh-transformer-jax_b200"))

from oracle import eval_harness_oracle as eo  # noqa: E402
from oracle import gptj_oracle as go  # noqa: E402
from oracle import spec  # noqa: E402
from tasks import eval_harness as eh  # noqa: E402
from tasks import util as tu  # noqa: E402


def _requests(n, rng, seq):
    out = []
    for _ in range(n):
        nc, nk = int(rng.integers(1, 2 * seq)), int(rng.integers(1, 9))
        out.append((rng.integers(0, 512, nc).tolist(), rng.integers(0, 512, nk).tolist()))
    return out


@pytest.mark.parametrize("seq", [16, 64])
def test_request_to_sample(seq):
    rng = np.random.default_rng(seq)
    for ctx, cont in _requests(50, rng, seq) + [([1], [2]), (list(range(seq)), [7, 8])]:
        a, b = eh.process_tokens(ctx, cont, seq), eo.process_tokens(ctx, cont, seq)
        for k in ("obs", "target", "eval_mask"):
            assert np.array_equal(a[k], b[k]), k
        assert a["ctx_length"] == b["ctx_length"] == seq
        assert a["eval_mask"].sum() == min(len(cont), seq - 1, len(ctx) + len(cont) - 1)


def test_grouper_and_batches():
    assert list(tu.grouper(3, "ABCDEFG", "x")) == [tuple("ABC"), tuple("DEF"), tuple("Gxx")]
    rng = np.random.default_rng(1)
    samples = [eh.process_tokens(c, k, 32) for c, k in _requests(7, rng, 32)]
    mine, ref = list(tu.sample_batch(iter(samples), 3, samples[0])), list(eo.sample_batch(iter(samples), 3, samples[0]))
    assert len(mine) == len(ref) == 3
    for a, b in zip(mine, ref):
        for k in a:
            assert np.array_equal(a[k], b[k]), k
    assert mine[-1]["ctx_length"].tolist() == [32, 0, 0] and not mine[-1]["eval_mask"][1:].any()


@pytest.mark.parametrize("min_seq", [None, 8, 32])
def test_shrink_seq(min_seq):
    rng = np.random.default_rng(2)
    for trial in range(30):
        seq = 64
        reqs = [(rng.integers(0, 512, int(rng.integers(1, 40 if trial % 2 else 8))).tolist(), [3, 4])
                for _ in range(4)]
        samples = [eh.process_tokens(c, k, seq) for c, k in reqs]
        batch = next(tu.sample_batch(iter(samples), 4, samples[0]))
        want = eo.shrink_seq({k: v.copy() for k, v in batch.items()}, min_seq)
        got = tu.shrink_seq({k: v.copy() for k, v in batch.items()}, min_seq)
        for k in ("obs", "target", "eval_mask"):
            assert np.array_equal(got[k], want[k]), (trial, k)


def test_aggregation():
    rng = np.random.default_rng(3)
    B, T = 6, 20
    out = {"correct": rng.random((B, T)) < 0.7, "all_loss": rng.random((B, T)).astype(np.float32),
           "last_loss": rng.random(B).astype(np.float32)}
    mask = rng.random((B, T)) < 0.3
    mask[0] = False
    out["correct"][1] = True
    a, b = eh.aggregate_eval(out, mask), eo.aggregate(out, mask)
    for k in ("total", "correct", "last_correct"):
        assert a[k] == b[k], k
    assert np.isclose(a["last_loss"], b["last_loss"])
    assert np.allclose(a["mask_loss"], b["mask_loss"]) and np.array_equal(a["each_correct"], b["each_correct"])
    assert not a["each_correct"][0] and a["each_correct"][1] == bool(mask[1].any())


def test_adaptor_scores_continuations_with_the_oracle_network():
    cfg = spec.tiny_config(1, seq=64)
    net = go.CausalTransformer(cfg, spec.make_params(cfg, seed=2))
    rng = np.random.default_rng(4)
    reqs = _requests(5, rng, 20)
    ad = eh.EvalHarnessAdaptor(net, seq=64, batch=2, shrink=True, min_seq=16)
    res = ad.loglikelihood(reqs)
    assert len(res) == 5 and all(isinstance(r[0], float) and isinstance(r[1], bool) for r in res)
    # one request on its own, no shrinking: the same log-likelihood
    solo = eh.EvalHarnessAdaptor(net, seq=64, batch=1, shrink=False).loglikelihood(reqs[2:3])
    assert np.isclose(solo[0][0], res[2][0], rtol=1e-4, atol=1e-4) and solo[0][1] == res[2][1]
    with pytest.raises(Exception):
        ad.greedy_until([])
    with pytest.raises(ValueError):
        ad.loglikelihood([("text", "needs a tokenizer")])
