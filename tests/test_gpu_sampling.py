"""GPU parity of the sampling kernel: token ids bit-exact against the oracle
given identical logits and uniforms."""
import numpy as np
import pytest

from oracle import gptj_oracle as go
from oracle import sampling_oracle as so
from oracle import spec

pytestmark = pytest.mark.gpu


def _sample_gpu(cuda_device, logits, uniforms, top_p, temp):
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.sampling import nucleaus_sample
    toks, info = nucleaus_sample(torch.from_numpy(uniforms).to(cuda_device), torch.from_numpy(logits).to(cuda_device),
                                 None, top_p=top_p, temp=temp)
    assert info is None and toks.dtype == np.uint32
    return toks


@pytest.mark.parametrize("vocab,scale", [(50400, 0.5), (50400, 3.0), (50400, 8.0), (512, 1.0), (12, 1.0), (65535, 2.0)])
def test_sampler_bit_exact_against_oracle(cuda_device, vocab, scale):
    rng = np.random.default_rng(vocab + int(scale * 10))
    rows = 6
    lg = (rng.standard_normal((rows, vocab)) * scale).astype(np.float32)
    un = rng.random((rows, vocab), dtype=np.float32).clip(so.TINY, None)
    top_p = np.array([0.9, 0.5, 0.0, 1.0, 0.999, 0.05], np.float32)
    temp = np.array([1.0, 0.75, 1.0, 1.3, 0.2, 2.0], np.float32)
    got = _sample_gpu(cuda_device, lg, un, top_p, temp)
    want = so.nucleaus_sample(un, lg, top_p, temp)
    assert np.array_equal(got, want)


def test_sampler_tie_order_and_signed_zero(cuda_device):
    vocab = 2048
    rng = np.random.default_rng(9)
    lg = rng.integers(-3, 4, size=(4, vocab)).astype(np.float32)        # heavy ties
    lg[0, ::7] = -0.0
    un = rng.random((4, vocab), dtype=np.float32).clip(so.TINY, None)
    for top_p in (0.0, 0.3, 0.9):
        got = _sample_gpu(cuda_device, lg, un, np.full(4, top_p, np.float32), np.ones(4, np.float32))
        assert np.array_equal(got, so.nucleaus_sample(un, lg, top_p, 1.0))
    # top_p -> 0 is the arg-max with the highest index among equal logits
    top = _sample_gpu(cuda_device, lg, un, np.zeros(4, np.float32), np.ones(4, np.float32))
    for r in range(4):
        assert top[r] == np.flatnonzero(lg[r] == lg[r].max())[-1]


def test_softmax_sample_is_unfiltered(cuda_device):
    import torch
    from mesh_transformer.sampling import softmax_sample
    rng = np.random.default_rng(10)
    lg = rng.standard_normal((3, 512)).astype(np.float32)
    un = rng.random((3, 512), dtype=np.float32).clip(so.TINY, None)
    got, _ = softmax_sample(torch.from_numpy(un).to(cuda_device), torch.from_numpy(lg).to(cuda_device), None, temp=0.9)
    score = (lg / np.float32(0.9)).astype(np.float32) + so.gumbel(un)
    assert np.array_equal(got, np.argmax(score, -1).astype(np.uint32))


def test_sampled_generate_follows_the_oracle_sampler(cuda_device):
    """End to end: at every step the token the device sampled equals the oracle
    sampler applied to the logits the device produced and the same uniforms."""
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.sampling import nucleaus_sample
    from mesh_transformer.transformer_shard import CausalTransformer
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=8, stress=True)
    net = CausalTransformer(dict(cfg, sampler=nucleaus_sample), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    lens = np.array([40, 17], np.uint32)
    ctx = np.zeros((2, 64), np.uint32)
    for b in range(2):
        ctx[b, 64 - lens[b]:] = spec.token_ids(20 + b, 1, int(lens[b]), 512)[0]
    steps = 24
    un = np.random.default_rng(11).random((steps, 2, 512), dtype=np.float32).clip(so.TINY, None)
    opts = {"top_p": np.array([0.9, 0.6]), "temp": np.array([1.0, 0.8])}
    _, out = net.generate(ctx, lens, steps, opts, return_logits=True, uniforms=un)
    toks, logits = out[0], out[2]
    for t in range(steps):
        want = so.nucleaus_sample(un[t], logits[:, t, 0], opts["top_p"].astype(np.float32),
                                  opts["temp"].astype(np.float32))
        assert np.array_equal(toks[:, t, 0], want)
    # and the logits themselves track the oracle model driven by the same tokens
    ref = go.CausalTransformerShard(cfg, params)
    for b in range(2):
        _, (nxt, state) = ref.generate_initial(ctx[b], lens[b])
        for t in range(steps):
            lg, state = ref.generate_once(nxt, state)
            assert np.abs(lg[0] - logits[b, t, 0]).max() / np.abs(lg).max() <= 2e-2
            nxt = toks[b, t]
    # a seeded run without explicit uniforms is reproducible
    import random
    random.seed(5)
    a = net.generate(ctx, lens, 6, opts)[1][0]
    random.seed(5)
    b2 = net.generate(ctx, lens, 6, opts)[1][0]
    assert np.array_equal(a, b2)


def test_sampler_edge_thresholds_and_large_vocab(cuda_device):
    """top_p at and beyond its range, a vocabulary above 65535, and a row dominated by one logit."""
    vocab = 70001
    rng = np.random.default_rng(21)
    rows = 9
    lg = (rng.standard_normal((rows, vocab)) * 2.0).astype(np.float32)
    lg[3, 123] = 40.0                                           # one entry holds nearly all the weight
    lg[4, :] = 0.25                                             # every logit equal: ranking by index decides
    un = rng.random((rows, vocab), dtype=np.float32).clip(so.TINY, None)
    top_p = np.array([-1.0, 1e-30, 1.0, 0.5, 0.37, 1.5, np.inf, 0.9999999, 2.0 ** -20], np.float32)
    temp = np.array([1.0, 1.0, 0.5, 1.0, 1.0, 3.0, 1.0, 0.1, 1.0], np.float32)
    got = _sample_gpu(cuda_device, lg, un, top_p, temp)
    assert np.array_equal(got, so.nucleaus_sample(un, lg, top_p, temp))


def test_sampler_cut_inside_a_group_of_equal_logits(cuda_device):
    """Quantised logits: the threshold falls inside a run of equal values, so the higher indices of the
    run stay and the lower ones go (descending index order among equals)."""
    vocab = 50400
    rng = np.random.default_rng(22)
    lg = np.round(rng.standard_normal((5, vocab)) * 1.5).astype(np.float32) * 0.5
    un = rng.random((5, vocab), dtype=np.float32).clip(so.TINY, None)
    for top_p in (0.11, 0.5, 0.93):
        tp = np.full(5, top_p, np.float32)
        got = _sample_gpu(cuda_device, lg, un, tp, np.ones(5, np.float32))
        assert np.array_equal(got, so.nucleaus_sample(un, lg, tp, 1.0))
    # the filter itself: the kept set is a prefix of the (value desc, index desc) order
    _, removed = so.nucleaus_filter(lg[:1], 0.5)
    order = np.lexsort((-np.arange(vocab), -lg[0]))
    kept_sorted = ~removed[0][order]
    assert kept_sorted[0] and not np.any(np.diff(kept_sorted.astype(np.int8)) > 0)


@pytest.mark.parametrize("vocab,scale", [(50400, 0.5), (50400, 3.0), (512, 1.0), (12, 1.0)])
def test_nucleaus_filter_returns_the_oracle_filter(cuda_device, vocab, scale):
    """sampling.py:10-38 on its own: logits - 1e10 * removed, equal to the oracle's filter entry by entry."""
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.sampling import nucleaus_filter
    rng = np.random.default_rng(vocab + 77)
    lg = (rng.standard_normal((5, vocab)) * scale).astype(np.float32)
    lg[4] = np.round(lg[4])                                              # ties across the cut
    top_p = np.array([0.9, 0.5, 0.0, 1.0, 0.7], np.float32)
    got = nucleaus_filter(torch.from_numpy(lg).to(cuda_device), top_p).cpu().numpy()
    for r in range(5):
        want, removed = so.nucleaus_filter(lg[r:r + 1], top_p[r])
        assert np.array_equal(got[r], want[0])
        assert removed[0].sum() == (got[r] != lg[r]).sum()
    row = np.array([[-2, -1, 0, 0.8, 0, 0.1, 0.3, 0.4, 0.5, 0.6, 0.7, -3]], np.float32)     # sampling.py:49
    want = row.copy()
    want[0, [0, 1, 11]] -= np.float32(1e10)
    assert np.array_equal(nucleaus_filter(row).cpu().numpy(), want)


def test_generate_scan_with_the_device_generator(cuda_device):
    """generate() without supplied uniforms: one library call runs the whole scan, the uniforms come from the
    counter-based device generator keyed like the reference's PRNG key (transformer_shard.py:327).  Every sampled
    id equals the oracle sampler's on the step's own logits and on the uniforms that generator yields for
    (seed, position); the same key reproduces the tokens, another key does not."""
    import ctypes
    import random
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer._lib import check, lib
    from mesh_transformer.sampling import nucleaus_sample
    from mesh_transformer.transformer_shard import CausalTransformer
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=51, stress=True)
    net = CausalTransformer(dict(cfg, sampler=nucleaus_sample), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    ctx = spec.left_pad(spec.token_ids(3, 3, 20, 512), 64)
    opts = {"top_p": np.array([0.9, 0.5, 1.0]), "temp": np.array([1.0, 0.7, 1.5])}
    random.seed(1234)
    _, out = net.generate(ctx, [20] * 3, 10, opts, return_logits=True)
    seed = net.last_seed
    u = torch.empty((3, 512), dtype=torch.float32, device=cuda_device)
    means = []
    for t in range(10):
        check(lib.mtj_k_rng_uniforms(ctypes.c_uint64(seed), 63 + t, 3, 512, u.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream))
        un = u.cpu().numpy()
        assert un.min() >= so.TINY and un.max() < 1.0
        means.append(un.mean())
        want = so.nucleaus_sample(un, out[2][:, t, 0], opts["top_p"].astype(np.float32), opts["temp"].astype(np.float32))
        assert np.array_equal(out[0][:, t, 0], want), f"step {t}"
    assert abs(np.mean(means) - 0.5) < 0.02
    random.seed(1234)
    again = net.generate(ctx, [20] * 3, 10, opts)[1][0]
    assert np.array_equal(again, out[0])
    other = net.generate(ctx, [20] * 3, 10, opts)[1][0]           # the next key of Python's generator
    assert not np.array_equal(other, out[0])
    net.close()


@pytest.mark.parametrize("vocab,scale", [(50400, 3.0), (512, 1.0), (12, 1.0)])
def test_top_k_branch_matches_the_oracle(cuda_device, vocab, scale):
    """sampling.py:15-26: entries of sorted rank >= top_k lose 1e10 * (their own index); the top-p rule still works
    on the unmasked logits.  Filter output and sampled ids equal the oracle's, for top_k inside a group of equal
    logits, top_k = 1, top_k >= vocab (no entry is masked), top_k <= 0 (every entry but token 0 is)."""
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.sampling import nucleaus_filter, nucleaus_sample
    rng = np.random.default_rng(vocab + 5)
    rows = 7
    lg = (rng.standard_normal((rows, vocab)) * scale).astype(np.float32)
    lg[1] = np.round(lg[1])                                              # rank top_k falls among equal logits
    lg[2] = np.round(lg[2] * 0.5)
    top_k = np.array([min(40, vocab - 1), 5, max(1, vocab // 3), 1, vocab, vocab + 9, 0], np.int32)
    top_p = np.array([0.9, 0.8, 1.0, 0.9, 0.5, 0.95, 0.9], np.float32)
    temp = np.array([1.0, 0.7, 1.3, 1.0, 2.0, 0.9, 1.0], np.float32)
    got = nucleaus_filter(torch.from_numpy(lg).to(cuda_device), top_p, top_k).cpu().numpy()
    for r in range(rows):
        want, _ = so.nucleaus_filter(lg[r:r + 1], top_p[r], top_k[r])
        assert np.array_equal(got[r], want[0]), f"row {r}"
        if r not in (1, 2):                          # (inside a group of equal logits the cut may move by the group)
            plain = so.nucleaus_filter_plain(lg[r:r + 1], top_p[r], top_k[r:r + 1])
            assert (plain[0] != want[0]).sum() <= 16                     # the pinned cut moves a few entries at most
    u = rng.uniform(so.TINY, 1.0, size=(rows, vocab)).astype(np.float32)
    toks, _ = nucleaus_sample(torch.from_numpy(u).to(cuda_device), torch.from_numpy(lg).to(cuda_device), None,
                              top_p=top_p, temp=temp, top_k=top_k)
    assert np.array_equal(toks, so.nucleaus_sample(u, lg, top_p, temp, top_k))
    one = nucleaus_filter(torch.from_numpy(lg[:2]).to(cuda_device), 0.9, 3).cpu().numpy()        # scalar options
    assert np.array_equal(one, so.nucleaus_filter(lg[:2], 0.9, 3)[0])


def test_generate_with_top_k(cuda_device):
    """generate() hands sampler_options["top_k"] to the device sampler: every id equals the oracle sampler's on the
    step's own logits and the supplied uniforms."""
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.sampling import nucleaus_sample
    from mesh_transformer.transformer_shard import CausalTransformer
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=52, stress=True)
    net = CausalTransformer(dict(cfg, sampler=nucleaus_sample), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    ctx = spec.left_pad(spec.token_ids(4, 2, 20, 512), 64)
    rng = np.random.default_rng(9)
    u = rng.uniform(so.TINY, 1.0, size=(6, 2, 512)).astype(np.float32)
    opts = {"top_p": np.array([0.95, 1.0]), "temp": np.array([1.0, 1.2]), "top_k": np.array([4, 50])}
    _, out = net.generate(ctx, [20] * 2, 6, opts, return_logits=True, uniforms=u)
    for t in range(6):
        want = so.nucleaus_sample(u[t], out[2][:, t, 0], opts["top_p"].astype(np.float32),
                                  opts["temp"].astype(np.float32), opts["top_k"])
        assert np.array_equal(out[0][:, t, 0], want), f"step {t}"
    _, no_k = net.generate(ctx, [20] * 2, 6, {"top_p": opts["top_p"], "temp": opts["temp"]}, return_logits=True,
                           uniforms=u)
    assert not np.array_equal(no_k[0], out[0])                           # top_k = 4 changes what is sampled
    net.close()
