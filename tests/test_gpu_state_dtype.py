"""GPU tests of the state / dtype surface of CausalTransformer (reference transformer_shard.py:185,216,
250-253; util.py:87-92) and of re-assigning ``network.state`` on a live runtime."""
import numpy as np
import pytest

from oracle import gptj_oracle as go
from oracle import sampling_oracle as so
from oracle import spec

pytestmark = pytest.mark.gpu

GREEDY = lambda b: {"top_p": np.zeros(b), "temp": np.ones(b)}


def _rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def _net(cfg, params, cuda_device):
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.transformer_shard import CausalTransformer
    net = CausalTransformer(dict(cfg), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    return net


def test_unrounded_fp32_weights_tiny_config(cuda_device):
    """The CPU-runnable configuration as written: fp32 N(0, 0.02) weights that are NOT pre-rounded to bf16.
    The reference's generate uses fp32 params as stored (transformer_shard.py:216); this library packs every
    matrix to bf16 on load (move_xmap's cast).  The oracle runs the unrounded weights in fp32, so the
    difference measured here is the whole cost of that cast: it has to stay inside the path's bars
    (logits 2e-2, mean loss 1e-3); a greedy id may differ from the fp32 run only at a near-tie of the two
    best logits."""
    cfg = spec.tiny_config(1, seq=128)
    params = spec.make_params(cfg, seed=0, stress=False, bf16=False)
    assert params[spec.PREFIX + "layer_0/~/linear"]["w"].dtype == np.float32
    assert not np.array_equal(spec.round_bf16(params[spec.PREFIX + "layer_0/~/linear"]["w"]),
                              params[spec.PREFIX + "layer_0/~/linear"]["w"])
    net = _net(cfg, params, cuda_device)
    ids = spec.token_ids(0, 2, 128, 512)
    lens = np.array([96, 96], np.uint32)
    ctx = spec.left_pad(ids[:, :96], 128)
    _, out = net.generate(ctx, lens, 32, GREEDY(2), return_logits=True)
    _, ref = go.CausalTransformer(cfg, params).generate(ctx, lens, 32, return_logits=True)
    assert _rel(out[2][:, 0], ref[2][:, 0]) <= 2e-2
    same = (out[0] == ref[0])[:, :, 0]
    for b in range(2):
        if same[b].all():
            continue
        t = int(np.argmin(same[b]))                      # first differing step: must be a near-tie in the oracle
        top2 = np.sort(ref[2][b, t, 0])[-2:]
        assert top2[1] - top2[0] <= 2e-2 * np.abs(ref[2][b, t]).max(), "greedy ids differ away from a tie"
        assert _rel(out[2][b, :t + 1], ref[2][b, :t + 1]) <= 2e-2
    sample = {"obs": ids[:, :-1], "target": ids[:, 1:]}
    ev, evr = net.eval(sample), go.CausalTransformer(cfg, params).eval(sample)
    assert np.abs(ev["loss"] - evr["loss"]).max() <= 1e-3
    net.close()


def test_move_xmap_to_bf16_to_f32_round_trip(cuda_device):
    """device_serve.py:132-134: drop opt_state, move_xmap(state) casts fp32 leaves to bf16; the network then
    runs exactly what a network given pre-rounded fp32 weights runs."""
    import torch
    from mesh_transformer.util import to_bf16, to_f32
    cfg = spec.tiny_config(1, seq=64)
    raw = spec.make_params(cfg, seed=4, stress=True, bf16=False)
    net = _net(cfg, raw, cuda_device)
    net.state = {"params": raw, "step": np.array(0), "opt_state": {"junk": np.zeros(3, np.float32)}}
    del net.state["opt_state"]
    net.state = net.move_xmap(net.state, np.zeros(1))
    leaf = net.state["params"][spec.PREFIX + "layer_0/~/linear"]["w"]
    assert isinstance(leaf, torch.Tensor) and leaf.dtype == torch.bfloat16
    assert int(np.asarray(net.state["step"])) == 0                     # non-float leaves are untouched
    back = to_f32(net.state)["params"][spec.PREFIX + "layer_0/~/linear"]["w"]
    assert back.dtype == torch.float32
    assert np.array_equal(back.numpy(), spec.round_bf16(raw[spec.PREFIX + "layer_0/~/linear"]["w"]))
    assert to_bf16(to_f32(net.state))["params"][spec.PREFIX + "layer_0/~/linear"]["w"].dtype == torch.bfloat16
    rounded = {m: {k: spec.round_bf16(v) for k, v in leaves.items()} for m, leaves in raw.items()}
    ctx = spec.left_pad(spec.token_ids(1, 1, 30, 512), 64)
    got = net.generate(ctx, [30], 16, GREEDY(1), return_logits=True)[1]
    _, ref = go.CausalTransformer(cfg, rounded).generate(ctx, [30], 16, return_logits=True)
    assert np.array_equal(got[0], ref[0])
    assert _rel(got[2], ref[2]) <= 2e-2
    net.close()


def test_early_cast_initialises_bf16_params(cuda_device):
    """transformer_shard.py:185: with "early_cast" in the config the initial params are bf16."""
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.transformer_shard import CausalTransformer
    cfg = spec.tiny_config(1, seq=64)
    for early, want in ((False, torch.float32), (True, torch.bfloat16)):
        c = dict(cfg, **({"early_cast": True} if early else {}))
        net = CausalTransformer(c)
        assert all(v.dtype == want for m in net.state["params"].values() for v in m.values())
        ctx = spec.left_pad(spec.token_ids(1, 1, 10, 512), 64)
        toks = net.generate(ctx, [10], 4, GREEDY(1))[1][0]
        assert toks.shape == (1, 4, 1)
        net.close()


def test_state_can_be_reassigned_on_a_live_runtime(cuda_device):
    """Assigning ``network.state`` again after a generate reloads every leaf into the same device runtime
    (device_serve.py:129 followed by a later checkpoint swap)."""
    cfg = spec.tiny_config(1, seq=64)
    pa, pb = spec.make_params(cfg, seed=41, stress=True), spec.make_params(cfg, seed=42, stress=True)
    ctx = spec.left_pad(spec.token_ids(2, 1, 30, 512), 64)
    net = _net(cfg, pa, cuda_device)
    a = net.generate(ctx, [30], 12, GREEDY(1))[1][0]
    rt = net._rt
    net.state = {"params": pb, "step": np.array(0)}
    b = net.generate(ctx, [30], 12, GREEDY(1))[1][0]
    assert net._rt is rt, "the runtime is reused"
    assert np.array_equal(a, go.CausalTransformer(cfg, pa).generate(ctx, [30], 12)[1][0])
    assert np.array_equal(b, go.CausalTransformer(cfg, pb).generate(ctx, [30], 12)[1][0])
    assert not np.array_equal(a, b)
    net.close()


def test_a_missing_leaf_is_reported_even_if_another_is_loaded_twice(cuda_device):
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer._lib import MtjError
    from mesh_transformer._runtime import ShardRuntime
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=43)
    rt = ShardRuntime(cfg, max_batch=1, max_gen=2)
    skipped = spec.PREFIX + "layer_1/~/linear_3"
    for mod, leaves in params.items():
        for leaf, v in leaves.items():
            if mod != skipped:
                rt.load_param(f"{mod}/{leaf}", v[0])
    first = spec.PREFIX + "layer_0/~/linear_3"
    rt.load_param(first + "/w", params[first]["w"][0])                  # a duplicate must not fill the gap
    ctx = torch.zeros((1, 64), dtype=torch.int32, device=cuda_device)
    with pytest.raises(MtjError, match="parameters missing"):
        rt.prefill(ctx, [10])
    rt.load_param(skipped + "/w", params[skipped]["w"][0])
    rt.prefill(ctx, [10])
    rt.close()


def test_sampler_options_default_to_the_reference_defaults(cuda_device):
    """generate(..., {"temp": t}) samples with top_p = 0.9 like nucleaus_sample's signature
    (sampling.py:41), not greedily."""
    from mesh_transformer.sampling import nucleaus_sample
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=44, stress=True)
    net = _net(dict(cfg, sampler=nucleaus_sample), params, cuda_device)
    ctx = spec.left_pad(spec.token_ids(3, 2, 20, 512), 64)
    un = np.random.default_rng(9).random((8, 2, 512), dtype=np.float32).clip(so.TINY, None)
    temp = np.array([1.3, 0.6])
    _, out = net.generate(ctx, [20, 20], 8, {"temp": temp}, return_logits=True, uniforms=un)
    for t in range(8):
        want = so.nucleaus_sample(un[t], out[2][:, t, 0], np.full(2, 0.9, np.float32), temp.astype(np.float32))
        assert np.array_equal(out[0][:, t, 0], want)
    greedy = net.generate(ctx, [20, 20], 8, {"top_p": np.zeros(2), "temp": temp})[1][0]
    assert not np.array_equal(greedy, out[0]), "sampling with top_p 0.9 collapsed to arg-max"
    net.close()


def test_load_ckpt_skips_optimizer_state_leaves(cuda_device, tmp_path):
    """A training checkpoint holds optimizer-state leaves before the params in flatten order; load_ckpt reads
    the params and the step out of it (the reference's callers delete opt_state, device_sample.py:74-79)."""
    from mesh_transformer.checkpoint import write_ckpt
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=45, stress=True)
    path = str(tmp_path) + "/"
    opt = {"count": np.zeros((1,), np.int32), "mu": {"a": np.ones((1, 5), np.float32), "b": np.ones((1, 2, 3), np.float32)}}
    write_ckpt({"opt_state": opt, "params": params, "step": np.array(7)}, path, 0)
    net = _net(cfg, spec.make_params(cfg, seed=46), cuda_device)
    net.load_ckpt(path)
    assert int(np.asarray(net.state["step"]).reshape(-1)[0]) == 7
    ctx = spec.left_pad(spec.token_ids(3, 1, 25, 512), 64)
    got = net.generate(ctx, [25], 8, GREEDY(1))[1][0]
    assert np.array_equal(got, go.CausalTransformer(cfg, params).generate(ctx, [25], 8)[1][0])
    net.close()
