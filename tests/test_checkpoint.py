"""v1 checkpoint format and re-sharding: the host module against the restated reference rules."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "mesh-transformer-jax_b200"))

from oracle import checkpoint_oracle as co  # noqa: E402
from oracle import spec  # noqa: E402


def _ckpt():
    # importing the package needs the built library (no fallback); the checkpoint module itself is host-only
    import importlib.util
    path = os.path.join(ROOT, "mesh-transformer-jax_b200", "mesh_transformer", "checkpoint.py")
    s = importlib.util.spec_from_file_location("mtj_checkpoint_under_test", path)
    m = importlib.util.module_from_spec(s)
    s.loader.exec_module(m)
    return m


def _state(mp, seed=3, trained_ln=True):
    cfg = dict(spec.tiny_config(), cores_per_replica=mp)
    fw = spec.full_weights(cfg, seed=seed)
    if trained_ln:
        rng = np.random.default_rng(7)
        for lw in fw["layers"]:
            lw["ln_scale"] = (1 + 0.1 * rng.standard_normal(lw["ln_scale"].shape)).astype(np.float32)
            lw["ln_offset"] = (0.1 * rng.standard_normal(lw["ln_offset"].shape)).astype(np.float32)
            lw["ff_out_b"] = (0.1 * rng.standard_normal(lw["ff_out_b"].shape)).astype(np.float32)
            lw["ff_in_b"] = (0.1 * rng.standard_normal(lw["ff_in_b"].shape)).astype(np.float32)
        fw["embed_b"] = (0.1 * rng.standard_normal(fw["embed_b"].shape)).astype(np.float32)
        fw["proj_b"] = (0.1 * rng.standard_normal(fw["proj_b"].shape)).astype(np.float32)
    return cfg, {"params": spec.shard_params(cfg, fw), "step": np.full((mp,), 11, np.int32), "opt_state": None}


@pytest.mark.parametrize("n", [0, 1, 15, 16, 17, 26, 33, 100])
def test_split_rule(n):
    ck = _ckpt()
    a = list(range(n))
    assert ck.split(a, 16) == co.split(a, 16)
    assert sum(len(c) for c in ck.split(a, 16)) == n


def test_flatten_order_is_sorted_keys_and_skips_none():
    ck = _ckpt()
    _, st = _state(2)
    assert [id(x) for _, x in ck.tree_flatten(st)] == [id(x) for x in co.tree_flatten(st)]
    paths = [p for p, _ in ck.tree_flatten(st)]
    assert paths[-1] == ("step",) and all(p[0] == "params" for p in paths[:-1])


def test_files_are_interchangeable_with_the_reference_layout(tmp_path):
    ck = _ckpt()
    _, st = _state(2)
    d1, d2 = str(tmp_path / "a") + "/", str(tmp_path / "b") + "/"
    for s in range(2):
        ck.write_ckpt(st, d1, s)
        co.write_ckpt(st, d2, s)
    for s in range(2):
        mine, ref = co.read_shard(f"{d1}shard_{s}"), ck.read_shard(f"{d2}shard_{s}/")
        assert len(mine) == len(ref) == len(co.tree_flatten(st))
        for a, b, leaf in zip(mine, ref, co.tree_flatten(st)):
            assert np.array_equal(a, b) and np.array_equal(a, np.asarray(leaf)[s])
        assert sorted(os.listdir(f"{d1}shard_{s}")) == sorted(f"{i}.npz" for i in range(16))


def test_bfloat16_leaves_round_trip_as_two_byte_void(tmp_path):
    ck = _ckpt()
    t = torch.randn((2, 5, 8)).to(torch.bfloat16)
    st = {"params": {"m": {"w": t}}, "step": np.zeros((2,), np.int32), "opt_state": None}
    d = str(tmp_path) + "/"
    for s in range(2):
        ck.write_ckpt(st, d, s)
    raw = co.read_shard(f"{d}shard_1")
    assert raw[0].dtype == np.dtype("V2") and raw[0].shape == (5, 8)
    back = ck.read_ckpt(st, d, 2)
    assert back["params"]["m"]["w"].dtype == torch.bfloat16
    assert torch.equal(back["params"]["m"]["w"], t)
    assert back["opt_state"] is None


def test_reshard_heuristic_matches_the_reference_rules():
    ck = _ckpt()
    cfg4, st4 = _state(4)
    cfg1, st1 = _state(1)
    for (path, x), (_, old) in zip(ck.tree_flatten(st4), ck.tree_flatten(st1)):
        want = co.reshard(np.asarray(x), np.asarray(old).shape)
        got = ck.reshard(np.asarray(x), np.asarray(old).shape).numpy()
        assert got.shape == want.shape and np.allclose(got, want, rtol=0, atol=0), path
    # the heuristic is exact for weights, column-parallel biases and untouched LayerNorms ...
    p4, p1 = st4["params"], st1["params"]
    for mod in p4:
        for leaf in p4[mod]:
            got = ck.reshard(p4[mod][leaf], p1[mod][leaf].shape).numpy()
            role = ck.parameter_role(mod, leaf)
            if role in ("column", "row"):
                assert np.array_equal(got, p1[mod][leaf]), (mod, leaf)
    # ... and scales a trained LayerNorm like a bias every shard adds (reference behaviour, checkpoint.py:108-110)
    ln = next(m for m in p4 if m.endswith("layer_0/~/replicated_layer_norm"))
    assert np.allclose(ck.reshard(p4[ln]["scale"], p1[ln]["scale"].shape).numpy(), 4 * p1[ln]["scale"])


@pytest.mark.parametrize("n_in,n_out", [(8, 1), (8, 2), (4, 2), (2, 1), (4, 4)])
def test_reshard_by_role_gives_the_directly_sharded_tree(n_in, n_out):
    ck = _ckpt()
    cfg = dict(spec.tiny_config(), n_heads=8)
    fw_cfg = dict(cfg, cores_per_replica=n_in)
    fw = spec.full_weights(fw_cfg, seed=5)
    rng = np.random.default_rng(1)
    fw["embed_b"] = rng.standard_normal(fw["embed_b"].shape).astype(np.float32)
    for lw in fw["layers"]:
        lw["ff_out_b"] = rng.standard_normal(lw["ff_out_b"].shape).astype(np.float32)
        lw["ln_scale"] = rng.standard_normal(lw["ln_scale"].shape).astype(np.float32)
    src = spec.shard_params(dict(cfg, cores_per_replica=n_in), fw)
    dst = spec.shard_params(dict(cfg, cores_per_replica=n_out), fw)
    for mod in src:
        for leaf in src[mod]:
            got = ck.reshard_by_role(mod, leaf, src[mod][leaf], n_out).numpy()
            assert got.shape == dst[mod][leaf].shape, (mod, leaf)
            assert np.array_equal(got, dst[mod][leaf]), (mod, leaf)


def test_summed_bias_keeps_its_sum_when_every_shard_holds_a_copy():
    ck = _ckpt()
    b = np.stack([np.arange(6, dtype=np.float32)] * 8)           # the training layout: identical copies
    got = ck.reshard_by_role("causal_transformer_shard/~/layer_0/~/linear_5", "b", b, 2).numpy()
    assert np.array_equal(got.sum(0), b.sum(0)) and np.array_equal(got[0], 4 * b[0])


def test_read_ckpt_reshards_by_role_and_keeps_the_optimiser_slot(tmp_path):
    ck = _ckpt()
    cfg4, st4 = _state(4)
    cfg2, st2 = _state(2)
    d = str(tmp_path) + "/"
    for s in range(4):
        ck.write_ckpt(st4, d, s)
    template = dict(st2, opt_state={"count": np.zeros((2,), np.int32)})
    out = ck.read_ckpt(template, d, 4, 2, by_role=True)
    assert out["opt_state"] is template["opt_state"]                 # no optimiser state on disk: slot kept
    assert np.array_equal(out["step"].numpy(), [11, 11])
    for mod in st2["params"]:
        for leaf in st2["params"][mod]:
            assert np.array_equal(out["params"][mod][leaf].numpy(), st2["params"][mod][leaf]), (mod, leaf)
    with pytest.raises(AssertionError):
        ck.read_ckpt({"params": {"m": {"w": np.zeros((4, 3))}}, "step": np.zeros((4,)), "opt_state": None}, d, 4)
