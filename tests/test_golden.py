"""Committed golden vectors (tests/golden/tiny_gptj.npz, made by make_golden.py
from the CPU oracle): the oracle must keep reproducing them, and the CUDA path
must match them within the path's tolerances."""
import os

import numpy as np
import pytest

from oracle import gptj_oracle as go
from oracle import sampling_oracle as so
from oracle import spec

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_gptj.npz"))


def _model():
    cfg = spec.tiny_config(1, seq=128)
    return cfg, spec.make_params(cfg, seed=0, stress=False)


def test_oracle_reproduces_golden_vectors():
    cfg, params = _model()
    net = go.CausalTransformer(cfg, params)
    ids = G["ids"]
    logits = np.stack([net._shard().logits(ids[b]) for b in range(2)])
    assert np.abs(logits[:, -8:] - G["logits_last8"]).max() < 1e-5
    assert np.abs(logits[:, ::16, :64] - G["logits_pos"]).max() < 1e-5
    ev = net.eval({"obs": ids[:, :-1], "target": ids[:, 1:]})
    assert np.abs(ev["all_loss"] - G["all_loss"]).max() < 1e-5
    _, gen = net.generate(G["ctx"], G["lens"], 32)
    assert np.array_equal(gen[0], G["greedy_tokens"])
    assert np.array_equal(so.nucleaus_sample(G["s_unif"], G["s_logits"], G["s_top_p"], G["s_temp"]), G["s_tokens"])


@pytest.mark.gpu
def test_cuda_path_matches_golden_vectors(cuda_device):
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.sampling import nucleaus_sample
    from mesh_transformer.transformer_shard import CausalTransformer
    cfg, params = _model()
    net = CausalTransformer(dict(cfg), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    ids = G["ids"]
    rel = lambda a, b: float(np.abs(a - b).max() / np.abs(b).max())
    ev = net.eval({"obs": ids[:, :-1], "target": ids[:, 1:]})
    assert np.abs(ev["all_loss"] - G["all_loss"]).max() <= 2e-2
    assert abs(ev["all_loss"].mean() - G["all_loss"].mean()) <= 1e-3
    _, gen = net.generate(G["ctx"], G["lens"], 32, {"top_p": np.zeros(2), "temp": np.ones(2)}, return_logits=True)
    assert np.array_equal(gen[0], G["greedy_tokens"])
    assert rel(gen[2][:, 0, 0, :], G["greedy_logits_first"]) <= 2e-2
    rt = net._runtime(2, 32)
    last8 = rt.forward_logits(torch.from_numpy(ids.view(np.int32)).to(cuda_device), None, 8).cpu().numpy()
    assert rel(last8, G["logits_last8"]) <= 2e-2
    toks, _ = nucleaus_sample(torch.from_numpy(G["s_unif"]).to(cuda_device), G["s_logits"], None,
                              top_p=G["s_top_p"], temp=G["s_temp"])
    assert np.array_equal(toks, G["s_tokens"])
