"""The CPU oracle checked against itself and an independent implementation."""
import numpy as np
import pytest

from oracle import gptj_oracle as go
from oracle import spec


@pytest.fixture(scope="module")
def tiny_full():
    cfg = spec.tiny_config(1)
    return spec.full_weights(cfg, seed=0, stress=True)


@pytest.mark.parametrize("mp", [2, 4])
def test_shard_count_does_not_change_results(tiny_full, mp):
    ids = spec.token_ids(0, 2, 128, 512)
    outs = []
    for m in (1, mp):
        cfg = spec.tiny_config(m)
        net = go.CausalTransformer(cfg, spec.shard_params(cfg, tiny_full))
        logits = net._shard().logits(ids[0])
        ev = net.eval({"obs": ids[:, :-1], "target": ids[:, 1:]})
        _, gen = net.generate(ids, np.array([128, 100]), 6, return_logits=True)
        outs.append((logits, ev, gen))
    a, b = outs
    assert np.abs(a[0] - b[0]).max() < 5e-6
    assert np.abs(a[1]["all_loss"] - b[1]["all_loss"]).max() < 5e-6
    assert (a[1]["correct"] == b[1]["correct"]).all()
    assert (a[2][0] == b[2][0]).all()
    assert np.abs(a[2][2] - b[2][2]).max() < 5e-6


def test_against_hf_gptj(tiny_full):
    """transformers' GPTJForCausalLM with weights mapped as to_hf_weights.py:160-173,
    :384-397 does (transpose, wte = table + summed bias)."""
    torch = pytest.importorskip("torch")
    tr = pytest.importorskip("transformers")
    cfg = spec.tiny_config(2)
    fw = tiny_full
    hc = tr.GPTJConfig(vocab_size=512, n_positions=128, n_embd=256, n_layer=2, n_head=4,
                       rotary_dim=16, activation_function="gelu_new", layer_norm_epsilon=1e-5,
                       attn_pdrop=0.0, embd_pdrop=0.0, resid_pdrop=0.0)
    model = tr.GPTJForCausalLM(hc).float().eval()
    t = lambda a: torch.tensor(np.ascontiguousarray(a.T))
    sd = {"transformer.wte.weight": torch.tensor(fw["embed_w"] + fw["embed_b"])}
    for i, lw in enumerate(fw["layers"]):
        b = f"transformer.h.{i}."
        sd[b + "ln_1.weight"] = torch.tensor(lw["ln_scale"])
        sd[b + "ln_1.bias"] = torch.tensor(lw["ln_offset"])
        sd[b + "attn.q_proj.weight"] = t(lw["q"])
        sd[b + "attn.v_proj.weight"] = t(lw["v"])
        sd[b + "attn.k_proj.weight"] = t(lw["k"])
        sd[b + "attn.out_proj.weight"] = t(lw["o"])
        sd[b + "mlp.fc_in.weight"] = t(lw["ff_in_w"])
        sd[b + "mlp.fc_in.bias"] = torch.tensor(lw["ff_in_b"])
        sd[b + "mlp.fc_out.weight"] = t(lw["ff_out_w"])
        sd[b + "mlp.fc_out.bias"] = torch.tensor(lw["ff_out_b"])
    sd["transformer.ln_f.weight"] = torch.tensor(fw["lnf_scale"])
    sd["transformer.ln_f.bias"] = torch.tensor(fw["lnf_offset"])
    sd["lm_head.weight"] = t(fw["proj_w"])
    sd["lm_head.bias"] = torch.tensor(fw["proj_b"])
    model.load_state_dict(sd, strict=False)
    ids = spec.token_ids(0, 2, 128, 512)
    with torch.no_grad():
        hf = model(torch.tensor(ids.astype(np.int64))).logits.numpy()
    net = go.CausalTransformer(cfg, spec.shard_params(cfg, fw))
    ours = np.stack([net._shard().logits(ids[b]) for b in range(2)])
    assert np.abs(hf - ours).max() < 1e-5


def test_decode_matches_full_forward():
    """The sliding-window decode (layers.py:316-344) reproduces the logits a full
    causal forward gives for the same tokens while nothing has been evicted."""
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=1)
    net = go.CausalTransformer(cfg, params)
    prompt = spec.token_ids(3, 1, 20, 512)
    ctx = spec.left_pad(prompt, 64)
    _, out = net.generate(ctx, np.array([20]), 5, return_logits=True)
    toks = out[0][0, :, 0]
    seq = np.concatenate([prompt[0], toks])
    full = net._shard().logits(seq)
    for t in range(5):
        assert np.abs(full[19 + t] - out[2][0, t, 0]).max() < 2e-5


def test_eval_key_mask_and_dict():
    cfg = spec.tiny_config(1, seq=32)
    net = go.CausalTransformer(cfg, spec.make_params(cfg, seed=2))
    ids = spec.token_ids(5, 2, 33, 512)
    out = net.eval({"obs": ids[:, :-1], "target": ids[:, 1:], "ctx_length": np.array([32, 10])})
    assert out["loss"].shape == (2,) and out["all_loss"].shape == (2, 32)
    assert np.allclose(out["loss"], out["all_loss"].mean(-1))
    assert np.allclose(out["last_loss"], out["all_loss"][:, -1])
    # keys beyond ctx_length are invisible: positions <= ctx_length are unaffected by it
    ref = net.eval({"obs": ids[:, :-1], "target": ids[:, 1:]})
    assert np.abs(out["all_loss"][1, :11] - ref["all_loss"][1, :11]).max() < 1e-5
    assert np.abs(out["all_loss"][1, 12:] - ref["all_loss"][1, 12:]).max() > 1e-4
