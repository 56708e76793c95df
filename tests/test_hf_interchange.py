"""Sharded tree <-> Hugging Face GPT-J state dict (to_hf_weights.py name map and un-sharding rules)."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "mesh-transformer-jax_b200"))

from oracle import gptj_oracle as go  # noqa: E402
from oracle import spec  # noqa: E402


def _params(mp, seed=4):
    cfg = dict(spec.tiny_config(), cores_per_replica=mp)
    fw = spec.full_weights(cfg, seed, stress=True)
    return cfg, fw, spec.shard_params(cfg, fw)


def test_name_map():
    from mesh_transformer.hf_interchange import PREFIX, leaf_to_hf_id
    assert leaf_to_hf_id(PREFIX + "embedding_shard/~/linear", "w") == "transformer.wte.weight"
    assert leaf_to_hf_id(PREFIX + "layer_7/~/linear", "w") == "transformer.h.7.attn.q_proj.weight"
    assert leaf_to_hf_id(PREFIX + "layer_7/~/linear_1", "w") == "transformer.h.7.attn.v_proj.weight"
    assert leaf_to_hf_id(PREFIX + "layer_7/~/linear_2", "w") == "transformer.h.7.attn.k_proj.weight"
    assert leaf_to_hf_id(PREFIX + "layer_0/~/linear_3", "w") == "transformer.h.0.attn.out_proj.weight"
    assert leaf_to_hf_id(PREFIX + "layer_12/~/linear_4", "b") == "transformer.h.12.mlp.fc_in.bias"
    assert leaf_to_hf_id(PREFIX + "layer_12/~/linear_5", "w") == "transformer.h.12.mlp.fc_out.weight"
    assert leaf_to_hf_id(PREFIX + "layer_3/~/replicated_layer_norm", "scale") == "transformer.h.3.ln_1.weight"
    assert leaf_to_hf_id(PREFIX + "projection_shard/~/replicated_layer_norm", "offset") == "transformer.ln_f.bias"
    assert leaf_to_hf_id(PREFIX + "projection_shard/~/linear", "b") == "lm_head.bias"
    with pytest.raises(NotImplementedError):
        leaf_to_hf_id("opt_state/foo", "w")
    with pytest.raises(NotImplementedError):
        leaf_to_hf_id(PREFIX + "layer_3/~/linear", "gain")


@pytest.mark.parametrize("mp", [1, 4])
def test_exported_state_dict_runs_in_transformers_and_matches_the_oracle(mp):
    tr = pytest.importorskip("transformers")
    from mesh_transformer.hf_interchange import hf_config, to_hf_state_dict
    cfg, fw, p = _params(mp)
    sd = to_hf_state_dict(p, cfg, torch_dtype=torch.float32)
    hc = hf_config(cfg, torch.float32)
    assert hc["n_embd"] == 256 and hc["rotary_dim"] == cfg["pe_rotary_dims"] and hc["torch_dtype"] == "float32"
    conf = tr.GPTJConfig(vocab_size=hc["vocab_size"], n_positions=hc["n_positions"], n_embd=hc["n_embd"],
                         n_layer=hc["n_layer"], n_head=hc["n_head"], rotary_dim=hc["rotary_dim"],
                         activation_function=hc["activation_function"], layer_norm_epsilon=hc["layer_norm_epsilon"],
                         attn_pdrop=0.0, embd_pdrop=0.0, resid_pdrop=0.0)
    model = tr.GPTJForCausalLM(conf).float().eval()
    res = model.load_state_dict(sd, strict=False)
    assert all(k.endswith("attn.bias") or k.endswith("attn.masked_bias") for k in res.unexpected_keys)
    assert not [k for k in res.missing_keys if "attn.bias" not in k and "masked_bias" not in k
                and "inv_freq" not in k and "embed_positions" not in k]
    ids = spec.token_ids(0, 2, 64, 512)
    with torch.no_grad():
        hl = model(torch.tensor(ids.astype(np.int64))).logits.numpy()
    net = go.CausalTransformer(cfg, p)
    ol = np.stack([net._shard().logits(ids[b]) for b in range(2)])
    assert np.abs(hl - ol).max() <= 2e-4 * np.abs(ol).max()


@pytest.mark.parametrize("mp_in,mp_out", [(4, 1), (2, 4)])
def test_import_inverts_export(mp_in, mp_out):
    from mesh_transformer.hf_interchange import from_hf_state_dict, to_hf_state_dict
    cfg, fw, p = _params(mp_in)
    fw["embed_b"][:] = 0                                      # HF keeps the embedding bias folded into the table
    p = spec.shard_params(cfg, fw)
    sd = to_hf_state_dict(p, cfg, torch_dtype=torch.float32)
    back = from_hf_state_dict(sd, dict(cfg, cores_per_replica=mp_out))
    want = spec.shard_params(dict(cfg, cores_per_replica=mp_out), fw)
    assert sorted(back) == sorted(want)
    for mod in want:
        for leaf in want[mod]:
            assert np.array_equal(back[mod][leaf].numpy(), want[mod][leaf]), (mod, leaf)
