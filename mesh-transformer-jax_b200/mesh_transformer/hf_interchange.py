"""Sharded parameter tree <-> Hugging Face ``GPTJForCausalLM`` state dict
(reference: to_hf_weights.py:160-173 name map, :227-249,327-335 un-sharding rules,
:386-397 embedding bias fold, :405-414 attention mask buffers, :415-449 config).

Host side, torch only.  The un-sharding uses the by-role rules of
``checkpoint.reshard_by_role`` (LayerNorm from shard 0, embedding / ff-out
biases summed over shards, column- / row-parallel concatenation), which is
what to_hf_weights.py does leaf by leaf.
"""
from __future__ import annotations

import re

import torch

from .checkpoint import _from_numpy, reshard_by_role

PREFIX = "causal_transformer_shard/~/"

# Haiku module inside a layer -> GPT-J sub-module (to_hf_weights.py:160-168)
LAYER_MODULES = {
    "linear": "attn.q_proj",
    "linear_1": "attn.v_proj",
    "linear_2": "attn.k_proj",
    "linear_3": "attn.out_proj",
    "linear_4": "mlp.fc_in",
    "linear_5": "mlp.fc_out",
    "replicated_layer_norm": "ln_1",
}
# inside the projection shard (to_hf_weights.py:170-173)
PROJECTION_MODULES = {"linear": "lm_head", "replicated_layer_norm": "transformer.ln_f"}


LEAF_KINDS = {"w": "weight", "scale": "weight", "b": "bias", "offset": "bias"}
_LAYER = re.compile(r"layer_(\d+)$")


def leaf_to_hf_id(module: str, leaf: str) -> str:
    """'causal_transformer_shard/~/layer_3/~/linear_4', 'b' -> 'transformer.h.3.mlp.fc_in.bias': a lookup in the
    two tables above (the reference walks the same names in to_hf_weights.py:176-225).  Anything the tables do
    not hold (optimizer state, other module trees) raises NotImplementedError."""
    parts = module[len(PREFIX):].split("/~/") if module.startswith(PREFIX) else []
    kind = LEAF_KINDS.get(leaf)
    if len(parts) == 2 and kind is not None:
        top, inner = parts
        layer = _LAYER.match(top)
        if top == "embedding_shard" and inner == "linear":
            return f"transformer.wte.{kind}"
        if layer and inner in LAYER_MODULES:
            return f"transformer.h.{int(layer.group(1))}.{LAYER_MODULES[inner]}.{kind}"
        if top == "projection_shard" and inner in PROJECTION_MODULES:
            return f"{PROJECTION_MODULES[inner]}.{kind}"
    raise NotImplementedError(f"no Hugging Face GPT-J name for parameter '{module}/{leaf}'")


def _as_tensor(x):
    return x if isinstance(x, torch.Tensor) else _from_numpy(x)


def to_hf_state_dict(params: dict, config: dict, torch_dtype=torch.float16) -> dict:
    """``params``: the two-level tree with all shards on the leading axis.  Linear
    weights are stored [in, out] here and [out, in] in the HF model (transposed,
    to_hf_weights.py:383); the embedding table is not transposed and absorbs the
    summed embedding bias, which HF has no slot for (:386-397)."""
    out = {}
    wte_w = wte_b = None
    for module in sorted(params):
        for leaf in sorted(params[module]):
            hf_id = leaf_to_hf_id(module, leaf)
            x = reshard_by_role(module, leaf, _as_tensor(params[module][leaf]).cpu(), 1)[0].to(torch.float32)
            if hf_id == "transformer.wte.weight":
                wte_w = x
            elif hf_id == "transformer.wte.bias":
                wte_b = x
            else:
                out[hf_id] = (x.T if x.dim() == 2 else x).contiguous().to(torch_dtype)
    out["transformer.wte.weight"] = (wte_w + (wte_b if wte_b is not None else 0.0)).to(torch_dtype)
    n_seq = config["seq"]
    mask = torch.tril(torch.ones((n_seq, n_seq), dtype=torch.bool)).view(1, 1, n_seq, n_seq)
    for i in range(config["layers"]):
        out[f"transformer.h.{i}.attn.bias"] = mask
        out[f"transformer.h.{i}.attn.masked_bias"] = torch.tensor(-1e9, dtype=torch_dtype)
    return out


def hf_config(config: dict, torch_dtype=torch.float16) -> dict:
    """The config.json written beside the weights (to_hf_weights.py:415-449)."""
    return {
        "activation_function": "gelu_new",
        "architectures": ["GPTJForCausalLM"],
        "attn_pdrop": 0.0,
        "bos_token_id": 50256,
        "embd_pdrop": 0.0,
        "eos_token_id": 50256,
        "gradient_checkpointing": False,
        "initializer_range": 0.02,
        "layer_norm_epsilon": 1e-05,
        "model_type": "gptj",
        "n_embd": config["d_model"],
        "n_head": config["n_heads"],
        "n_layer": config["layers"],
        "n_positions": config["seq"],
        "rotary_dim": config["pe_rotary_dims"],
        "summary_activation": None,
        "summary_first_dropout": 0.1,
        "summary_proj_to_labels": True,
        "summary_type": "cls_index",
        "summary_use_proj": True,
        "transformers_version": "4.10.0.dev0",
        "tokenizer_class": "GPT2Tokenizer",
        "task_specific_params": {"text-generation": {"do_sample": True, "temperature": 1.0, "max_length": 50}},
        "torch_dtype": str(torch_dtype).split(".")[-1],
        "use_cache": True,
        "vocab_size": config["n_vocab"],
    }


def from_hf_state_dict(sd: dict, config: dict, dtype=torch.float32) -> dict:
    """The inverse map: an HF GPT-J state dict -> the sharded tree for
    ``config['cores_per_replica']`` shards.  Biases that every shard adds before
    the all-reduce (ff-out) go to shard 0 in full, zeros elsewhere; the embedding
    bias stays zero (HF keeps it folded into the table)."""
    mp = config["cores_per_replica"]
    d, L = config["d_model"], config["layers"]

    def get(name):
        return sd[name].to(torch.float32)

    def cols(w):                                             # [in, out] -> [mp, in, out / mp]
        return torch.stack(torch.chunk(w, mp, dim=1)).to(dtype).contiguous()

    def rows(w):                                             # [in, out] -> [mp, in / mp, out]
        return torch.stack(torch.chunk(w, mp, dim=0)).to(dtype).contiguous()

    def rep(v):
        return torch.stack([v] * mp).to(dtype).contiguous()

    def first(v):
        return torch.stack([v] + [torch.zeros_like(v)] * (mp - 1)).to(dtype).contiguous()

    p = {PREFIX + "embedding_shard/~/linear": {"w": rows(get("transformer.wte.weight")),
                                               "b": torch.zeros((mp, d), dtype=dtype)}}
    for i in range(L):
        h, base = f"transformer.h.{i}.", PREFIX + f"layer_{i}/~/"
        p[base + "replicated_layer_norm"] = {"scale": rep(get(h + "ln_1.weight")), "offset": rep(get(h + "ln_1.bias"))}
        p[base + "linear"] = {"w": cols(get(h + "attn.q_proj.weight").T)}
        p[base + "linear_1"] = {"w": cols(get(h + "attn.v_proj.weight").T)}
        p[base + "linear_2"] = {"w": cols(get(h + "attn.k_proj.weight").T)}
        p[base + "linear_3"] = {"w": rows(get(h + "attn.out_proj.weight").T)}
        p[base + "linear_4"] = {"w": cols(get(h + "mlp.fc_in.weight").T),
                                "b": torch.stack(torch.chunk(get(h + "mlp.fc_in.bias"), mp)).to(dtype).contiguous()}
        p[base + "linear_5"] = {"w": rows(get(h + "mlp.fc_out.weight").T), "b": first(get(h + "mlp.fc_out.bias"))}
    p[PREFIX + "projection_shard/~/replicated_layer_norm"] = {"scale": rep(get("transformer.ln_f.weight")),
                                                             "offset": rep(get("transformer.ln_f.bias"))}
    p[PREFIX + "projection_shard/~/linear"] = {
        "w": cols(get("lm_head.weight").T),
        "b": torch.stack(torch.chunk(get("lm_head.bias"), mp)).to(dtype).contiguous()}
    return p
