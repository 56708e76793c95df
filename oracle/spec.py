"""Seeded synthetic configs, weights and inputs shared by the parity tests.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The parameter tree mirrors the Haiku tree the reference builds
(names: to_hf_weights.py:160-173,183-186; shapes: mesh_transformer/layers.py:185,
235-258,550-559).  Every leaf carries a leading shard axis of size
``cores_per_replica`` like ``CausalTransformer.state["params"]``
(transformer_shard.py:218-222).
"""
from __future__ import annotations

import numpy as np

PREFIX = "causal_transformer_shard/~/"


def tiny_config(mp: int = 1, seq: int = 128) -> dict:
    """The CPU-runnable GPT-J-style case: L2 d256 h4 dh64 R16 V512."""
    return {
        "layers": 2, "d_model": 256, "n_heads": 4, "n_vocab": 512,
        "norm": "layernorm", "pe": "rotary", "pe_rotary_dims": 16,
        "seq": seq, "cores_per_replica": mp, "per_replica_batch": 1,
    }


def gptj6b_config(mp: int = 1) -> dict:
    """configs/6B_roto_256.json:1-12 of the reference."""
    return {
        "layers": 28, "d_model": 4096, "n_heads": 16, "n_vocab": 50400,
        "norm": "layernorm", "pe": "rotary", "pe_rotary_dims": 64,
        "seq": 2048, "cores_per_replica": mp, "per_replica_batch": 1,
    }


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even) and return it as fp32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))   # wraps like the low 32 bits of a wider sum
    r &= np.uint32(0xFFFF0000)
    return r.view(np.float32).reshape(a.shape)


def full_weights(config: dict, seed: int = 0, stress: bool = False,
                 bf16: bool = True) -> dict:
    """Un-sharded model weights, N(0, 0.02) matrices from PCG64(seed).

    Leaf order is fixed (embedding, layers in order q,v,k,o,ff_in,ff_out,
    final LN, projection).  ``stress`` makes LN scale/offset and all biases
    non-trivial so layers.py:25-34 and :256-258 are exercised.
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    d, V, L = config["d_model"], config["n_vocab"], config["layers"]

    def mat(*shape):
        w = rng.normal(0.0, 0.02, size=shape).astype(np.float32)
        return round_bf16(w) if bf16 else w

    def vec(n, base):
        if not stress:
            return np.full((n,), base, np.float32)
        v = (base + rng.normal(0.0, 0.1, size=(n,))).astype(np.float32)
        return round_bf16(v) if bf16 else v

    fw = {"embed_w": mat(V, d), "embed_b": vec(d, 0.0), "layers": []}
    for _ in range(L):
        fw["layers"].append({
            "ln_scale": vec(d, 1.0), "ln_offset": vec(d, 0.0),
            "q": mat(d, d), "v": mat(d, d), "k": mat(d, d), "o": mat(d, d),
            "ff_in_w": mat(d, 4 * d), "ff_in_b": vec(4 * d, 0.0),
            "ff_out_w": mat(4 * d, d), "ff_out_b": vec(d, 0.0),
        })
    fw["lnf_scale"] = vec(d, 1.0)
    fw["lnf_offset"] = vec(d, 0.0)
    fw["proj_w"] = mat(d, V)
    fw["proj_b"] = vec(V, 0.0)
    return fw


def shard_params(config: dict, fw: dict) -> dict:
    """Slice un-sharded weights into the reference's per-shard Haiku tree.

    Column-parallel q/v/k/ff_in (layers.py:249-251,256), row-parallel o/ff_out
    (:253,257), vocab-sharded embedding rows (:176,185) and projection columns
    (:555,559).  Biases that every shard adds before the all-reduce
    (embedding b, ff_out b) are effective as their SUM over shards
    (layers.py:191-193,290,313): shard 0 carries the full bias, the others 0.
    """
    mp = config["cores_per_replica"]
    d, V, L = config["d_model"], config["n_vocab"], config["layers"]
    assert V % mp == 0 and d % mp == 0

    def cols(w):  # [in, out] -> [mp, in, out/mp]
        return np.stack(np.split(w, mp, axis=1))

    def rows(w):  # [in, out] -> [mp, in/mp, out]
        return np.stack(np.split(w, mp, axis=0))

    def rep(v):
        return np.stack([v] * mp)

    def first(v):
        z = np.zeros_like(v)
        return np.stack([v] + [z] * (mp - 1))

    p = {PREFIX + "embedding_shard/~/linear":
         {"w": rows(fw["embed_w"]), "b": first(fw["embed_b"])}}
    for i in range(L):
        lw = fw["layers"][i]
        base = PREFIX + f"layer_{i}/~/"
        p[base + "replicated_layer_norm"] = {"scale": rep(lw["ln_scale"]),
                                             "offset": rep(lw["ln_offset"])}
        p[base + "linear"] = {"w": cols(lw["q"])}
        p[base + "linear_1"] = {"w": cols(lw["v"])}
        p[base + "linear_2"] = {"w": cols(lw["k"])}
        p[base + "linear_3"] = {"w": rows(lw["o"])}
        p[base + "linear_4"] = {"w": cols(lw["ff_in_w"]),
                                "b": np.stack(np.split(lw["ff_in_b"], mp))}
        p[base + "linear_5"] = {"w": rows(lw["ff_out_w"]),
                                "b": first(lw["ff_out_b"])}
    p[PREFIX + "projection_shard/~/replicated_layer_norm"] = {
        "scale": rep(fw["lnf_scale"]), "offset": rep(fw["lnf_offset"])}
    p[PREFIX + "projection_shard/~/linear"] = {
        "w": cols(fw["proj_w"]), "b": np.stack(np.split(fw["proj_b"], mp))}
    return p


def make_params(config: dict, seed: int = 0, stress: bool = False,
                bf16: bool = True) -> dict:
    return shard_params(config, full_weights(config, seed, stress, bf16))


def token_ids(seed: int, batch: int, length: int, vocab: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, vocab, size=(batch, length)).astype(np.uint32)


def left_pad(tokens: np.ndarray, seq: int) -> np.ndarray:
    """device_serve.py:162-175 -- zero-pad on the left up to ``seq``."""
    b, n = tokens.shape
    out = np.zeros((b, seq), np.uint32)
    out[:, seq - n:] = tokens
    return out
