"""Module classes of the reference's layers.py for the GPT-J path, as thin
host objects over one GPU runtime (``ShardRuntime``) whose parameters have been
loaded.  Like the reference's modules they work on ONE sequence (unbatched
``[T, ...]`` arrays; the reference vmaps them over the batch).

The attention / feed-forward / projection pieces of a layer are fused in the
CUDA kernels, so ``self_attn``, ``ff`` and ``qvk_proj`` are not separately
callable; RMSNorm, T5 relative positions, learned positions and the V2 modules
are outside the path (``getnorm`` raises like layers.py:77).
"""
from __future__ import annotations

import numpy as np
import torch

from ._runtime import ShardRuntime, validate_config
from .util import g_psum


def getnorm(type):
    """layers.py:61-77: only "layernorm" (ReplicatedLayerNorm, fused into the
    consuming projection kernel) exists on this path."""
    if type == "layernorm":
        return "layernorm"
    raise Exception("Not implemented")


def fixed_pos_embedding(n_pos: int, dim: int):
    """(sin, cos) tables [n_pos, dim/2] in float64 (layers.py:128-134); the
    library builds the same table internally for its RoPE epilogue."""
    inv_freq = 1.0 / (10000 ** (np.arange(0, dim, 2) / dim))
    ang = np.arange(n_pos)[:, None] * inv_freq[None, :]
    return np.sin(ang), np.cos(ang)


def _key_limit_from_bias(attn_bias, T):
    """The reference's attn_bias on this path is 0 or the eval key mask
    ``(arange(T) > ctx_length) * -1e10`` (transformer_shard.py:130)."""
    if attn_bias is None or (np.isscalar(attn_bias) and attn_bias == 0):
        return None
    m = np.asarray(attn_bias)
    if m.ndim != 1 or m.shape[0] != T:
        raise NotImplementedError("attn_bias must be 0 or a per-key mask of length T")
    masked = m != 0
    first = int(np.argmax(masked)) if masked.any() else T
    if not masked[first:].all():
        raise NotImplementedError("only masks of the form arange(T) > ctx_length are supported")
    return first - 1


class EmbeddingShard:
    """layers.py:165-202 (pe != "fixed")."""

    def __init__(self, config, name=None, runtime: ShardRuntime | None = None):
        validate_config(config)
        assert config["n_vocab"] % config["cores_per_replica"] == 0           # layers.py:172
        self.in_dim = config["n_vocab"]
        self.out_dim = config["d_model"]
        self.in_dim_per_shard = self.in_dim // config["cores_per_replica"]
        self.runtime = runtime

    def __call__(self, x, dtype=None):
        ids = torch.as_tensor(np.asarray(x).astype(np.int64).astype(np.int32)).to(self.runtime.device)
        out, _ = self.runtime.embed(ids.contiguous())
        return g_psum(out)                                                   # layers.py:193


class TransformerLayerShard:
    """layers.py:229-366."""

    def __init__(self, config, name=None, init_scale=1., runtime: ShardRuntime | None = None):
        validate_config(config)
        heads, dim, shards = config["n_heads"], config["d_model"], config["cores_per_replica"]
        getnorm(config["norm"])
        self.is_rotary = config["pe"] == "rotary"
        self.dim = dim
        self.dim_per_head = dim // heads
        self.heads_per_shard = heads // shards
        self.dim_per_shard = dim // shards
        self.pe_rotary_dims = config.get("pe_rotary_dims", self.dim_per_head)
        self.index = int(name.split("_")[-1]) if name else 0
        self.runtime = runtime

    def self_attn(self, q, v, k, attn_bias):
        raise NotImplementedError("attention is fused with the projections in the CUDA kernels")

    def ff(self, x):
        raise NotImplementedError("the feed-forward is fused with the projections in the CUDA kernels")

    def qvk_proj(self, x):
        raise NotImplementedError("the q/v/k projections are fused with LayerNorm and RoPE in the CUDA kernels")

    def __call__(self, x, attn_bias):
        """g_psum(attn_out + dense_out) for a full causal sequence (layers.py:299-313)."""
        T = x.shape[0]
        lim = _key_limit_from_bias(attn_bias, T)
        return self.runtime.layer(self.index, x, 1, T, 0, None, None if lim is None else [lim])

    def get_init_decode_state(self, x, given_length, attn_bias):
        """layers.py:347-366: the first T - given_length keys are left padding."""
        T = x.shape[0]
        if _key_limit_from_bias(attn_bias, T) is not None:
            raise NotImplementedError("attn_bias must be 0 when building a decode state")
        given = int(given_length)
        out = self.runtime.layer(self.index, x, 1, T, 0, [T - given], None)
        return out, {"tokens_decoded": given, "window": T, "pad": T - given, "pos": T, "k": None, "v": None}

    def decode_once(self, decode_state, x, attn_bias):
        """layers.py:316-344: one token; K/V live in the runtime's cache."""
        assert x.shape[0] == 1                                               # layers.py:320
        st = dict(decode_state)
        out = self.runtime.layer(self.index, x, 1, 1, st["pos"], [st["pad"]], None, decode=True)
        st["tokens_decoded"] += 1
        st["pos"] += 1
        return out, st


class ProjectionShard:
    """layers.py:545-593."""

    def __init__(self, config, name=None, runtime: ShardRuntime | None = None):
        validate_config(config)
        assert config["n_vocab"] % config["cores_per_replica"] == 0           # layers.py:552
        getnorm(config["norm"])
        self.dim = config["n_vocab"]
        self.dim_per_shard = self.dim // config["cores_per_replica"]
        self.runtime = runtime

    def __call__(self, x):
        """LN -> Linear -> all_gather, vocabulary shard-major (layers.py:561-567)."""
        return self.runtime.projection(x)

    def loss(self, x, targets, z_loss=1):
        """layers.py:569-593 for z_loss == 0 (the eval path, transformer_shard.py:47,65)."""
        if float(z_loss) != 0.0:
            raise NotImplementedError("z_loss belongs to training, which is outside this path")
        t = torch.as_tensor(np.asarray(targets).astype(np.int64).astype(np.int32)).to(self.runtime.device)
        return self.runtime.projection_loss(x, t.contiguous())
