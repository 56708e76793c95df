"""Restatement of the reference's v1 checkpoint format and re-sharding rules
(mesh_transformer/checkpoint.py:16-175) in NumPy.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the
reference holds no test or fixture for its checkpoint code and its own module
cannot be imported here (jax, ray and smart_open are absent), so these
functions restate it line by line and are checked for self-consistency only.

Format (checkpoint.py:16,57-79,82-92): the state pytree is flattened in JAX
order (dict keys sorted, ``None`` holds no leaves), every leaf is indexed with
the shard number on its leading axis, the list of leaves is cut into 16
consecutive pieces and piece ``i`` is stored as ``shard_{s}/{i}.npz`` with the
arrays as positional entries (``arr_0`` ...).  bfloat16 leaves come back from
``np.load`` as 2-byte void (``V2``) and are relabelled (:20-23,153-155).
"""
from __future__ import annotations

import io
import os

import numpy as np

PIECES = 16                                   # checkpoint.py:16


def tree_flatten(tree):
    """Leaves in jax.tree_flatten order: dict keys sorted, None is an empty node."""
    if tree is None:
        return []
    if isinstance(tree, dict):
        out = []
        for k in sorted(tree):
            out += tree_flatten(tree[k])
        return out
    if isinstance(tree, (list, tuple)):
        out = []
        for v in tree:
            out += tree_flatten(v)
        return out
    return [tree]


def split(a, n):
    """checkpoint.py:52-54: n consecutive chunks, the first len(a) % n one longer."""
    k, m = divmod(len(a), n)
    return [a[i * k + min(i, m):(i + 1) * k + min(i + 1, m)] for i in range(n)]


def write_ckpt(pytree, directory, shard):
    """checkpoint.py:57-79 (the thread pool and the retry loop are I/O plumbing)."""
    leaves = [np.asarray(x)[shard] for x in tree_flatten(pytree)]
    os.makedirs(os.path.join(directory, f"shard_{shard}"), exist_ok=True)
    for idx, chunk in enumerate(split(leaves, PIECES)):
        with open(os.path.join(directory, f"shard_{shard}", f"{idx}.npz"), "wb") as f:
            np.savez(f, *chunk)


def read_shard(ckpt_dir):
    """checkpoint.py:82-92."""
    out = []
    for idx in range(PIECES):
        with open(os.path.join(ckpt_dir, f"{idx}.npz"), "rb") as f:
            z = np.load(io.BytesIO(f.read()))
            for name in z:
                out.append(z[name])
    return out


def reshard(x, old_shape):
    """checkpoint.py:95-132 for one stacked leaf ``x`` = [shards_in, ...] and the
    target shape ``old_shape`` = [shards_out, ...]."""
    x = np.asarray(x)
    if x.ndim == 1:                                           # :96-99 scalar per shard (step)
        return x[0:1]
    if x.ndim == 2:                                           # :101-117 LN / bias
        if (x[1:] == x[-1]).all():
            if (x[1:] == 0).all() or (x[1:] == 1).all():
                return x[0:1]                                 # :106-107 untouched LN
            return x[0:1] * x.shape[0] / old_shape[0]         # :108-110 "shard bias"
        return x.reshape(old_shape)                           # :111-113 column-parallel bias
    if x.ndim == 3:                                           # :119-128 weights
        if x.shape[0] * x.shape[2] == old_shape[2]:
            return np.transpose(x, (1, 0, 2)).reshape(old_shape)      # column-parallel
        if x.shape[0] * x.shape[1] == old_shape[1]:
            return x.reshape(old_shape)                               # row-parallel
        raise Exception(f"unimplemented, {x.shape}, {old_shape}")
    raise Exception(f"unimplemented, {x}")


def read_ckpt_leaves(template_leaves, directory, shards_in, shards_out=None):
    """The leaf loop of checkpoint.py:135-175: stack the shards of every leaf and
    re-shard when the shard counts differ."""
    if shards_out is None:
        shards_out = shards_in
    shards = [read_shard(os.path.join(directory, f"shard_{i}")) for i in range(shards_in)]
    out = []
    for old, *all_shards in zip(template_leaves, *shards):
        x = np.stack(all_shards)
        if shards_out != shards_in:
            x = reshard(x, np.asarray(old).shape)
        assert x.shape == np.asarray(old).shape, f"Incompatible checkpoints {x.shape} vs {np.asarray(old).shape}"
        out.append(x)
    return out
