"""v1 checkpoint reader / writer / re-sharder of the reference
(mesh_transformer/checkpoint.py:16-175), host side, NumPy + torch only.

On-disk format (same files the reference writes and reads): the state pytree
is flattened in JAX order (dict keys sorted, ``None`` contributes nothing),
each leaf is indexed with the shard number, the leaf list is cut into 16
consecutive pieces and piece ``i`` becomes ``<dir>shard_{s}/{i}.npz`` with
positional arrays.  bfloat16 leaves are stored as 2-byte void (``V2``), which
is what ``np.savez`` makes of a JAX bfloat16 array and what the reference
relabels on load (checkpoint.py:20-23,153-155).

Leaves handed back are ``torch`` tensors on the CPU (NumPy has no bfloat16);
``ShardRuntime.load_params`` takes them as they are.

Re-sharding N -> M shards comes in two forms:

* ``reshard(x, old_shape)`` reproduces the reference's shape/value heuristic
  (checkpoint.py:95-132), including what it does to a trained LayerNorm (any
  replicated vector that is not all 0 or all 1 is scaled by N/M like a bias that
  every shard adds) and its weight rule, which is only meaningful for M = 1.
* ``reshard_by_role(module, leaf, x, shards_out)`` uses the parameter's role
  (to_hf_weights.py:160-173,227-249): LayerNorm copies are taken from shard 0,
  biases added on every shard (embedding, ff-out) keep their SUM, column-
  parallel leaves are concatenated on the output axis, row-parallel on the
  input axis, for any M that divides N.  ``read_ckpt(..., by_role=True)``.
"""
from __future__ import annotations

import io
import os

import numpy as np
import torch

pieces = 16  # files per shard directory (checkpoint.py:16)

_V2 = np.dtype("V2")


# ------------------------------------------------------------------ pytree ----
def tree_flatten(tree, path=()):
    """[(path, leaf)] in jax.tree_flatten order: dict keys sorted, None is empty."""
    if tree is None:
        return []
    if isinstance(tree, dict):
        out = []
        for k in sorted(tree):
            out += tree_flatten(tree[k], path + (k,))
        return out
    if isinstance(tree, (list, tuple)):
        out = []
        for i, v in enumerate(tree):
            out += tree_flatten(v, path + (i,))
        return out
    return [(path, tree)]


def tree_unflatten(template, leaves):
    """Rebuild ``template``'s structure from an iterator of leaves (same order as tree_flatten)."""
    it = iter(leaves)

    def build(t):
        if t is None:
            return None
        if isinstance(t, dict):
            return {k: build(t[k]) for k in sorted(t)}
        if isinstance(t, (list, tuple)):
            return type(t)(build(v) for v in t)
        return next(it)

    return build(template)


def _to_numpy(x):
    """Leaf -> NumPy array as np.savez would store it (bf16 as V2)."""
    if isinstance(x, torch.Tensor):
        x = x.detach().cpu().contiguous()
        if x.dtype == torch.bfloat16:
            return x.view(torch.int16).numpy().view(_V2)
        return x.numpy()
    return np.asarray(x)


def _from_numpy(a):
    """Stored array -> torch tensor (V2 relabelled as bfloat16)."""
    a = np.ascontiguousarray(a)
    if a.dtype == _V2:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


def split(a, n):
    """n consecutive chunks of ``a``; the first ``len(a) % n`` chunks hold one more (checkpoint.py:52-54)."""
    base, extra = divmod(len(a), n)
    out, start = [], 0
    for i in range(n):
        stop = start + base + (1 if i < extra else 0)
        out.append(a[start:stop])
        start = stop
    return out


# ------------------------------------------------------------------- write ----
def write_ckpt(pytree, dir, shard):
    """Writes shard ``shard`` of ``pytree`` (checkpoint.py:57-79).  A leaf whose
    leading axis has length 1 is taken as this process's only shard."""
    leaves = []
    for _, leaf in tree_flatten(pytree):
        a = _to_numpy(leaf)
        if a.ndim == 0:                                      # a scalar kept once per process (the step counter)
            leaves.append(a)
        else:
            leaves.append(a[0] if a.shape[0] == 1 else a[shard])
    shard_dir = f"{dir}shard_{shard}/"
    os.makedirs(shard_dir, exist_ok=True)
    for idx, chunk in enumerate(split(leaves, pieces)):
        tmp = f"{shard_dir}{idx}.npz.tmp"
        with open(tmp, "wb") as f:
            np.savez(f, *chunk)
        os.replace(tmp, f"{shard_dir}{idx}.npz")


# -------------------------------------------------------------------- read ----
def read_shard(ckpt_dir):
    """All leaves of one shard directory, in flatten order (checkpoint.py:82-92)."""
    out = []
    for idx in range(pieces):
        with open(f"{ckpt_dir}{idx}.npz", "rb") as f:
            z = np.load(io.BytesIO(f.read()))
            for name in z.files:
                out.append(z[name])
    return out


def reshard(x, old_shape):
    """The reference's heuristic for one stacked leaf [shards_in, ...] and the
    target shape [shards_out, ...] (checkpoint.py:95-132)."""
    t = x if isinstance(x, torch.Tensor) else _from_numpy(np.asarray(x))
    old_shape = tuple(int(v) for v in old_shape)
    if t.dim() == 1:
        return t[0:1]
    if t.dim() == 2:
        same = bool((t[1:] == t[-1]).all())
        if same:
            if bool((t[1:] == 0).all()) or bool((t[1:] == 1).all()):
                return t[0:1]
            return t[0:1] * t.shape[0] / old_shape[0]
        return t.reshape(old_shape)
    if t.dim() == 3:
        if t.shape[0] * t.shape[2] == old_shape[2]:
            return t.permute(1, 0, 2).reshape(old_shape)
        if t.shape[0] * t.shape[1] == old_shape[1]:
            return t.reshape(old_shape)
        raise Exception(f"unimplemented, {tuple(t.shape)}, {old_shape}")
    raise Exception(f"unimplemented, {t}")


def parameter_role(module: str, leaf: str) -> str:
    """'replicated' | 'summed' | 'column' | 'row' | 'scalar' for a Haiku module path and leaf name
    (to_hf_weights.py:160-173,227-249; layers.py:185,249-258,559)."""
    last = module.rsplit("/", 1)[-1]
    if "replicated_layer_norm" in last:
        return "replicated"
    if "embedding_shard" in module:
        return "row" if leaf == "w" else "summed"
    if "projection_shard" in module:
        return "column"
    if last in ("linear", "linear_1", "linear_2", "linear_4"):
        return "column"
    if last == "linear_3":
        return "row"
    if last == "linear_5":
        return "row" if leaf == "w" else "summed"
    raise KeyError(f"no sharding role known for {module}/{leaf}")


def reshard_by_role(module: str, leaf: str, x, shards_out: int):
    """[shards_in, ...] -> [shards_out, ...] for any shards_out dividing shards_in."""
    t = x if isinstance(x, torch.Tensor) else _from_numpy(np.asarray(x))
    n_in = t.shape[0]
    if n_in % shards_out:
        raise ValueError(f"cannot re-shard {n_in} shards into {shards_out}")
    g = n_in // shards_out                                   # old shards per new shard
    role = parameter_role(module, leaf)
    if role == "replicated":
        return t[0:1].expand((shards_out,) + tuple(t.shape[1:])).clone()
    if role == "summed":
        # every shard adds its copy before the all-reduce: a new shard carries the sum of the g it replaces
        grouped = t.reshape((shards_out, g) + tuple(t.shape[1:]))
        return grouped.to(torch.float32).sum(dim=1).to(t.dtype)
    grouped = t.reshape((shards_out, g) + tuple(t.shape[1:]))
    if role == "column":
        if t.dim() == 2:                                     # bias [n_in, out/n_in]
            return grouped.reshape(shards_out, -1)
        return grouped.permute(0, 2, 1, 3).reshape(shards_out, t.shape[1], g * t.shape[2])
    if role == "row":
        return grouped.reshape(shards_out, g * t.shape[1], t.shape[2])
    raise AssertionError(role)


def read_ckpt(pytree, dir, shards_in, shards_out=None, load_opt=True, by_role=False):
    """Loads ``shards_in`` shard directories into the structure of ``pytree``
    whose leaves carry ``shards_out`` on their leading axis (checkpoint.py:135-175).
    When the checkpoint holds no optimiser state, ``pytree['opt_state']`` is kept
    as it is (the reference retries without it, :163-175)."""
    if shards_out is None:
        shards_out = shards_in
    shards = [read_shard(f"{dir}shard_{i}/") for i in range(shards_in)]
    original_opt_state = pytree.get("opt_state") if isinstance(pytree, dict) else None

    def unshard(template):
        flat = tree_flatten(template)
        if any(len(s) != len(flat) for s in shards):
            raise AssertionError(f"Incompatible checkpoints: {len(shards[0])} leaves on disk, {len(flat)} expected")
        out = []
        for i, (path, old) in enumerate(flat):
            x = _from_numpy(np.stack([s[i] for s in shards]))
            old_shape = tuple(old.shape) if hasattr(old, "shape") else tuple(np.asarray(old).shape)
            if old_shape == ():                              # scalar kept once per process: every shard holds it
                out.append(x[0])
                continue
            if shards_out != shards_in:
                if by_role and x.dim() == 1:                 # one scalar per shard (the step counter)
                    x = x[0:1].expand(shards_out).clone()
                elif by_role and len(path) >= 2 and isinstance(path[-1], str):
                    x = reshard_by_role(path[-2], path[-1], x, shards_out)
                else:
                    x = reshard(x, old_shape)
            assert tuple(x.shape) == old_shape, f"Incompatible checkpoints {tuple(x.shape)} vs {old_shape}"
            out.append(x)
        return tree_unflatten(template, out)

    try:
        loaded = unshard(pytree)
    except AssertionError:
        if not (isinstance(pytree, dict) and pytree.get("opt_state") is not None):
            raise
        load_opt = False                                     # the checkpoint carries no optimiser state
        slim = {k: v for k, v in pytree.items() if k != "opt_state"}
        loaded = unshard(slim)
    if isinstance(loaded, dict) and (not load_opt or "opt_state" not in loaded):
        loaded["opt_state"] = original_opt_state
    return loaded
