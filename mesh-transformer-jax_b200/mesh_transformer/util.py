"""Dtype casts and "shard"-axis collectives of the reference's util.py
(forward semantics only: util.py:87-96,100-147,176-178)."""
from __future__ import annotations

import numpy as np
import torch


def _map_leaves(fn, tree):
    if isinstance(tree, dict):
        return {k: _map_leaves(fn, v) for k, v in tree.items()}
    if isinstance(tree, (list, tuple)):
        return type(tree)(_map_leaves(fn, v) for v in tree)
    return fn(tree)


def to_bf16(t):
    """fp32 leaves -> bf16, everything else untouched (util.py:91-92).
    NumPy has no bf16, so fp32 NumPy leaves become torch bf16 tensors."""
    def cast(x):
        if isinstance(x, torch.Tensor):
            return x.to(torch.bfloat16) if x.dtype == torch.float32 else x
        if isinstance(x, np.ndarray) and x.dtype == np.float32 and x.ndim > 0:
            return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16)
        return x
    return _map_leaves(cast, t)


def to_f32(t):
    """bf16 leaves -> fp32 (util.py:87-88)."""
    def cast(x):
        if isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16:
            return x.to(torch.float32)
        return x
    return _map_leaves(cast, t)


def f_psum(x):
    """Identity in the forward pass (util.py:100-103)."""
    return x


def g_psum(x: torch.Tensor) -> torch.Tensor:
    """All-reduce sum over the shard axis (util.py:133-136)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        x = x.clone()
        dist.all_reduce(x)
    return x


def head_print(*args, **kwargs):
    """Print on the first process only (util.py:176-178)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0:
        print(*args, **kwargs)
