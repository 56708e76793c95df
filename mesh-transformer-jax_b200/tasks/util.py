"""Batching helpers of the lm-eval adaptor (reference: tasks/util.py:6-61)."""
from __future__ import annotations

import numpy as np

_KEYS = ("obs", "target", "eval_mask")


def grouper(n, iterable, fillvalue):
    """grouper(3, 'ABCDEFG', 'x') -> ABC DEF Gxx (tasks/util.py:6-9)."""
    group = []
    for item in iterable:
        group.append(item)
        if len(group) == n:
            yield tuple(group)
            group = []
    if group:
        yield tuple(group + [fillvalue] * (n - len(group)))


def shrink_seq(examples, min_seq=None):
    """Halves the sequence axis while no evaluated position would be cut off
    (tasks/util.py:13-31); never goes below ``min_seq``."""
    length = examples["obs"].shape[-1]
    last_needed = int(np.max(examples["eval_mask"] * np.arange(length))) + 1
    new_length = length
    while True:
        half = new_length // 2
        if (min_seq is not None and half < min_seq) or not last_needed < half:
            break
        new_length = half
    if new_length != length:
        for k in _KEYS:
            examples[k] = examples[k][:, :new_length]
    return examples


def sample_batch(examples, bs, zero_example_shape):
    """Batches of ``bs`` samples, the last one filled with all-zero samples whose
    ctx_length is 0 (tasks/util.py:34-61)."""
    filler = {k: np.zeros_like(zero_example_shape[k]) for k in _KEYS}
    filler["ctx_length"] = 0
    for batch in grouper(bs, examples, filler):
        yield {k: np.array([s[k] for s in batch]) for k in _KEYS + ("ctx_length",)}
