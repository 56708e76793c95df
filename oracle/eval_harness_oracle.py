"""Restatement of the reference's lm-eval adaptor arithmetic in NumPy: request ->
padded sample (tasks/eval_harness.py:24-46), sequence shrinking and batching
(tasks/util.py:13-61) and the masked aggregation of the eval result
(mesh_transformer/TPU_cluster.py:66-114).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the
reference has no test for these functions and lm_eval / ftfy / the GPT-2
tokenizer files are absent here, so tokenisation is outside this restatement
(it starts from token lists).
"""
from __future__ import annotations

from itertools import zip_longest

import numpy as np


def process_tokens(ctx_tokens, cont_tokens, seq):
    """tasks/eval_harness.py:32-46 from the two token lists on."""
    all_tokens = list(ctx_tokens) + list(cont_tokens)
    all_tokens = np.array(all_tokens)[-seq:]
    provided_ctx = len(all_tokens) - 1
    pad_amount = seq - provided_ctx
    return {
        "obs": np.pad(all_tokens[:-1], ((0, pad_amount),), constant_values=50256),
        "target": np.pad(all_tokens[1:], ((0, pad_amount),), constant_values=50256),
        "ctx_length": seq,
        "eval_mask": np.logical_and(np.arange(0, seq) > len(all_tokens) - len(cont_tokens) - 2,
                                    np.arange(0, seq) < len(all_tokens) - 1),
    }


def shrink_seq(examples, min_seq=None):
    """tasks/util.py:13-31."""
    length = examples["obs"].shape[-1]
    new_length = length // 2
    if min_seq is not None and new_length < min_seq:
        return examples
    max_length = np.max(examples["eval_mask"] * np.arange(0, length)) + 1
    if max_length < new_length:
        examples = dict(examples)
        for k in ("obs", "target", "eval_mask"):
            examples[k] = examples[k][:, :new_length]
        return shrink_seq(examples, min_seq=min_seq)
    return examples


def sample_batch(examples, bs, zero_example_shape):
    """tasks/util.py:34-61."""
    zero = {"obs": np.zeros_like(zero_example_shape["obs"]), "target": np.zeros_like(zero_example_shape["target"]),
            "eval_mask": np.zeros_like(zero_example_shape["eval_mask"]), "ctx_length": 0}
    args = [iter(examples)] * bs
    for batch in zip_longest(fillvalue=zero, *args):
        yield {k: np.array([s[k] for s in batch]) for k in ("obs", "target", "eval_mask", "ctx_length")}


def aggregate(output, eval_mask):
    """TPU_cluster.py:82-114 for one node's output."""
    correct_and_valid = np.logical_and(output["correct"], eval_mask)
    correct_tokens_count = np.sum(correct_and_valid, -1)
    valid_tokens_count = np.sum(eval_mask, -1)
    correct_example = np.logical_and(valid_tokens_count == correct_tokens_count, valid_tokens_count > 0)
    valid_example = valid_tokens_count > 0
    return {
        "total": sum(valid_example),
        "correct": sum(correct_example),
        "last_correct": sum(correct_and_valid[:, -1]),
        "last_loss": sum(valid_example * output["last_loss"]),
        "mask_loss": np.array(np.sum(output["all_loss"] * eval_mask, -1).tolist()),
        "each_correct": np.array(correct_example.tolist()),
    }
