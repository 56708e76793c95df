"""lm-evaluation-harness adaptor over ``CausalTransformer.eval`` (reference:
tasks/eval_harness.py:24-88 and the masked aggregation of
mesh_transformer/TPU_cluster.py:66-114).

The tokenizer is injected (the reference builds GPT2TokenizerFast('gpt2') and
runs ftfy over the text, :15-30; neither the vocabulary files nor ftfy exist
offline): any object with ``encode(str) -> list[int]`` works, and requests may
also be given as ready token lists.  The class does not derive from
``lm_eval.base.LM`` (not installed); it offers the same three methods.
"""
from __future__ import annotations

import numpy as np

from .util import sample_batch, shrink_seq

PAD_TOKEN = 50256          # "<|endoftext|>" (tasks/eval_harness.py:19,40-41)


def process_tokens(ctx_tokens, cont_tokens, seq):
    """One (context, continuation) pair as the padded sample ``eval`` takes
    (tasks/eval_harness.py:32-46): the last ``seq`` tokens, inputs and next-token
    targets right-padded with the end-of-text id, ``eval_mask`` on the positions
    whose target is a continuation token."""
    tokens = np.asarray(list(ctx_tokens) + list(cont_tokens))[-seq:]
    n, n_cont = len(tokens), len(cont_tokens)
    obs = np.full((seq,), PAD_TOKEN, dtype=tokens.dtype)
    target = np.full((seq,), PAD_TOKEN, dtype=tokens.dtype)
    obs[:n - 1] = tokens[:-1]
    target[:n - 1] = tokens[1:]
    pos = np.arange(seq)
    return {"obs": obs, "target": target, "ctx_length": seq,
            "eval_mask": (pos > n - n_cont - 2) & (pos < n - 1)}


def process_request(x, seq, tokenizer=None, fix_text=None):
    """``x`` = (context, continuation) as text (needs ``tokenizer``) or as token lists."""
    ctx, cont = x
    if isinstance(ctx, str):
        if tokenizer is None:
            raise ValueError("text requests need a tokenizer")
        fix = fix_text if fix_text is not None else (lambda s: s)
        ctx = tokenizer.encode("<|endoftext|>" + fix(ctx))
        cont = tokenizer.encode(fix(cont))
    return process_tokens(ctx, cont, seq)


def aggregate_eval(output, eval_mask):
    """Per-example masked loss and all-correct flags plus the totals of
    TPU_cluster.py:82-114 from ``CausalTransformer.eval``'s dict."""
    mask = np.asarray(eval_mask, bool)
    hit = np.asarray(output["correct"], bool) & mask
    n_valid, n_hit = mask.sum(-1), hit.sum(-1)
    valid = n_valid > 0
    each_correct = valid & (n_valid == n_hit)
    return {
        "total": int(valid.sum()),
        "correct": int(each_correct.sum()),
        "last_correct": int(hit[:, -1].sum()),
        "last_loss": float((valid * np.asarray(output["last_loss"])).sum()),
        "mask_loss": (np.asarray(output["all_loss"]) * mask).sum(-1),
        "each_correct": each_correct,
    }


class EvalHarnessAdaptor:
    def __init__(self, network, seq, batch, shrink, min_seq=None, tokenizer=None, fix_text=None):
        self.tpu = network                 # anything with .eval(sample) -> dict of loss / all_loss / correct
        self.seq = seq
        self.batch = batch
        self.shrink = shrink
        self.min_seq = min_seq
        self.tokenizer = tokenizer
        self.fix_text = fix_text

    def greedy_until(self, requests):
        raise Exception("unimplemented")

    def loglikelihood_rolling(self, requests):
        raise Exception("unimplemented")

    def convert_requests(self, requests):
        return (process_request(r, self.seq, self.tokenizer, self.fix_text) for r in requests)

    def loglikelihood(self, requests):
        """[(log-likelihood of the continuation, continuation is the greedy choice)] per request
        (tasks/eval_harness.py:70-88).  The trailing fill samples of the last batch are dropped."""
        requests = list(requests)
        if not requests:
            return []
        zero_example = process_request(requests[0], self.seq, self.tokenizer, self.fix_text)
        output = []
        for b in sample_batch(self.convert_requests(requests), self.batch, zero_example):
            if self.shrink:
                b = shrink_seq(b, min_seq=self.min_seq)
            mask = b["eval_mask"]
            out = aggregate_eval(self.tpu.eval({k: b[k] for k in ("obs", "target", "ctx_length")}), mask)
            for loss, correct in zip(out["mask_loss"], out["each_correct"]):
                output.append((float(-loss), bool(correct)))
        return output[:len(requests)]
