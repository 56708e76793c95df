"""Helpers that lay synthetic K/V out in the library's paged cache format."""
import ctypes

import numpy as np

PAGE = 64


def build_paged_kv(rng, batch, heads, d_head, ring_pages, positions):
    """Random K/V for absolute positions [lo, hi) per sequence, written into
    pools [pages][heads][64][d_head] through a shuffled page table with ring
    addressing: slot = (pos // 64) % ring_pages."""
    import torch
    n_pages = batch * ring_pages
    table = rng.permutation(n_pages).astype(np.int32).reshape(batch, ring_pages)
    kpool = np.zeros((n_pages, heads, PAGE, d_head), np.float32)
    vpool = np.zeros_like(kpool)
    keys, vals = [], []
    for b, (lo, hi) in enumerate(positions):
        k = rng.standard_normal((hi - lo, heads, d_head)).astype(np.float32)
        v = rng.standard_normal((hi - lo, heads, d_head)).astype(np.float32)
        k = torch.from_numpy(k).to(torch.bfloat16).float().numpy()
        v = torch.from_numpy(v).to(torch.bfloat16).float().numpy()
        for i, pos in enumerate(range(lo, hi)):
            page = table[b, (pos // PAGE) % ring_pages]
            kpool[page, :, pos % PAGE] = k[i]
            vpool[page, :, pos % PAGE] = v[i]
        keys.append(k)
        vals.append(v)
    return table, kpool, vpool, keys, vals


def attention_reference(q, keys, vals, d_head):
    """softmax(q.k / sqrt(d_head)) . v per head, fp32 (layers.py:275-283)."""
    logits = np.einsum("hd,thd->ht", q, keys) / np.float32(np.sqrt(d_head))
    logits = logits - logits.max(-1, keepdims=True)
    w = np.exp(logits)
    w = w / w.sum(-1, keepdims=True)
    return np.einsum("ht,thd->hd", w, vals).astype(np.float32)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())
