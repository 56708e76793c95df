"""Samplers of the reference's sampling.py on the B200 path.

``nucleaus_sample`` / ``softmax_sample`` keep the reference signature
``(key, logits, sampler_input, **options) -> (token, info)``
(sampling.py:6-7,41-44).  ``key`` is what the randomness comes from: a float32
tensor of pre-drawn uniforms in [tiny, 1) with the shape of ``logits`` (the
form the parity tests use), a ``torch.Generator``, or an int seed.  The
arithmetic runs in libmtj_b200's sampling kernel (``nucleaus_filter`` returns
the kernel's own selection); the top-k branch of the reference filter
(sampling.py:15-26) is not implemented.
"""
from __future__ import annotations

import numpy as np
import torch

from ._lib import check, lib

TINY = float(np.finfo(np.float32).tiny)


def draw_uniforms(key, shape, device) -> torch.Tensor:
    """Uniforms in [tiny, 1) like jax.random.gumbel's input (minval=tiny)."""
    if isinstance(key, torch.Tensor):
        return key.to(device=device, dtype=torch.float32).contiguous()
    if isinstance(key, torch.Generator):
        gen = key
    else:
        gen = torch.Generator(device=device)
        gen.manual_seed(int(key) & ((1 << 63) - 1))
    u = torch.rand(shape, generator=gen, device=device, dtype=torch.float32)
    return u.clamp_(min=TINY)


def _per_row(value, rows, device):
    t = torch.as_tensor(np.asarray(value, dtype=np.float32)).reshape(-1)
    if t.numel() == 1:
        t = t.expand(rows)
    return t.to(device).contiguous()


def _per_row_int(value, rows, device):
    """None stays None (the reference's top_k = None); a scalar or [rows] becomes an int32 device tensor."""
    if value is None:
        return None
    t = torch.as_tensor(np.asarray(value, dtype=np.int64).clip(-2**31, 2**31 - 1).astype(np.int32)).reshape(-1)
    if t.numel() == 1:
        t = t.expand(rows)
    return t.to(device).contiguous()


def nucleaus_sample(key, logits, _=None, top_p=0.9, temp=1, top_k=None):
    """logits [rows, vocab] (CUDA tensor or array) -> (uint32 token ids [rows], None)."""
    if not isinstance(logits, torch.Tensor):
        logits = torch.as_tensor(np.asarray(logits, dtype=np.float32))
    if not logits.is_cuda:
        logits = logits.cuda()
    logits = logits.to(torch.float32).contiguous()
    rows, vocab = logits.shape
    dev = logits.device
    with torch.cuda.device(dev):
        u = draw_uniforms(key, (rows, vocab), dev)
        tp, tt, tk = _per_row(top_p, rows, dev), _per_row(temp, rows, dev), _per_row_int(top_k, rows, dev)
        nbytes = lib.mtj_sample_scratch_bytes(rows, vocab)
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
        out = torch.empty((rows,), dtype=torch.int32, device=dev)
        check(lib.mtj_sample_top_p(logits.data_ptr(), u.data_ptr(), tp.data_ptr(),
                                   tk.data_ptr() if tk is not None else None, tt.data_ptr(), rows, vocab,
                                   scratch.data_ptr(), nbytes, out.data_ptr(),
                                   torch.cuda.current_stream(dev).cuda_stream))
        return out.cpu().numpy().view(np.uint32), None


def softmax_sample(key, logits, _=None, temp=1):
    """sampling.py:6-7: categorical(logits / temp), i.e. no nucleus filter."""
    return nucleaus_sample(key, logits, None, top_p=float("inf"), temp=temp)


def nucleaus_filter(logits, top_p=0.9, top_k=None):
    """sampling.py:10-38: ``logits - 1e10 * removed`` as a CUDA tensor [rows, vocab]; with ``top_k`` also
    ``- 1e10 * index`` for the entries of sorted rank >= top_k (:15-26)."""
    if not isinstance(logits, torch.Tensor):
        logits = torch.as_tensor(np.asarray(logits, dtype=np.float32))
    if not logits.is_cuda:
        logits = logits.cuda()
    logits = logits.to(torch.float32).contiguous()
    rows, vocab = logits.shape
    dev = logits.device
    with torch.cuda.device(dev):
        out = torch.empty_like(logits)
        tp, tk = _per_row(top_p, rows, dev), _per_row_int(top_k, rows, dev)
        check(lib.mtj_nucleus_filter(logits.data_ptr(), tp.data_ptr(), tk.data_ptr() if tk is not None else None,
                                     rows, vocab, out.data_ptr(),
                                     torch.cuda.current_stream(dev).cuda_stream))
        return out
