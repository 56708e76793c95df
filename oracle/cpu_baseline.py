"""Timed CPU arm: the oracle's decode step (the reference's algorithm restated
in NumPy, see gptj_oracle.py) at a given model shape on the host cores.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see oracle/__init__.py).

The sample is bounded: all layers share ONE set of layer weights (fp32, larger
than any CPU cache, so the per-layer memory traffic and arithmetic are those of
distinct layers), the decode state is filled with random K/V instead of running
a prefill, and only a few decode steps are timed.  Every step does what the
reference does per token (transformer_shard.py:97-115, layers.py:316-344):
embedding, per layer LayerNorm, q/v/k projections, window shift by
concatenation, re-rotation of the whole window, attention over all seq-1 slots,
FF, and the vocabulary projection.
"""
from __future__ import annotations

import os
import time

import numpy as np

from . import gptj_oracle as go
from .spec import PREFIX


def _shared_layer_params(config: dict, seed: int = 0) -> dict:
    rng = np.random.Generator(np.random.PCG64(seed))
    d, V, L = config["d_model"], config["n_vocab"], config["layers"]

    def mat(*shape):
        return rng.standard_normal(size=(1,) + shape, dtype=np.float32) * np.float32(0.02)

    layer = {
        "replicated_layer_norm": {"scale": np.ones((1, d), np.float32), "offset": np.zeros((1, d), np.float32)},
        "linear": {"w": mat(d, d)}, "linear_1": {"w": mat(d, d)}, "linear_2": {"w": mat(d, d)},
        "linear_3": {"w": mat(d, d)},
        "linear_4": {"w": mat(d, 4 * d), "b": np.zeros((1, 4 * d), np.float32)},
        "linear_5": {"w": mat(4 * d, d), "b": np.zeros((1, d), np.float32)},
    }
    p = {PREFIX + "embedding_shard/~/linear": {"w": mat(V, d), "b": np.zeros((1, d), np.float32)}}
    for i in range(L):
        for k, v in layer.items():
            p[PREFIX + f"layer_{i}/~/{k}"] = v
    p[PREFIX + "projection_shard/~/replicated_layer_norm"] = layer["replicated_layer_norm"]
    p[PREFIX + "projection_shard/~/linear"] = {"w": mat(d, V), "b": np.zeros((1, V), np.float32)}
    return p


def decode_tokens_per_s(config: dict, steps: int = 4, warmup: int = 1, batch: int = 1,
                        threads: int | None = None) -> dict:
    """Returns {"value": tok/s, "cores": threads used, "sample": description}."""
    cfg = dict(config, cores_per_replica=1)
    threads = threads or os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits
        limiter = threadpool_limits(limits=threads)
    except Exception:        # pragma: no cover - threadpoolctl is optional
        limiter = None
    params = _shared_layer_params(cfg)
    net = go.CausalTransformerShard(cfg, params)
    W = cfg["seq"] - 1
    h, dh = cfg["n_heads"], cfg["d_model"] // cfg["n_heads"]
    rng = np.random.Generator(np.random.PCG64(1))
    kv = rng.standard_normal(size=(W, h, dh), dtype=np.float32) * np.float32(0.3)
    states = [[[{"k": kv, "v": kv, "tokens_decoded": W}] for _ in range(cfg["layers"])] for _ in range(batch)]
    tok = [np.array([rng.integers(0, cfg["n_vocab"])], np.uint32) for _ in range(batch)]

    def step():
        for b in range(batch):
            logits, states[b] = net.generate_once(tok[b], states[b])
            tok[b], _ = go.greedy_sampler(None, logits, None)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    if limiter is not None:
        limiter.restore_original_limits()
    return {
        "value": steps * batch / dt,
        "cores": threads,
        "seconds": dt,
        "sample": (f"{steps} decode steps x batch {batch} at window {W}, {cfg['layers']} layers sharing one "
                   f"fp32 layer weight set, random K/V state instead of a prefill"),
    }
