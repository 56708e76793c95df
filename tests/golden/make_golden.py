"""Generates tests/golden/tiny_gptj.npz.

The reference (JAX/Haiku, jax 0.2.12) cannot be imported without jax, so these
vectors come from the CPU oracle (oracle/gptj_oracle.py, oracle/sampling_oracle.py),
whose model part is cross-checked against transformers' GPTJForCausalLM in
tests/test_oracle_model.py.  They pin the oracle against accidental change and
give the CUDA path a fixed target.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import gptj_oracle as go  # noqa: E402
from oracle import sampling_oracle as so  # noqa: E402
from oracle import spec  # noqa: E402


def main():
    cfg = spec.tiny_config(1, seq=128)
    params = spec.make_params(cfg, seed=0, stress=False)        # the tiny CPU-parity configuration: N(0, 0.02), LN 1/0, biases 0
    ids = spec.token_ids(0, 2, 128, 512)                        # uniform ids [2, 128]
    net = go.CausalTransformer(cfg, params)
    logits = np.stack([net._shard().logits(ids[b]) for b in range(2)])
    ev = net.eval({"obs": ids[:, :-1], "target": ids[:, 1:]})
    # 32-step greedy decode with KV cache from a left-padded 96-token prompt and from a full window
    lens = np.array([96, 128], np.uint32)
    ctx = np.zeros((2, 128), np.uint32)
    for b in range(2):
        ctx[b, 128 - lens[b]:] = ids[b, :lens[b]]
    _, gen = net.generate(ctx, lens, 32, return_logits=True)
    # sampler vectors
    rng = np.random.default_rng(7)
    s_logits = (rng.standard_normal((4, 512)) * 2).astype(np.float32)
    s_unif = rng.random((4, 512), dtype=np.float32).clip(so.TINY, None)
    s_top_p = np.array([0.9, 0.5, 0.0, 1.0], np.float32)
    s_temp = np.array([1.0, 0.75, 1.0, 1.5], np.float32)
    s_tokens = so.nucleaus_sample(s_unif, s_logits, s_top_p, s_temp)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_gptj.npz")
    np.savez_compressed(
        out, ids=ids, logits_last8=logits[:, -8:, :].astype(np.float32), logits_pos=logits[:, ::16, :64].astype(np.float32),
        all_loss=ev["all_loss"], correct=ev["correct"], ctx=ctx, lens=lens,
        greedy_tokens=gen[0], greedy_logits_first=gen[2][:, 0, 0, :].astype(np.float32),
        s_logits=s_logits, s_unif=s_unif, s_top_p=s_top_p, s_temp=s_temp, s_tokens=s_tokens)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
