"""Serving loop (queue -> batch -> generate) against the oracle network, no HTTP."""
import os
import sys
import threading

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "mesh-transformer-jax_b200"))

from oracle import gptj_oracle as go  # noqa: E402
from oracle import spec  # noqa: E402
import serve  # noqa: E402


class ByteTokenizer:
    def encode(self, text):
        if text == "boom":
            raise ValueError("cannot tokenise")
        return [b for b in text.encode("utf-8")]

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)


def test_pad_context_follows_the_reference_rule():
    seq = 8
    for toks in ([], [5], [1, 2, 3], list(range(8)), list(range(20))):
        padded, n = serve.pad_context(toks, seq)
        pad_amount = max(seq - len(toks), 0)                        # device_serve.py:171-175
        want = np.pad(np.asarray(toks, np.int64), ((pad_amount, 0),)).astype(np.uint32)[-seq:]
        assert np.array_equal(padded, want) and n == len(toks)


def test_requests_are_batched_generated_and_answered():
    cfg = spec.tiny_config(1, seq=64)
    net = go.CausalTransformer(cfg, spec.make_params(cfg, seed=3))
    tok = ByteTokenizer()
    svc = serve.CompletionService(net, tok, seq=64, total_batch=4, gen_length=5)
    worker = threading.Thread(target=svc.serve_forever, daemon=True)
    reqs = [{"context": "hello world", "top_p": 0.0, "temp": 1.0}, {"context": "abc", "top_p": 0, "temp": 0.75},
            {"context": "boom", "top_p": 0.0, "temp": 1.0}]
    answers = [None] * len(reqs)

    def client(i):
        answers[i] = svc.complete(reqs[i])

    clients = [threading.Thread(target=client, args=(i,)) for i in range(len(reqs))]
    for c in clients:
        c.start()
    worker.start()
    for c in clients:
        c.join(timeout=120)
    svc.stop()
    assert all(a is not None and "completion" in a for a in answers)
    # top_p = 0 keeps only the arg-max: the completion equals a direct greedy generate of the same prompt
    for i in (0, 1):
        padded, n = serve.pad_context(tok.encode(reqs[i]["context"]), 64)
        out = net.generate(padded[None], np.array([n]), 5, {"top_p": np.zeros(1), "temp": np.ones(1)})
        assert answers[i]["completion"] == tok.decode(out[1][0][0, :, 0])


def test_full_queue_is_refused():
    svc = serve.CompletionService(None, ByteTokenizer(), seq=8, total_batch=2)
    for _ in range(serve.MAX_PENDING + 1):
        svc.requests_queue.put(({}, None))
    assert svc.complete({"context": "x", "top_p": 1, "temp": 1}) == {"error": "queue full, try again later"}
