"""Request queue -> batch -> ``network.generate`` serving loop of the reference
(device_serve.py:46-66 the ``/complete`` handler, :138-194 the loop), without the
HTTP layer: ``CompletionService.complete(content)`` is the body of the POST
handler (same JSON in, same JSON out), ``serve_once`` is one turn of the loop.

The tokenizer is injected (``encode(str) -> list[int]``, ``decode(ids) -> str``);
the reference uses GPT2TokenizerFast('gpt2') (:136), whose files are not
available offline.  Mount ``complete`` under any web framework, e.g.
``app.post("/complete")(lambda body: service.complete(body))``.
"""
from __future__ import annotations

import threading
import time
from queue import Empty, Queue

import numpy as np

MAX_PENDING = 100          # device_serve.py:53
FILLER_CONTEXT = "whatever"  # device_serve.py:158


def pad_context(tokens, seq):
    """Left-pads (or keeps the last ``seq`` of) a token list; returns (uint32 [seq], length) as
    device_serve.py:169-177 does -- the length is the untruncated token count."""
    tokens = list(tokens)
    padded = np.zeros(seq, np.uint32)
    kept = tokens[-seq:]
    if kept:
        padded[seq - len(kept):] = np.asarray(kept, np.uint32)
    return padded, len(tokens)


class CompletionService:
    def __init__(self, network, tokenizer, seq, total_batch, gen_length=256):
        self.network, self.tokenizer = network, tokenizer
        self.seq, self.total_batch, self.gen_length = seq, total_batch, gen_length
        self.requests_queue: Queue = Queue()
        self._stop = threading.Event()

    # ---- the POST /complete body (device_serve.py:46-64) ----
    def complete(self, content: dict) -> dict:
        if self.requests_queue.qsize() > MAX_PENDING:
            return {"error": "queue full, try again later"}
        response_queue: Queue = Queue()
        self.requests_queue.put(({"context": content["context"], "top_p": float(content["top_p"]),
                                  "temp": float(content["temp"])}, response_queue))
        return {"completion": response_queue.get()}

    # ---- one turn of the loop (device_serve.py:138-194) ----
    def gather(self, poll_s=0.01):
        """Up to ``total_batch`` queued requests; waits until there is at least one."""
        batch = []
        while len(batch) < self.total_batch and not self._stop.is_set():
            try:
                batch.append(self.requests_queue.get(block=False))
            except Empty:
                if batch:
                    break
                time.sleep(poll_s)
        return batch

    def serve_once(self, poll_s=0.01) -> int:
        batch = self.gather(poll_s)
        if not batch:
            return 0
        contexts = [o["context"] for o, _ in batch]
        top_p = [o["top_p"] for o, _ in batch]
        temp = [o["temp"] for o, _ in batch]
        fill = self.total_batch - len(batch)
        contexts += [FILLER_CONTEXT] * fill
        top_p += [1] * fill
        temp += [1] * fill
        tokenized, lengths = [], []
        for ctx in contexts:
            padded, length = np.zeros(self.seq, np.uint32), 0
            try:
                padded, length = pad_context(self.tokenizer.encode(ctx), self.seq)
            except Exception:                                    # device_serve.py:178-179: the slot stays empty
                print("oops exception")
            tokenized.append(padded)
            lengths.append(length)
        # the reference passes the raw token count on (0 after a tokeniser failure, > seq for long prompts);
        # libmtj_b200 rejects lengths outside [1, seq], so they are clamped to what the padded row holds
        lengths = np.clip(np.array(lengths), 1, self.seq)
        output = self.network.generate(np.array(tokenized), lengths, self.gen_length,
                                       {"top_p": np.array(top_p), "temp": np.array(temp)})
        for ids, (_, q) in zip(output[1][0][:, :, 0], batch):
            q.put(self.tokenizer.decode(ids))
        return len(batch)

    def serve_forever(self):
        while not self._stop.is_set():
            self.serve_once()

    def stop(self):
        self._stop.set()
