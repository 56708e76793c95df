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


class ContinuousBatchingService:
    """The same ``/complete`` contract with continuous batching over the paged KV cache: a request joins the
    running decode batch at the next step (its prompt is prefilled into a free slot) and is answered as soon as
    ITS ``gen_length`` tokens exist, instead of waiting for a whole fixed batch to be gathered, padded with filler
    prompts and generated to the end (device_serve.py:143-160,183-192).  Needs the CUDA network (it drives the
    per-GPU runtime: ``start_batch`` / ``admit`` / ``decode_step``); sampling uses the device generator.

    A running batch can take ``epoch_steps`` decode steps (its position budget); the loop stops admitting when a
    new request could not finish inside the budget and opens a new batch once the active ones have drained."""

    def __init__(self, network, tokenizer, seq, slots, gen_length=256, epoch_steps=4096, seed=0):
        self.network, self.tokenizer = network, tokenizer
        self.seq, self.slots, self.gen_length = seq, slots, gen_length
        self.epoch_steps = max(epoch_steps, gen_length + 1)
        self.seed = seed
        self.requests_queue: Queue = Queue()
        self._stop = threading.Event()
        self.steps_taken = 0            # decode steps over the service's life (for tests / monitoring)
        self.admitted = 0

    def complete(self, content: dict) -> dict:
        if self.requests_queue.qsize() > MAX_PENDING:
            return {"error": "queue full, try again later"}
        response_queue: Queue = Queue()
        self.requests_queue.put(({"context": content["context"], "top_p": float(content["top_p"]),
                                  "temp": float(content["temp"])}, response_queue))
        return {"completion": response_queue.get()}

    def serve_forever(self, poll_s=0.002):
        import torch
        rt = self.network._runtime(self.slots, self.epoch_steps)
        dev = rt.device
        with torch.cuda.device(dev):
            top_p = torch.ones((self.slots,), dtype=torch.float32, device=dev)
            temp = torch.ones((self.slots,), dtype=torch.float32, device=dev)
            tok = torch.empty((self.slots,), dtype=torch.int32, device=dev)
            active = {}                  # slot -> [response queue, produced ids]
            epoch_left = 0
            while not self._stop.is_set():
                if epoch_left <= 0 and not active:
                    rt.set_seed(self.seed + self.steps_taken)
                    rt.start_batch(self.slots)
                    epoch_left = self.epoch_steps
                # admit waiting requests into free slots while the batch can still finish them
                while len(active) < self.slots and epoch_left > self.gen_length:
                    try:
                        req, q = self.requests_queue.get(block=False)
                    except Empty:
                        break
                    try:
                        ids = list(self.tokenizer.encode(req["context"]))[-self.seq:]
                    except Exception:                             # device_serve.py:178-179
                        print("oops exception")
                        ids = []
                    if not ids:
                        ids = [0]
                    slot = next(i for i in range(self.slots) if i not in active)
                    prompt = torch.tensor(ids, dtype=torch.int32, device=dev)
                    rt.admit(slot, prompt)
                    top_p[slot] = req["top_p"]
                    temp[slot] = req["temp"]
                    active[slot] = [q, []]
                    self.admitted += 1
                if not active:
                    if epoch_left <= self.gen_length:
                        epoch_left = 0                            # nothing left to drain: open a new batch
                        continue
                    time.sleep(poll_s)
                    continue
                rt.decode_step(None, tok, None, greedy=False, top_p=top_p, temp=temp, uniforms=None)
                epoch_left -= 1
                self.steps_taken += 1
                new = tok.cpu().numpy().view(np.uint32)
                for slot in list(active):
                    q, out = active[slot]
                    out.append(int(new[slot]))
                    if len(out) == self.gen_length:
                        q.put(self.tokenizer.decode(np.asarray(out, np.uint32)))
                        del active[slot]
            rt.check_device_status()

    def stop(self):
        self._stop.set()
