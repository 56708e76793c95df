"""The callers and formats either side of the path, driven over the CUDA network (not the oracle):
the serving loop (device_serve.py:138-194), the lm-eval adaptor (tasks/eval_harness.py:24-88) and the
Hugging Face interchange (to_hf_weights.py:160-449)."""
import threading

import numpy as np
import pytest

from oracle import gptj_oracle as go
from oracle import spec

pytestmark = pytest.mark.gpu


def _net(cfg, params, cuda_device):
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer.transformer_shard import CausalTransformer
    net = CausalTransformer(dict(cfg), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    return net


class ByteTokenizer:
    def encode(self, text):
        if text == "boom":
            raise ValueError("cannot tokenise")
        return [b for b in text.encode("utf-8")]

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)


def test_completion_service_with_concurrent_clients(cuda_device):
    """Six clients post at once, the loop batches them four at a time (one full batch, one filled up with the
    filler prompt), and every greedy completion equals a direct greedy generate of the oracle."""
    import serve
    from mesh_transformer.sampling import nucleaus_sample
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=3, stress=True)
    net = _net(dict(cfg, sampler=nucleaus_sample), params, cuda_device)
    tok = ByteTokenizer()
    svc = serve.CompletionService(net, tok, seq=64, total_batch=4, gen_length=6)
    reqs = [{"context": c, "top_p": 0.0, "temp": 1.0} for c in
            ("hello world", "abc", "boom", "the quick brown fox jumps over the lazy dog " * 3, "x", "tensor parallel")]
    reqs.append({"context": "sampled", "top_p": 0.9, "temp": 0.8})
    answers = [None] * len(reqs)

    def client(i):
        answers[i] = svc.complete(reqs[i])

    clients = [threading.Thread(target=client, args=(i,)) for i in range(len(reqs))]
    for c in clients:
        c.start()
    served = 0
    while served < len(reqs):
        served += svc.serve_once()
    for c in clients:
        c.join(timeout=60)
    assert all(a is not None and "completion" in a for a in answers)
    ref = go.CausalTransformer(cfg, params)
    for i, r in enumerate(reqs[:-1]):
        if r["context"] == "boom":
            continue
        padded, n = serve.pad_context(tok.encode(r["context"]), 64)
        out = ref.generate(padded[None], np.array([min(n, 64)]), 6)
        assert answers[i]["completion"] == tok.decode(out[1][0][0, :, 0]), r["context"]
    assert len(answers[-1]["completion"].split()) == 6
    net.close()


def test_eval_harness_adaptor_over_the_cuda_network(cuda_device):
    """loglikelihood() of (context, continuation) requests: masked log-likelihoods within the loss tolerance of
    the oracle network's, the all-correct flags equal except where the oracle's own top-2 logits are a near-tie."""
    from tasks import eval_harness as eh
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=9, stress=True)
    net = _net(cfg, params, cuda_device)
    rng = np.random.default_rng(5)
    reqs = []
    for _ in range(11):
        nc, nk = int(rng.integers(1, 90)), int(rng.integers(1, 7))
        reqs.append((rng.integers(0, 512, nc).tolist(), rng.integers(0, 512, nk).tolist()))
    for shrink in (False, True):
        got = eh.EvalHarnessAdaptor(net, seq=64, batch=4, shrink=shrink, min_seq=16).loglikelihood(reqs)
        want = eh.EvalHarnessAdaptor(go.CausalTransformer(cfg, params), seq=64, batch=4, shrink=shrink,
                                     min_seq=16).loglikelihood(reqs)
        assert len(got) == len(reqs)
        for (gl, gc), (wl, wc), (_, cont) in zip(got, want, reqs):
            assert abs(gl - wl) <= 2e-2 * len(cont)
        assert sum(gc != wc for (_, gc), (_, wc) in zip(got, want)) <= 1
    net.close()


def test_hf_state_dict_through_the_cuda_path_matches_transformers(cuda_device):
    """A Hugging Face GPT-J state dict -> from_hf_state_dict -> CUDA logits, against GPTJForCausalLM itself
    run in fp32 on the CPU with the same weights."""
    import torch
    tr = pytest.importorskip("transformers")
    from mesh_transformer.hf_interchange import from_hf_state_dict, hf_config
    cfg = spec.tiny_config(1, seq=64)
    hc = hf_config(cfg, torch.float32)
    conf = tr.GPTJConfig(vocab_size=hc["vocab_size"], n_positions=hc["n_positions"], n_embd=hc["n_embd"],
                         n_layer=hc["n_layer"], n_head=hc["n_head"], rotary_dim=hc["rotary_dim"],
                         activation_function=hc["activation_function"], layer_norm_epsilon=hc["layer_norm_epsilon"],
                         attn_pdrop=0.0, embd_pdrop=0.0, resid_pdrop=0.0)
    torch.manual_seed(0)
    model = tr.GPTJForCausalLM(conf).float().eval()
    with torch.no_grad():
        for name, p in model.named_parameters():            # bf16-exact weights: the library stores bf16
            if p.dim() > 1:
                p.copy_(p.to(torch.bfloat16).float())
            else:
                p.copy_((p + 0.05 * torch.randn_like(p)).to(torch.bfloat16).float())
    params = from_hf_state_dict(model.state_dict(), cfg)
    net = _net(cfg, params, cuda_device)
    ids = spec.token_ids(0, 2, 64, 512)
    rt = net._runtime(2, 8)
    got = rt.forward_logits(torch.from_numpy(ids.view(np.int32)).to(cuda_device), None, 64).cpu().numpy()
    with torch.no_grad():
        want = model(torch.tensor(ids.astype(np.int64))).logits.numpy()
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()
    ctx = spec.left_pad(ids[:1, :40], 64)
    toks = net.generate(ctx, [40], 8, {"top_p": np.zeros(1), "temp": np.ones(1)})[1][0][0, :, 0]
    seq_ids = torch.tensor(ids[:1, :40].astype(np.int64))
    with torch.no_grad():
        hf = model.generate(seq_ids, max_new_tokens=8, do_sample=False, pad_token_id=0)[0, 40:].numpy()
    assert np.array_equal(toks, hf.astype(np.uint32))
    net.close()


def test_continuous_batching_service(cuda_device):
    """Requests join a running decode batch at step granularity (mtj_start_batch / mtj_admit): three slots, eight
    requests arriving while others are being decoded, a position budget small enough to force a second batch.
    Every greedy completion equals the oracle's greedy generate of the same left-padded prompt -- a sequence
    admitted in mid-flight sits at shifted absolute positions, which changes nothing (rotary attention depends on
    distances only)."""
    import time
    import serve
    from mesh_transformer.sampling import nucleaus_sample
    cfg = spec.tiny_config(1, seq=64)
    params = spec.make_params(cfg, seed=13, stress=True)
    net = _net(dict(cfg, sampler=nucleaus_sample), params, cuda_device)
    tok = ByteTokenizer()
    gen = 8
    svc = serve.ContinuousBatchingService(net, tok, seq=64, slots=3, gen_length=gen, epoch_steps=30)
    texts = ["hello world", "abc", "the quick brown fox jumps over the lazy dog " * 3, "x", "tensor parallel",
             "paged key value cache", "boom", "zz top"]
    reqs = [{"context": c, "top_p": 0.0, "temp": 1.0} for c in texts]
    reqs[3] = {"context": "x", "top_p": 0.9, "temp": 0.8}                 # one sampled request among the greedy ones
    answers = [None] * len(reqs)

    def client(i):
        time.sleep(0.01 * i)                                              # arrivals spread over the decode steps
        answers[i] = svc.complete(reqs[i])

    worker = threading.Thread(target=svc.serve_forever, daemon=True)
    clients = [threading.Thread(target=client, args=(i,)) for i in range(len(reqs))]
    worker.start()
    for c in clients:
        c.start()
    for c in clients:
        c.join(timeout=120)
    svc.stop()
    worker.join(timeout=30)
    assert all(a is not None and "completion" in a for a in answers)
    assert svc.admitted == len(reqs)
    # fixed batches of three would take 3 x 8 steps only if all requests were there at the start and no batch
    # had to be padded; here nothing waits for a batch to fill and no slot decodes a filler prompt to the end
    assert svc.steps_taken <= len(reqs) * gen
    ref = go.CausalTransformer(cfg, params)
    for i, r in enumerate(reqs):
        if r["top_p"] != 0.0:
            assert len(answers[i]["completion"].split()) == gen
            continue
        ids = tok.encode(r["context"]) if r["context"] != "boom" else [0]
        padded, n = serve.pad_context(ids, 64)
        out = ref.generate(padded[None], np.array([min(n, 64)]), gen)
        assert answers[i]["completion"] == tok.decode(out[1][0][0, :, 0]), r["context"]
    net.close()
