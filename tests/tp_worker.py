"""Tensor-parallel parity worker: run under torch.distributed.run with one
process per GPU (or, with MTJ_TP_CPU=1, as gloo ranks on CPU for the host-side
helpers only).  Rank 0 prints TP_OK when everything matched the oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mesh-transformer-jax_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

from oracle import gptj_oracle as go  # noqa: E402
from oracle import spec  # noqa: E402


def cpu_checks(rank, world):
    from mesh_transformer._runtime import gather_vocab_shards
    from mesh_transformer.util import g_psum
    x = torch.full((3,), float(rank + 1))
    assert torch.equal(g_psum(x), torch.full((3,), float(sum(range(1, world + 1)))))
    assert torch.equal(x, torch.full((3,), float(rank + 1)))          # input untouched
    local = torch.arange(4, dtype=torch.float32).reshape(1, 4) + 10 * rank
    full = gather_vocab_shards(local)
    assert full.shape == (1, 4 * world) and full[0, 4 * (world - 1)].item() == 10 * (world - 1)
    from mesh_transformer.transformer_shard import _world
    assert _world() == (rank, world)


def gpu_checks(rank, world):
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    from mesh_transformer.sampling import nucleaus_sample
    from mesh_transformer.transformer_shard import CausalTransformer
    from oracle import sampling_oracle as so
    cfg = spec.tiny_config(world, seq=64)
    if world > 4:                                   # the tiny configuration has 4 heads: 8 shards need 8
        cfg = dict(cfg, d_model=512, n_heads=8)
    full = spec.full_weights(cfg, seed=5, stress=True)
    params = spec.shard_params(cfg, full)
    lens = np.array([64, 30], np.uint32)
    ctx = np.zeros((2, 64), np.uint32)
    for b in range(2):
        ctx[b, 64 - lens[b]:] = spec.token_ids(10 + b, 1, int(lens[b]), 512)[0]
    net = CausalTransformer(dict(cfg, sampler=nucleaus_sample), init_weights=False)
    net.state = {"params": params, "step": np.array(0)}
    _, out = net.generate(ctx, lens, 32, {"top_p": np.zeros(2), "temp": np.ones(2)}, return_logits=True)
    # one sequence takes the whole-step kernel with its in-kernel exchange, without the logits read-back
    _, one = net.generate(ctx[:1], lens[:1], 32, {"top_p": np.zeros(1), "temp": np.ones(1)})
    _, two = net.generate(ctx, lens, 32, {"top_p": np.zeros(2), "temp": np.ones(2)})
    for _ in range(3):                              # the same call gives the same tokens every time
        again = net.generate(ctx[:1], lens[:1], 32, {"top_p": np.zeros(1), "temp": np.ones(1)})[1][0]
        assert np.array_equal(again, one[0]), "the single-sequence decode is not reproducible"
    # nucleus sampling on gathered logits with supplied uniforms
    un = np.random.default_rng(3).random((6, 2, 512), dtype=np.float32).clip(so.TINY, None)
    opts = {"top_p": np.array([0.9, 0.6]), "temp": np.array([1.0, 0.8])}
    _, samp = net.generate(ctx, lens, 6, opts, return_logits=True, uniforms=un)
    ids = spec.token_ids(0, 2, 64, 512)
    rt = net._runtime(2, 32)
    fl = rt.forward_logits(torch.from_numpy(ids.view(np.int32)).cuda(), None, 64).cpu().numpy()
    sample = {"obs": ids[:, :-1], "target": ids[:, 1:], "ctx_length": np.array([63, 20])}
    ev = net.eval(sample)
    net._rt.check_device_status()
    if rank == 0:
        ref_net = go.CausalTransformer(cfg, params)
        _, ref = ref_net.generate(ctx, lens, 32, return_logits=True)
        rel = lambda a, b: float(np.abs(a - b).max() / np.abs(b).max())
        assert rel(out[2], ref[2]) <= 2e-2, rel(out[2], ref[2])
        assert np.array_equal(out[0], ref[0]), "greedy ids differ"
        assert np.array_equal(one[0], ref[0][:1]), "greedy ids of the single sequence differ"
        assert np.array_equal(two[0], ref[0]), "greedy ids without the logits read-back differ"
        shard = go.CausalTransformerShard(cfg, params)
        for b in range(2):
            assert rel(fl[b], shard.logits(ids[b])) <= 2e-2
        for t in range(6):
            want = so.nucleaus_sample(un[t], samp[2][:, t, 0], opts["top_p"].astype(np.float32),
                                      opts["temp"].astype(np.float32))
            assert np.array_equal(samp[0][:, t, 0], want), "sampled ids differ from the oracle sampler"
        evr = ref_net.eval(sample)
        assert np.abs(ev["all_loss"] - evr["all_loss"]).max() <= 2e-2
        assert np.abs(ev["loss"] - evr["loss"]).max() <= 1e-3
    # every rank must have produced the same tokens (replicated sampler)
    for arr in (out[0], one[0], samp[0]):
        t = torch.from_numpy(np.ascontiguousarray(arr).astype(np.int64)).cuda()
        ts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(ts, t)
        assert all(torch.equal(ts[0], x) for x in ts)
    dist.barrier()
    net.close()


def peer_loss_checks(rank, world):
    """One rank leaves between calls (it simply stops taking part): the others learn of it on the host,
    within the deadline, before they would launch anything."""
    import time
    from mesh_transformer.health import PeerLostError, PeerMonitor
    mon = PeerMonitor.from_process_group(timeout_s=1.5)
    assert mon.step() == 1 and mon.step() == 2               # everybody is there
    if rank == world - 1:
        time.sleep(4.0)                                       # stays away from call 3 (then exits normally)
        return
    t0 = time.monotonic()
    try:
        mon.step()
    except PeerLostError as e:
        assert e.missing == [world - 1] and e.step == 3
        assert 1.0 <= time.monotonic() - t0 <= 3.5
    else:
        raise AssertionError("the missing rank went unnoticed")
    if rank == 0:
        print("TP_OK", flush=True)


def main():
    if os.environ.get("MTJ_TP_CPU") == "2":
        dist.init_process_group("gloo")
        peer_loss_checks(dist.get_rank(), dist.get_world_size())
        return
    cpu = os.environ.get("MTJ_TP_CPU") == "1"
    dist.init_process_group("gloo" if cpu else "nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    (cpu_checks if cpu else gpu_checks)(rank, world)
    dist.barrier()
    if rank == 0:
        print("TP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
