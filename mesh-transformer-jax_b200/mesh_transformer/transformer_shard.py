"""Host-side mirror of the reference's model runtime API for the GPT-J path.

``CausalTransformer`` keeps the constructor, ``state`` dict, ``eval``,
``generate``, ``move_xmap``, ``write_ckpt``/``load_ckpt`` surface of
mesh_transformer/transformer_shard.py:118-339 of the reference; the work runs
in libmtj_b200's CUDA kernels on one GPU per shard (one process per GPU, the
"shard" axis being the torch.distributed world).  Training (``train``) and the
pjit "V2" model are outside this path.
"""
from __future__ import annotations

import random
import time

import numpy as np
import torch

from ._runtime import PREFIX, ShardRuntime, param_shapes, validate_config
from .util import head_print, to_bf16


def _world():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class CausalTransformerShard:
    """Per-shard program (transformer_shard.py:21-115) bound to one GPU."""

    def __init__(self, config, runtime: ShardRuntime | None = None, **runtime_kw):
        validate_config(config)
        self.config = config
        self.heads = config["n_heads"]
        self.heads_per_shard = config["n_heads"] // config["cores_per_replica"]
        self.runtime = runtime if runtime is not None else ShardRuntime(config, **runtime_kw)

    def generate_initial(self, context_dev: torch.Tensor, length):
        """Prefill context[:, :-1]; the last token is held back for the first
        decode step (transformer_shard.py:74-95).  The reference also returns
        the prefill logits, which its caller discards (:196); they are not
        computed here."""
        self.runtime.prefill(context_dev, length)

    def generate_once(self, new_tok_dev=None, tokens_out=None, logits_out=None, **sampler):
        """One decode step over all layers plus the sampler
        (transformer_shard.py:97-115,198-210)."""
        self.runtime.decode_step(new_tok_dev, tokens_out, logits_out, **sampler)

    def generate_scan(self, gen_length, tokens_out=None, logits_out=None, **sampler):
        """The ``lax.scan`` over generate_once + sampler (transformer_shard.py:198-212): all steps are enqueued
        by one library call, the sampled token feeding the next step on the device."""
        self.runtime.generate_steps(gen_length, tokens_out, logits_out, **sampler)


class CausalTransformer:
    def __init__(self, config, device=None, init_weights: bool = True):
        self.config = config
        validate_config(config)
        rank, world = _world()
        # transformer_shard.py:257 -- the mesh's mp size must match the config
        assert world == config["cores_per_replica"], \
            "run one process per shard: world size must equal cores_per_replica"
        self.rank = rank
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.gen_length = 1
        self.return_logits = False
        self._rt: ShardRuntime | None = None
        self._rt_caps = (0, 0)
        self._dirty = True
        self._state = None
        self.last_generate_timing = None
        # optional host-side liveness check of the shard group before every tensor-parallel call
        # (config key "mtj_peer_timeout_s", seconds; see health.py)
        self._monitor = None
        if world > 1 and config.get("mtj_peer_timeout_s"):
            from .health import PeerMonitor
            self._monitor = PeerMonitor.from_process_group(float(config["mtj_peer_timeout_s"]))
        if init_weights:
            self.state = self._init_state(seed=42)
            n = sum(int(np.prod(v.shape)) for m in self._state["params"].values() for v in m.values())
            head_print(f"Total parameters: {n * config['cores_per_replica'] // 1}")

    # -- state ---------------------------------------------------------------
    @property
    def state(self):
        return self._state

    @state.setter
    def state(self, value):
        self._state = value
        self._dirty = True

    def _init_state(self, seed: int):
        """Random initialisation with the reference's scales (layers.py:185,
        253-258; transformer_shard.py:35): truncated normal, std 1/sqrt(fan_in)
        for plain Linears, 1/sqrt(n_vocab) for the table, (2/layers)/sqrt(d)
        for the two output projections; LN scale 1, everything else 0.  Leaves
        carry a leading axis holding this process's shard."""
        cfg = self.config
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed + 1000 * self.rank)
        dtype = torch.bfloat16 if "early_cast" in cfg else torch.float32
        d, L = cfg["d_model"], cfg["layers"]

        def tn(shape, std):
            t = torch.empty((1,) + tuple(shape), dtype=torch.float32, device=self.device)
            torch.nn.init.trunc_normal_(t, mean=0.0, std=std, a=-2 * std, b=2 * std, generator=gen)
            return t.to(dtype)

        params = {}
        for mod, leaves in param_shapes(cfg).items():
            out = {}
            for leaf, shape in leaves.items():
                if leaf == "scale":
                    out[leaf] = torch.ones((1,) + shape, dtype=dtype, device=self.device)
                elif leaf in ("offset", "b"):
                    out[leaf] = torch.zeros((1,) + shape, dtype=dtype, device=self.device)
                elif "embedding_shard" in mod:
                    out[leaf] = tn(shape, 1.0 / np.sqrt(cfg["n_vocab"]))
                elif mod.endswith("linear_3") or mod.endswith("linear_5"):
                    out[leaf] = tn(shape, (2.0 / L) / np.sqrt(d))
                elif mod.endswith("linear_5") or mod.endswith("linear_4") or "projection_shard" in mod \
                        or mod.endswith("linear") or mod.endswith("linear_1") or mod.endswith("linear_2"):
                    fan_in = shape[0] if not mod.endswith("linear_5") else shape[0] * cfg["cores_per_replica"]
                    out[leaf] = tn(shape, 1.0 / np.sqrt(fan_in))
            params[mod] = out
        return {"params": params, "step": np.array(0), "opt_state": None}

    def move_xmap(self, state, _):
        """to_bf16 over the state (transformer_shard.py:250-253)."""
        return to_bf16(state)

    def write_ckpt(self, path, shard):
        """transformer_shard.py:282-283.  One process holds one shard: the call
        writes ``<path>shard_{shard}/`` when ``shard`` is this process's rank and
        does nothing otherwise, so the reference's loop over all shards works."""
        from .checkpoint import write_ckpt
        if shard == self.rank:
            write_ckpt(self._state, path, shard)

    def load_ckpt(self, path, shards_in=None):
        """transformer_shard.py:285-286.  Reads this rank's shard directory; with
        ``shards_in`` different from cores_per_replica the checkpoint is
        re-sharded by parameter role first."""
        from .checkpoint import read_ckpt, tree_flatten, tree_unflatten
        mp = self.config["cores_per_replica"]
        shards_in = mp if shards_in is None else shards_in
        if shards_in == mp:
            from .checkpoint import _from_numpy, read_shard
            leaves = [_from_numpy(a) for a in read_shard(f"{path}shard_{self.rank}/")]
            slim = {k: v for k, v in self._state.items() if k != "opt_state"}
            flat = tree_flatten(slim)
            if len(leaves) > len(flat):
                # a training checkpoint: optimizer-state leaves come first in flatten order
                # ("opt_state" < "params" < "step"); the callers of this path delete them (device_sample.py:74-79)
                leaves = leaves[len(leaves) - len(flat):]
            if len(leaves) != len(flat):
                raise AssertionError(f"Incompatible checkpoints: {len(leaves)} leaves on disk, {len(flat)} expected")
            for a, (_, old) in zip(leaves, flat):
                if a.numel() > 1 and tuple(a.shape) != tuple(old.shape) and tuple(a.shape) != tuple(old.shape[1:]):
                    raise AssertionError(f"Incompatible checkpoints: leaf of shape {tuple(a.shape)} where "
                                         f"{tuple(old.shape)} is expected")
            new = tree_unflatten(slim, [a if a.dim() == 0 or tuple(a.shape) == tuple(old.shape) else a[None]
                                        for a, (_, old) in zip(leaves, flat)])
        else:
            template = {"params": {m: {k: torch.empty((mp,) + tuple(v.shape[1:]), dtype=v.dtype, device="meta")
                                       for k, v in leaves.items()}
                                   for m, leaves in self._state["params"].items()},
                        "step": self._state.get("step")}
            full = read_ckpt(template, path, shards_in, mp, by_role=True)
            new = {"params": {m: {k: v[self.rank:self.rank + 1] for k, v in leaves.items()}
                              for m, leaves in full["params"].items()}, "step": full["step"]}
        new["opt_state"] = self._state.get("opt_state")
        self.state = new

    def train(self, sample):
        raise NotImplementedError("training is outside the forward/decode path")

    def close(self):
        """Frees the device runtime (collective across shards when mp > 1)."""
        if self._rt is not None:
            self._rt.close()
            self._rt = None
            self._rt_caps = (0, 0)

    # -- runtime -------------------------------------------------------------
    def _runtime(self, batch: int, gen_length: int) -> ShardRuntime:
        cap_b, cap_g = self._rt_caps
        if self._rt is None or batch > cap_b or gen_length > cap_g:
            if self._rt is not None:
                self._rt.close()
            cap_b, cap_g = max(batch, cap_b), max(gen_length, cap_g, 1)
            self._rt = ShardRuntime(self.config, rank=self.rank, device=self.device,
                                    max_batch=cap_b, max_gen=cap_g)
            self._rt_caps = (cap_b, cap_g)
            self._dirty = True
        if self._dirty:
            if self._state is None:
                raise RuntimeError("network.state has not been set")
            self._rt.load_params(self._state["params"])
            self._dirty = False
        return self._rt

    # -- eval ----------------------------------------------------------------
    def eval(self, sample):
        """transformer_shard.py:308-324: ``sample`` holds ``obs`` and ``target``
        [batch, T] and optionally ``ctx_length`` [batch]; returns the dict of
        transformer_shard.py:67-72 with a leading batch axis."""
        obs = np.ascontiguousarray(np.asarray(sample["obs"]), dtype=np.uint32)
        tgt = np.ascontiguousarray(np.asarray(sample["target"]), dtype=np.uint32)
        if "ctx_length" in sample:
            ctx_length = np.asarray(sample["ctx_length"]).reshape(-1)
        else:
            ctx_length = np.array([len(obs[0])] * len(obs))
        if self._monitor is not None:
            self._monitor.step()
        rt = self._runtime(obs.shape[0], max(self._rt_caps[1], 1))
        with torch.cuda.device(self.device):
            loss, correct = rt.eval_loss(torch.from_numpy(obs.view(np.int32)).to(self.device),
                                         torch.from_numpy(tgt.view(np.int32)).to(self.device), ctx_length)
            all_loss = loss.cpu().numpy()
            rt.check_device_status()
            return {"loss": all_loss.mean(-1), "last_loss": all_loss[:, -1], "all_loss": all_loss,
                    "correct": correct.cpu().numpy().astype(bool)}

    # -- generate ------------------------------------------------------------
    def generate(self, ctx, ctx_length, gen_length, sampler_options=None, return_logits=False, uniforms=None):
        """transformer_shard.py:326-339.  A config without ``"sampler"`` (a KeyError in the reference,
        :191) samples with ``nucleaus_sample``.  ``ctx`` is [batch, seq] left-padded
        token ids, ``ctx_length`` the number of real tokens per row.  Returns
        ``(final_state, (tokens[batch, gen, 1] uint32, None[, logits]))`` like
        the reference's scan output.  ``uniforms`` ([gen, batch, n_vocab] in
        [tiny, 1)) replaces the PRNG key stream for reproducible sampling; when
        omitted they are drawn on the device by a counter-based generator keyed
        by a seed taken from Python's ``random`` like the reference's key (:327).
        ``self.last_seed`` keeps that key."""
        sampler_options = sampler_options or {}
        ctx = np.ascontiguousarray(np.asarray(ctx), dtype=np.uint32)
        batch = ctx.shape[0]
        assert ctx.shape[1] == self.config["seq"], "context must be padded to config['seq']"
        lengths = np.asarray(ctx_length, dtype=np.uint32).reshape(batch)
        self.gen_length = gen_length
        self.return_logits = return_logits
        if self._monitor is not None:
            self._monitor.step()
        key = random.randint(0, 2 ** 60)   # the reference seeds its PRNG the same way (:327)
        if self.config["cores_per_replica"] > 1:
            # every shard samples the same token: all of them need the same key
            import torch.distributed as dist
            kt = torch.tensor([key], dtype=torch.int64,
                              device=self.device if dist.get_backend() == "nccl" else "cpu")
            dist.broadcast(kt, src=0)
            key = int(kt.item())
        self.last_seed = key
        sampler = self.config.get("sampler")
        name = getattr(sampler, "__name__", None)
        if sampler is not None and name not in ("nucleaus_sample", "softmax_sample"):
            raise NotImplementedError("only nucleaus_sample / softmax_sample run on the device path")
        rt = self._runtime(batch, gen_length)
        # options the caller leaves out take nucleaus_sample's own defaults (sampling.py:41: top_p 0.9, temp 1);
        # the arg-max shortcut below is taken only for an explicit top_p == 0 on every row
        top_p = np.asarray(sampler_options.get("top_p", np.full(batch, 0.9)), dtype=np.float32).reshape(batch)
        temp = np.asarray(sampler_options.get("temp", np.ones(batch)), dtype=np.float32).reshape(batch)
        top_k = sampler_options.get("top_k")
        if top_k is not None:
            if name == "softmax_sample":
                raise TypeError("softmax_sample() got an unexpected keyword argument 'top_k'")   # sampling.py:6
            top_k = np.broadcast_to(np.asarray(top_k, dtype=np.int64).clip(-2**31, 2**31 - 1).astype(np.int32).reshape(-1),
                                    (batch,)).copy()
        if name == "softmax_sample":
            top_p = np.full(batch, np.inf, np.float32)
        greedy = bool(np.all(top_p == 0.0)) and top_k is None
        with torch.cuda.device(self.device):
            t_start = time.perf_counter()
            ctx_dev = torch.from_numpy(ctx.view(np.int32)).pin_memory().to(self.device, non_blocking=True)
            toks = torch.empty((gen_length, batch), dtype=torch.int32, device=self.device)
            logits = None
            if return_logits:
                logits = torch.empty((gen_length, batch, self.config["n_vocab"]), dtype=torch.float32,
                                     device=self.device)
            samp = {"greedy": True}
            if not greedy:
                samp = {"greedy": False,
                        "top_p": torch.from_numpy(top_p).to(self.device),
                        "temp": torch.from_numpy(temp).to(self.device)}
                if uniforms is not None:
                    uniforms = torch.as_tensor(np.asarray(uniforms, dtype=np.float32)).to(self.device).contiguous()
                    assert tuple(uniforms.shape) == (gen_length, batch, self.config["n_vocab"])
                    samp["uniforms"] = uniforms
                else:
                    rt.set_seed(key)           # the scan's PRNG key: the uniforms are drawn on the device
            rt.set_top_k(None if top_k is None or greedy else torch.from_numpy(top_k).to(self.device))
            shard = CausalTransformerShard(self.config, runtime=rt)
            shard.generate_initial(ctx_dev, lengths)
            torch.cuda.current_stream(self.device).synchronize()
            t_prefilled = time.perf_counter()
            shard.generate_scan(gen_length, toks, logits, **samp)
            out_tokens = toks.cpu().numpy().view(np.uint32).T[:, :, None]
            rt.check_device_status()       # a bounded device-side wait that ran out must not pass as a result
            # wall-clock split of this call, like the timing prints of the reference's callers
            # (device_serve.py:156,194): context upload + prefill, then the scan with the tokens back on the host
            self.last_generate_timing = {"prefill_s": t_prefilled - t_start,
                                         "decode_s": time.perf_counter() - t_prefilled,
                                         "h2d_bytes": int(ctx.nbytes), "d2h_bytes": int(out_tokens.nbytes)}
            output = (out_tokens, None)
            if return_logits:
                output = output + (logits.permute(1, 0, 2)[:, :, None, :].cpu().numpy(),)
        return None, output
