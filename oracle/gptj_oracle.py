"""fp32 NumPy restatement of the reference's v1 (xmap) GPT-J forward path.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  PARITY UNPINNED: the
reference has no tests or golden vectors for this path; the checks that stand
in are listed in oracle/__init__.py.

Every function cites the reference lines it follows (paths relative to the
reference project).  The ``shard`` named axis is simulated explicitly: values
that live per shard are Python lists with one array per shard, and the
collectives are the small functions at the top.  The ``batch`` axis (an xmap
vmap in the reference) is a Python loop in the drivers at the bottom.

Third-party arithmetic (jax 0.2.12 / dm-haiku 0.0.5 / einops 0.3, none of it
under the reference tree) is restated from its published definition:
``hk.Linear`` = x @ w (+ b); ``jax.nn.softmax`` = exp(x - max) / sum;
``jax.nn.gelu`` = tanh approximation; ``jnp.var`` = biased variance.
"""
from __future__ import annotations

import numpy as np

from .spec import PREFIX

F32 = np.float32


# ----------------------------------------------------------------------------
# collectives over the simulated "shard" axis (mesh_transformer/util.py:100-147)
# ----------------------------------------------------------------------------
def f_psum(xs):
    """util.py:101-103 -- identity in the forward pass."""
    return xs


def g_psum(xs):
    """util.py:134-136 -- all-reduce sum over shards, in shard order."""
    s = xs[0].astype(F32, copy=True)
    for x in xs[1:]:
        s = s + x
    return [s for _ in xs]


def pmax(xs):
    m = xs[0]
    for x in xs[1:]:
        m = np.maximum(m, x)
    return [m for _ in xs]


def all_gather(xs):
    return [np.stack(xs) for _ in xs]


# ----------------------------------------------------------------------------
# layers.py
# ----------------------------------------------------------------------------
def replicated_layer_norm(xs, scales, offsets):
    """layers.py:17-36.  mean / biased variance over the last axis, eps inside
    the rsqrt; scale and offset are shard 0's copy (all_gather(...)[0])."""
    scale = all_gather(scales)[0][0]
    offset = all_gather(offsets)[0][0]
    out = []
    for x in xs:
        mean = np.mean(x, axis=-1, keepdims=True, dtype=F32)
        var = np.mean(np.square(x - mean), axis=-1, keepdims=True, dtype=F32)
        inv = scale * (F32(1.0) / np.sqrt(var + F32(1e-5)))
        out.append((inv * (x - mean) + offset).astype(F32))
    return out


def fixed_pos_embedding(n_pos: int, dim: int):
    """layers.py:128-134 -- float64 NumPy table, positions 0..n_pos-1."""
    inv_freq = 1. / (10000 ** (np.arange(0, dim, 2) / dim))
    sinusoid_inp = np.einsum('i , j -> i j', np.arange(n_pos), inv_freq)
    return np.sin(sinusoid_inp), np.cos(sinusoid_inp)


def rotate_every_two(x):
    """layers.py:137-143 -- (x0,x1,x2,x3,..) -> (-x1,x0,-x3,x2,..)."""
    x1 = x[:, :, ::2]
    x2 = x[:, :, 1::2]
    return np.stack((-x2, x1), axis=-1).reshape(x.shape)


def apply_rotary_pos_emb(x, sincos):
    """layers.py:146-148 -- sin/cos repeated x2 interleaved; the LAST
    len(x) positions of the table are used."""
    sin, cos = (np.repeat(t, 2, axis=1)[-x.shape[0]:, None, :] for t in sincos)
    return ((x * cos) + (rotate_every_two(x) * sin)).astype(F32)


def gelu(x):
    """jax.nn.gelu default (approximate=True), used at layers.py:289."""
    x = x.astype(F32)
    c = F32(np.sqrt(2.0 / np.pi))
    return (F32(0.5) * x * (F32(1.0) + np.tanh(c * (x + F32(0.044715) * x * x * x)))).astype(F32)


def softmax(x):
    """jax.nn.softmax over the last axis (layers.py:282, sampling.py:13)."""
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp((x - m).astype(F32))
    return (e / np.sum(e, axis=-1, keepdims=True, dtype=F32)).astype(F32)


class EmbeddingShard:
    """layers.py:165-202 (pe != "fixed")."""

    def __init__(self, config, params):
        self.mp = config["cores_per_replica"]
        assert config["n_vocab"] % self.mp == 0           # layers.py:172
        self.in_dim_per_shard = config["n_vocab"] // self.mp
        if config["pe"] == "fixed":
            raise NotImplementedError("pe == 'fixed' is outside the GPT-J path")
        p = params[PREFIX + "embedding_shard/~/linear"]
        self.w, self.b = p["w"], p["b"]

    def __call__(self, ids):
        """one_hot(ids - shard_start) @ w + b, then all-reduce (layers.py:187-193).
        The one-hot matmul is evaluated as its exact equivalent, a masked row
        gather; the bias is added on every shard before the sum."""
        ids = np.asarray(ids).astype(np.int64)
        outs = []
        for s in range(self.mp):
            local = ids - s * self.in_dim_per_shard
            hit = (local >= 0) & (local < self.in_dim_per_shard)
            rows = self.w[s][np.where(hit, local, 0)].astype(F32)
            rows = rows * hit[:, None].astype(F32)
            outs.append(rows + self.b[s].astype(F32, copy=False))
        return g_psum(outs)


class TransformerLayerShard:
    """layers.py:229-366."""

    def __init__(self, config, params, name):
        heads, dim = config["n_heads"], config["d_model"]
        self.mp = config["cores_per_replica"]
        if config["norm"] != "layernorm":
            raise NotImplementedError("only norm == 'layernorm' is on the GPT-J path")
        self.is_rotary = config["pe"] == "rotary"
        assert dim % heads == 0 and heads % self.mp == 0   # layers.py:238-239
        self.dim = dim
        self.dim_per_head = dim // heads
        self.heads_per_shard = heads // self.mp
        self.dim_per_shard = dim // self.mp
        self.pe_rotary_dims = config.get("pe_rotary_dims", self.dim_per_head)
        base = PREFIX + name + "/~/"
        self.ln = params[base + "replicated_layer_norm"]
        self.q_w = params[base + "linear"]["w"]
        self.v_w = params[base + "linear_1"]["w"]
        self.k_w = params[base + "linear_2"]["w"]
        self.o_w = params[base + "linear_3"]["w"]
        self.ff_in = params[base + "linear_4"]
        self.ff_out = params[base + "linear_5"]

    # layers.py:260-285, one shard
    def self_attn(self, s, q, v, k, attn_bias):
        if self.is_rotary:
            R = self.pe_rotary_dims
            k_rot, k_pass = k[:, :, :R], k[:, :, R:]
            q_rot, q_pass = q[:, :, :R], q[:, :, R:]
            sincos = fixed_pos_embedding(k_rot.shape[0], R)
            q_rot = apply_rotary_pos_emb(q_rot, sincos)
            k_rot = apply_rotary_pos_emb(k_rot, sincos)
            k = np.concatenate([k_rot, k_pass], axis=-1)
            q = np.concatenate([q_rot, q_pass], axis=-1)
        logits = np.einsum("thd,Thd->htT", q, k, optimize=True).astype(F32)
        logits = logits / np.sqrt(self.dim_per_head).astype(F32)
        logits = (logits + attn_bias).astype(F32)
        weights = softmax(logits)
        vec = np.einsum("htT,Thd->thd", weights, v, optimize=True).astype(F32)
        vec = vec.reshape((-1, self.dim_per_shard))
        return vec @ self.o_w[s].astype(F32, copy=False)

    # layers.py:287-290
    def ff(self, s, x):
        h = x @ self.ff_in["w"][s].astype(F32, copy=False) + self.ff_in["b"][s].astype(F32, copy=False)
        h = gelu(h)
        return h @ self.ff_out["w"][s].astype(F32, copy=False) + self.ff_out["b"][s].astype(F32, copy=False)

    # layers.py:292-297
    def qvk_proj(self, s, x):
        shp = x.shape[:-1] + (self.heads_per_shard, self.dim_per_head)
        q = (x @ self.q_w[s].astype(F32, copy=False)).reshape(shp)
        v = (x @ self.v_w[s].astype(F32, copy=False)).reshape(shp)
        k = (x @ self.k_w[s].astype(F32, copy=False)).reshape(shp)
        return q, v, k

    def _norm(self, xs):
        return replicated_layer_norm(f_psum(xs), self.ln["scale"], self.ln["offset"])

    def __call__(self, xs, attn_bias):
        """layers.py:299-313."""
        xs = self._norm(xs)
        seq_len = xs[0].shape[0]
        causal_mask = np.tril(np.ones((seq_len, seq_len)))
        bias = (-1e10 * (1. - causal_mask) + attn_bias).astype(F32)
        outs = []
        for s, x in enumerate(xs):
            q, v, k = self.qvk_proj(s, x)
            outs.append(self.self_attn(s, q, v, k, bias) + self.ff(s, x))
        return g_psum(outs)

    def decode_once(self, decode_states, xs, attn_bias):
        """layers.py:316-344.  ``decode_states`` is a per-shard list."""
        xs = self._norm(xs)
        assert xs[0].shape[0] == 1
        outs, new_states = [], []
        for s, x in enumerate(xs):
            st = decode_states[s]
            q, v, k = self.qvk_proj(s, x)
            v = np.concatenate((st["v"], v), axis=0)[1:]
            k = np.concatenate((st["k"], k), axis=0)[1:]
            tokens_decoded = int(st["tokens_decoded"]) + 1
            length = v.shape[0]
            # uint32 length - tokens_decoded compared with an int32 iota: once
            # tokens_decoded exceeds the window nothing is masked any more.
            masked_tokens = length - tokens_decoded
            attention_mask = np.arange(0, length) < masked_tokens
            bias = (-1e10 * attention_mask + attn_bias).astype(F32)
            outs.append(self.self_attn(s, q, v, k, bias) + self.ff(s, x))
            new_states.append({"tokens_decoded": tokens_decoded, "k": k, "v": v})
        return g_psum(outs), new_states

    def get_init_decode_state(self, xs, given_length, attn_bias):
        """layers.py:347-366."""
        xs = self._norm(xs)
        full_length = xs[0].shape[0]
        masked_tokens = full_length - int(given_length)
        causal_mask = np.tril(np.ones((full_length, full_length)))
        bias = -1e10 * (1. - causal_mask)
        bias = bias - 1e10 * (np.arange(0, full_length) < masked_tokens)
        bias = (bias + attn_bias).astype(F32)
        outs, states = [], []
        for s, x in enumerate(xs):
            q, v, k = self.qvk_proj(s, x)
            outs.append(self.self_attn(s, q, v, k, bias) + self.ff(s, x))
            states.append({"k": k, "v": v, "tokens_decoded": int(given_length)})
        return g_psum(outs), states


class ProjectionShard:
    """layers.py:545-593."""

    def __init__(self, config, params):
        self.mp = config["cores_per_replica"]
        assert config["n_vocab"] % self.mp == 0            # layers.py:552
        if config["norm"] != "layernorm":
            raise NotImplementedError("only norm == 'layernorm' is on the GPT-J path")
        self.dim_per_shard = config["n_vocab"] // self.mp
        self.ln = params[PREFIX + "projection_shard/~/replicated_layer_norm"]
        self.lin = params[PREFIX + "projection_shard/~/linear"]

    def _local_logits(self, xs):
        xs = replicated_layer_norm(xs, self.ln["scale"], self.ln["offset"])
        return [(x @ self.lin["w"][s].astype(F32, copy=False) + self.lin["b"][s].astype(F32, copy=False)).astype(F32)
                for s, x in enumerate(xs)]

    def __call__(self, xs):
        """layers.py:561-567 -- vocab order is shard-major."""
        proj = self._local_logits(xs)
        all_proj = all_gather(proj)[0]                      # [mp, T, V/mp]
        t = all_proj.shape[1]
        return np.transpose(all_proj, (1, 0, 2)).reshape(t, -1)

    def loss(self, xs, targets, z_loss=1):
        """layers.py:569-593."""
        logits = self._local_logits(f_psum(xs))
        targets = np.asarray(targets).astype(np.int64)
        gmax = pmax([l.max(-1, keepdims=True) for l in logits])
        logits = [(l - g).astype(F32) for l, g in zip(logits, gmax)]
        pred, sums = [], []
        for s, l in enumerate(logits):
            local = targets - s * self.dim_per_shard
            hit = (local >= 0) & (local < self.dim_per_shard)
            picked = np.take_along_axis(l, np.where(hit, local, 0)[:, None], axis=-1)[:, 0]
            pred.append((picked * hit).astype(F32))
            sums.append(np.exp(l).sum(axis=-1, dtype=F32))
        predicted_logits = g_psum(pred)[0]
        sum_exp_logits = g_psum(sums)[0]
        loss = np.log(sum_exp_logits) - predicted_logits
        loss = loss + (1e-4 * np.square(np.log(sum_exp_logits)) * z_loss).mean()
        correct = (0.0 == predicted_logits)
        return loss.astype(F32), correct


# ----------------------------------------------------------------------------
# transformer_shard.py
# ----------------------------------------------------------------------------
class CausalTransformerShard:
    """transformer_shard.py:21-115 (all shards of one replica in lock-step)."""

    def __init__(self, config, params):
        self.config = config
        self.mp = config["cores_per_replica"]
        if config["pe"] == "t5":
            raise NotImplementedError("pe == 't5' is outside the GPT-J path")
        self.embed = EmbeddingShard(config, params)
        self.transformer_layers = [TransformerLayerShard(config, params, f"layer_{i}")
                                   for i in range(config["layers"])]
        self.proj = ProjectionShard(config, params)

    def hidden(self, context, mask=0.0):
        """The residual stream before the projection (transformer_shard.py:55-60)."""
        attn_bias = 0 + mask
        xs = self.embed(context)
        for l in self.transformer_layers:
            res = l(xs, attn_bias)
            xs = [x + r for x, r in zip(xs, res)]
        return xs

    def eval(self, context, target, z_loss=0., mask=0.0):
        """transformer_shard.py:47-62."""
        return self.proj.loss(self.hidden(context, mask), target, z_loss)

    def logits(self, context, mask=0.0):
        """Full-sequence logits (proj(x) as in transformer_shard.py:95)."""
        return self.proj(self.hidden(context, mask))

    def loss(self, ctx, tgt, z_loss=False, mask=0.0):
        """transformer_shard.py:64-72."""
        loss, correct = self.eval(ctx, tgt, float(z_loss), mask=mask)
        return {"loss": loss.mean(), "last_loss": loss[-1].mean(),
                "all_loss": loss, "correct": correct}

    def generate_initial(self, context, length):
        """transformer_shard.py:74-95."""
        last = context[-1:]
        context = context[:-1]
        attn_bias = 0
        xs = self.embed(context)
        states = []
        for l in self.transformer_layers:
            res, layer_state = l.get_init_decode_state(xs, int(length) - 1, attn_bias)
            xs = [x + r for x, r in zip(xs, res)]
            states.append(layer_state)
        return self.proj(xs), (last.astype(np.uint32), states)

    def generate_once(self, new_tok, state):
        """transformer_shard.py:97-115."""
        attn_bias = 0
        xs = self.embed(new_tok)
        new_states = []
        for l, s in zip(self.transformer_layers, state):
            res, layer_state = l.decode_once(s, xs, attn_bias)
            xs = [x + r for x, r in zip(xs, res)]
            new_states.append(layer_state)
        return self.proj(xs), new_states


def greedy_sampler(_key, logits, _aux, **_opts):
    """nucleaus_sample with top_p -> 0 (sampling.py:29-36): only the first
    entry of the descending stable sort survives, i.e. the arg-max with the
    HIGHEST index among equal logits (sampling.py:11-12)."""
    v = logits.shape[-1]
    idx = v - 1 - np.argmax(logits[:, ::-1], axis=-1)
    return idx.astype(np.uint32), None


class CausalTransformer:
    """transformer_shard.py:118-339: eval and generate only, batch = loop."""

    def __init__(self, config, params):
        self.config = config
        self.state = {"params": params, "step": np.array(0)}

    def _shard(self):
        return CausalTransformerShard(self.config, self.state["params"])

    def eval(self, sample):
        """transformer_shard.py:308-324 and :123-132."""
        obs, tgt = np.asarray(sample["obs"]), np.asarray(sample["target"])
        if "ctx_length" in sample:
            ctx_length = np.asarray(sample["ctx_length"])
        else:
            ctx_length = np.array([len(obs[0])] * len(obs))
        net = self._shard()
        outs = []
        for b in range(obs.shape[0]):
            mask = (np.arange(0, len(obs[b])) > int(ctx_length[b])) * -1e10
            outs.append(net.loss(obs[b], tgt[b], mask=mask))
        return {k: np.stack([o[k] for o in outs]) for k in outs[0]}

    def generate(self, ctx, ctx_length, gen_length, sampler_options=None,
                 return_logits=False, sampler=greedy_sampler, sampler_inputs=None):
        """transformer_shard.py:190-216 and :326-339.  ``sampler_inputs`` is a
        per-(step, batch) payload handed to the sampler in place of the
        reference's PRNG key (e.g. pre-drawn uniforms)."""
        ctx = np.asarray(ctx)
        net = self._shard()
        sampler_options = sampler_options or {}
        toks, logs = [], []
        for b in range(ctx.shape[0]):
            opts = {k: np.asarray(v)[b] for k, v in sampler_options.items()}
            _, (next_token, state) = net.generate_initial(ctx[b], ctx_length[b])
            tb, lb = [], []
            for t in range(gen_length):
                logits, state = net.generate_once(next_token, state)
                aux = None if sampler_inputs is None else sampler_inputs[t][b]
                next_token, _ = sampler(aux, logits, None, **opts)
                next_token = np.asarray(next_token, np.uint32).reshape(1)
                tb.append(next_token)
                lb.append(logits)
            toks.append(np.stack(tb))
            logs.append(np.stack(lb))
        out = (np.stack(toks), None)
        if return_logits:
            out = out + (np.stack(logs),)
        return None, out
