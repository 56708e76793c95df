"""Per-GPU runtime object: owns the device arenas (as torch tensors) and the
libmtj_b200 handle.  torch is plumbing here (device memory, streams,
torch.distributed); all model math runs in the library's CUDA kernels."""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np
import torch

from . import _lib
from ._lib import MtjConfig, check, lib

PREFIX = "causal_transformer_shard/~/"


def validate_config(config: dict) -> None:
    """The assertions / errors of the reference constructors
    (layers.py:77,172,179,238-239,552; transformer_shard.py:42)."""
    if config.get("norm", "layernorm") != "layernorm":
        raise NotImplementedError("only norm == 'layernorm' is on the GPT-J path")
    if config.get("pe", "rotary") != "rotary":
        raise NotImplementedError("only pe == 'rotary' is on the GPT-J path")
    mp = config["cores_per_replica"]
    assert config["n_vocab"] % mp == 0
    assert config["d_model"] % config["n_heads"] == 0
    assert config["n_heads"] % mp == 0


def param_shapes(config: dict) -> dict:
    """Per-shard leaf shapes of the Haiku tree (layers.py:185,235-258,550-559)."""
    mp = config["cores_per_replica"]
    d, V, L = config["d_model"], config["n_vocab"], config["layers"]
    dl, ffl, Vl = d // mp, 4 * d // mp, V // mp
    s = {PREFIX + "embedding_shard/~/linear": {"w": (Vl, d), "b": (d,)}}
    for i in range(L):
        b = PREFIX + f"layer_{i}/~/"
        s[b + "replicated_layer_norm"] = {"scale": (d,), "offset": (d,)}
        s[b + "linear"] = {"w": (d, dl)}
        s[b + "linear_1"] = {"w": (d, dl)}
        s[b + "linear_2"] = {"w": (d, dl)}
        s[b + "linear_3"] = {"w": (dl, d)}
        s[b + "linear_4"] = {"w": (d, ffl), "b": (ffl,)}
        s[b + "linear_5"] = {"w": (ffl, d), "b": (d,)}
    s[PREFIX + "projection_shard/~/replicated_layer_norm"] = {"scale": (d,), "offset": (d,)}
    s[PREFIX + "projection_shard/~/linear"] = {"w": (d, Vl), "b": (Vl,)}
    return s


def gather_vocab_shards(local: torch.Tensor) -> torch.Tensor:
    """all_gather + transpose + flatten of ProjectionShard.__call__
    (layers.py:565-567): [..., V/mp] per rank -> [..., V], shard-major."""
    import torch.distributed as dist
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, local.contiguous())
    return torch.cat(parts, dim=-1)


class ShardRuntime:
    """One shard (rank) of the model on one GPU."""

    # Path-selection fields of mtj_config (include/mtj_b200.h); 0 = the library default.  Each can be given as a
    # keyword, as an optional key of the config dict ("mtj_<name>"; the reference ignores unknown keys) or, for
    # experiments, through the environment variable named here.
    TUNING = {"hilo_max_batch": "MTJ_TC_HILO_MAX_B", "mega_max_batch": "MTJ_MEGA_MAX_B",
              "tc_decode_min_batch": "MTJ_TC_DECODE_MIN_B", "wait_limit": "MTJ_WAIT_LIMIT"}

    def __init__(self, config: dict, rank: int = 0, device=None, max_batch: int = 1,
                 max_gen: int = 256, max_rows: int | None = None, **tuning):
        validate_config(config)
        if not torch.cuda.is_available():
            raise RuntimeError("libmtj_b200 needs a CUDA device; there is no CPU path")
        self.config = config
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.rank = rank
        self.mp = config["cores_per_replica"]
        seq = config["seq"]
        d_head = config["d_model"] // config["n_heads"]
        if max_rows is None:
            max_rows = min(max(seq, max_batch), 4096)
        unknown = set(tuning) - set(self.TUNING)
        if unknown:
            raise TypeError(f"unknown runtime options: {sorted(unknown)}")
        tune = []
        for name, env in self.TUNING.items():
            v = tuning.get(name)
            if v is None:
                v = config.get("mtj_" + name)
            if v is None and os.environ.get(env) not in (None, ""):
                v = int(os.environ[env])
                if name == "hilo_max_batch" and v == 0:
                    v = -1                         # the variable's 0 has always meant "never"
            tune.append(int(v) if v is not None else 0)
        self.tuning = dict(zip(self.TUNING, tune))
        cfg = MtjConfig(config["layers"], config["d_model"], config["n_heads"], config["n_vocab"],
                        config.get("pe_rotary_dims", d_head), seq, self.mp, rank,
                        max_batch, max_gen, max_rows, *tune)
        self.max_batch, self.max_gen, self.max_rows = max_batch, max_gen, max_rows
        self._h = ctypes.c_void_p()
        check(lib.mtj_create(ctypes.byref(cfg), ctypes.byref(self._h)))
        with torch.cuda.device(self.device):
            wb, sb = lib.mtj_weights_bytes(self._h), lib.mtj_workspace_bytes(self._h)
            self.weights_arena = torch.empty(wb + 256, dtype=torch.uint8, device=self.device)
            self.workspace = torch.empty(sb + 256, dtype=torch.uint8, device=self.device)
            check(lib.mtj_bind_arenas(self._h, self._aligned(self.weights_arena), wb,
                                      self._aligned(self.workspace), sb, self.stream))
        self.vocab_local = config["n_vocab"] // self.mp
        if self.mp > 1:
            self._init_comm()

    def _init_comm(self) -> None:
        """One NCCL communicator over the shard axis; the id travels through
        the torch.distributed world the processes were launched in."""
        import torch.distributed as dist
        assert dist.is_initialized() and dist.get_world_size() == self.mp, \
            "cores_per_replica > 1 needs one torch.distributed process per shard"
        uid = (ctypes.c_uint8 * 128)()
        if self.rank == 0:
            check(lib.mtj_comm_unique_id(uid))
        on_gpu = dist.get_backend() == "nccl"
        t = torch.tensor(list(uid), dtype=torch.uint8, device=self.device if on_gpu else "cpu")
        dist.broadcast(t, src=0)
        uid = (ctypes.c_uint8 * 128)(*t.cpu().tolist())
        with torch.cuda.device(self.device):
            check(lib.mtj_comm_init(self._h, uid))
            if os.environ.get("MTJ_NO_P2P") != "1" and self.mp <= 8:
                # exchange buffers for the peer-memory all-reduce of decode-size messages
                mine = (ctypes.c_uint8 * 64)()
                check(lib.mtj_p2p_export(self._h, mine))
                t = torch.tensor(list(mine), dtype=torch.uint8, device=self.device if on_gpu else "cpu")
                parts = [torch.empty_like(t) for _ in range(self.mp)]
                dist.all_gather(parts, t)
                allh = (ctypes.c_uint8 * (64 * self.mp))(*torch.cat(parts).cpu().tolist())
                check(lib.mtj_p2p_import(self._h, allh))

    @staticmethod
    def _aligned(t: torch.Tensor) -> int:
        return (t.data_ptr() + 255) // 256 * 256

    @property
    def stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def close(self):
        """Releases the handle.  With cores_per_replica > 1 this is collective:
        every rank must call it (it tears the NCCL communicator down)."""
        if getattr(self, "_h", None) is not None and self._h:
            torch.cuda.synchronize(self.device)
            lib.mtj_destroy(self._h)
            self._h = None

    def __del__(self):
        # At interpreter shutdown the CUDA context and the peers of a collective
        # communicator may already be gone: tearing the handle down then can
        # block, so it is only done while the interpreter is alive.
        if sys is None or sys.is_finalizing():
            return
        try:
            self.close()
        except Exception:
            pass

    # -- parameters ---------------------------------------------------------
    def load_param(self, name: str, value) -> None:
        """`name` is '<haiku module path>/<leaf>', `value` this shard's slice."""
        if isinstance(value, np.ndarray):
            value = torch.from_numpy(np.ascontiguousarray(value))
        t = value
        if t.dtype not in (torch.float32, torch.bfloat16):
            t = t.to(torch.float32)
        t = t.to(self.device, non_blocking=False).contiguous()
        shape = (ctypes.c_int64 * t.dim())(*t.shape)
        dt = _lib.MTJ_BF16 if t.dtype == torch.bfloat16 else _lib.MTJ_F32
        check(lib.mtj_load_param(self._h, name.encode(), t.data_ptr(), dt, t.dim(), shape, self.stream))
        torch.cuda.current_stream(self.device).synchronize()   # `t` may be a temporary

    def load_params(self, params: dict, shard_index: int | None = None) -> None:
        """`params` is the reference's two-level dict; leaves carry a leading
        shard axis (all shards, or only this one)."""
        for mod, leaves in params.items():
            for leaf, v in leaves.items():
                n = v.shape[0]
                idx = 0 if n == 1 else (self.rank if shard_index is None else shard_index)
                self.load_param(f"{mod}/{leaf}", v[idx])

    # -- path entry points --------------------------------------------------
    def prefill(self, ctx_dev: torch.Tensor, ctx_length) -> None:
        lens = _lib.u32_array(list(ctx_length))
        check(lib.mtj_prefill(self._h, ctx_dev.data_ptr(), lens, ctx_dev.shape[0], self.stream))

    def start_batch(self, batch: int) -> None:
        """Opens a running decode batch of ``batch`` idle slots (continuous batching)."""
        check(lib.mtj_start_batch(self._h, batch, self.stream))

    def admit(self, slot: int, prompt_dev: torch.Tensor) -> None:
        """Puts a prompt ([len] int32 on the device, 1 <= len <= seq) into one slot of the running batch."""
        prompt_dev = prompt_dev.contiguous()
        check(lib.mtj_admit(self._h, slot, prompt_dev.data_ptr(), prompt_dev.numel(), self.stream))
        torch.cuda.current_stream(self.device).synchronize()       # the caller may drop ``prompt_dev``

    def decode_step(self, tokens_in=None, tokens_out=None, logits_out=None, greedy=True,
                    top_p=None, temp=None, uniforms=None) -> None:
        p = lambda t: None if t is None else t.data_ptr()
        check(lib.mtj_decode_step(self._h, p(tokens_in), p(top_p), p(temp), p(uniforms),
                                  1 if greedy else 0, p(tokens_out), p(logits_out), self.stream))

    def set_seed(self, seed: int) -> None:
        """Key of the device generator that draws the sampler's uniforms when none are supplied."""
        check(lib.mtj_set_seed(self._h, int(seed) & ((1 << 64) - 1), self.stream))

    def set_top_k(self, top_k=None) -> None:
        """The sampler's top_k for the sampled steps that follow: an int32 device tensor [batch], or None."""
        if top_k is None:
            check(lib.mtj_set_top_k(self._h, None, 0, self.stream))
        else:
            check(lib.mtj_set_top_k(self._h, top_k.data_ptr(), int(top_k.numel()), self.stream))

    def generate_steps(self, gen_length: int, tokens_out=None, logits_out=None, greedy=True, top_p=None, temp=None,
                       uniforms=None) -> None:
        """The whole scan from one call: ``gen_length`` decode steps enqueued back to back.
        tokens_out [gen, batch] int32, logits_out [gen, batch, n_vocab], uniforms [gen, batch, n_vocab] or None."""
        p = lambda t: None if t is None else t.data_ptr()
        check(lib.mtj_generate(self._h, gen_length, 1 if greedy else 0, p(top_p), p(temp), p(uniforms),
                               p(tokens_out), p(logits_out), self.stream))

    def forward_logits(self, obs_dev: torch.Tensor, ctx_length, n_last: int) -> torch.Tensor:
        B, T = obs_dev.shape
        out = torch.empty((B, n_last, self.vocab_local), dtype=torch.float32, device=self.device)
        lens = None if ctx_length is None else _lib.u32_array(list(ctx_length))
        check(lib.mtj_forward_logits(self._h, obs_dev.data_ptr(), lens, B, T, n_last, out.data_ptr(),
                                     self.stream))
        if self.mp > 1:
            out = gather_vocab_shards(out)
        return out

    def eval_loss(self, obs_dev: torch.Tensor, target_dev: torch.Tensor, ctx_length):
        B, T = obs_dev.shape
        loss = torch.empty((B, T), dtype=torch.float32, device=self.device)
        correct = torch.empty((B, T), dtype=torch.uint8, device=self.device)
        lens = None if ctx_length is None else _lib.u32_array(list(ctx_length))
        check(lib.mtj_eval_loss(self._h, obs_dev.data_ptr(), target_dev.data_ptr(), lens, B, T,
                                loss.data_ptr(), correct.data_ptr(), self.stream))
        return loss, correct

    def layer(self, index: int, x: torch.Tensor, batch: int, T: int, pos0: int = 0, pad=None, key_limit=None,
              decode: bool = False) -> torch.Tensor:
        i32 = lambda v: None if v is None else (ctypes.c_int32 * len(v))(*[int(a) for a in v])
        x = x.to(self.device, torch.float32).contiguous()
        out = torch.empty_like(x)
        check(lib.mtj_k_layer(self._h, index, x.data_ptr(), batch, T, pos0, i32(pad), i32(key_limit),
                              1 if decode else 0, out.data_ptr(), self.stream))
        return out

    def projection(self, x: torch.Tensor) -> torch.Tensor:
        x = x.to(self.device, torch.float32).contiguous()
        rows = x.shape[0]
        out = torch.empty((rows, self.vocab_local), dtype=torch.float32, device=self.device)
        check(lib.mtj_k_projection(self._h, x.data_ptr(), rows, out.data_ptr(), self.stream))
        return gather_vocab_shards(out) if self.mp > 1 else out

    def projection_loss(self, x: torch.Tensor, targets: torch.Tensor):
        x = x.to(self.device, torch.float32).contiguous()
        rows = x.shape[0]
        loss = torch.empty((rows,), dtype=torch.float32, device=self.device)
        correct = torch.empty((rows,), dtype=torch.uint8, device=self.device)
        check(lib.mtj_k_projection_loss(self._h, x.data_ptr(), targets.data_ptr(), rows, loss.data_ptr(),
                                        correct.data_ptr(), self.stream))
        return loss, correct.bool()

    def embed(self, ids_dev: torch.Tensor):
        rows = ids_dev.numel()
        x = torch.empty((rows, self.config["d_model"]), dtype=torch.float32, device=self.device)
        stats = torch.empty((rows, 2), dtype=torch.float32, device=self.device)
        check(lib.mtj_k_embed(self._h, ids_dev.data_ptr(), rows, x.data_ptr(), stats.data_ptr(), self.stream))
        return x, stats

    FAMILIES = ("in_proj", "attention", "out_proj", "logits", "ff_in_proj")

    def profile_enable(self, on: bool) -> None:
        check(lib.mtj_profile_enable(self._h, 1 if on else 0))

    def profile_read(self) -> dict:
        ms = (ctypes.c_double * len(self.FAMILIES))()
        cnt = (ctypes.c_int64 * len(self.FAMILIES))()
        check(lib.mtj_profile_read(self._h, ms, cnt, self.stream))
        return {f: (ms[i], cnt[i]) for i, f in enumerate(self.FAMILIES)}

    def mega_trace(self, enable: bool, read: bool = False):
        """Phase time stamps (ns) of the persistent decode kernel's block 0."""
        n = 6 * self.config["layers"] + 3
        buf = (ctypes.c_uint64 * n)() if read else None
        check(lib.mtj_mega_trace(self._h, 1 if enable else 0, buf, n if read else 0, self.stream))
        return list(buf) if read else None

    def launch_count(self) -> int:
        return int(lib.mtj_launch_count(self._h))

    def check_device_status(self) -> None:
        check(lib.mtj_check_device_status(self._h, self.stream))
