"""ctypes binding of libmtj_b200.so (the C ABI declared in include/mtj_b200.h).

The shared library is the only compute back end: there is no CPU or eager
fallback.  Importing this module without the built library raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libmtj_b200.so")

MTJ_F32, MTJ_BF16 = 0, 1


class MtjError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"libmtj_b200 error {code}: {msg}")
        self.code = code


class MtjConfig(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "layers", "d_model", "n_heads", "n_vocab", "pe_rotary_dims", "seq",
        "cores_per_replica", "rank", "max_batch", "max_gen", "max_rows",
        "hilo_max_batch", "mega_max_batch", "tc_decode_min_batch", "wait_limit")]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python mesh-transformer-jax_b200/build.py` "
            "(nvcc, sm_100a); there is no fallback implementation")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
    sig = {
        "mtj_last_error": (ctypes.c_char_p, []),
        "mtj_version": (i32, []),
        "mtj_create": (i32, [ctypes.POINTER(MtjConfig), ctypes.POINTER(vp)]),
        "mtj_destroy": (i32, [vp]),
        "mtj_weights_bytes": (i64, [vp]),
        "mtj_workspace_bytes": (i64, [vp]),
        "mtj_bind_arenas": (i32, [vp, vp, i64, vp, i64, vp]),
        "mtj_load_param": (i32, [vp, ctypes.c_char_p, vp, i32, i32, ctypes.POINTER(i64), vp]),
        "mtj_comm_unique_id": (i32, [vp]),
        "mtj_comm_init": (i32, [vp, vp]),
        "mtj_p2p_export": (i32, [vp, vp]),
        "mtj_p2p_import": (i32, [vp, vp]),
        "mtj_prefill": (i32, [vp, vp, ctypes.POINTER(ctypes.c_uint32), i32, vp]),
        "mtj_start_batch": (i32, [vp, i32, vp]),
        "mtj_admit": (i32, [vp, i32, vp, i32, vp]),
        "mtj_decode_step": (i32, [vp, vp, vp, vp, vp, i32, vp, vp, vp]),
        "mtj_eval_loss": (i32, [vp, vp, vp, ctypes.POINTER(ctypes.c_uint32), i32, i32, vp, vp, vp]),
        "mtj_forward_logits": (i32, [vp, vp, ctypes.POINTER(ctypes.c_uint32), i32, i32, i32, vp, vp]),
        "mtj_sample_scratch_bytes": (i64, [i32, i32]),
        "mtj_sample_top_p": (i32, [vp, vp, vp, vp, vp, i32, i32, vp, i64, vp, vp]),
        "mtj_launch_count": (i64, [vp]),
        "mtj_check_device_status": (i32, [vp, vp]),
        "mtj_mega_trace": (i32, [vp, i32, ctypes.POINTER(ctypes.c_uint64), i32, vp]),
        "mtj_profile_enable": (i32, [vp, i32]),
        "mtj_profile_read": (i32, [vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(i64), vp]),
        "mtj_k_embed": (i32, [vp, vp, i32, vp, vp, vp]),
        "mtj_k_layer": (i32, [vp, i32, vp, i32, i32, i32, ctypes.POINTER(i32), ctypes.POINTER(i32), i32, vp, vp]),
        "mtj_k_projection": (i32, [vp, vp, i32, vp, vp]),
        "mtj_k_projection_loss": (i32, [vp, vp, vp, i32, vp, vp, vp]),
        "mtj_k_decode_attn_scratch_bytes": (i64, [i32, i32, i32, i32, i32]),
        "mtj_k_ln_gemv": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp]),
        "mtj_k_gemm_tc": (i32, [vp, vp, vp, i32, i32, i32, vp, vp]),
        "mtj_k_decode_attn_noalloc": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, i32, vp]),
        "mtj_set_seed": (i32, [vp, ctypes.c_uint64, vp]),
        "mtj_set_top_k": (i32, [vp, vp, i32, vp]),
        "mtj_generate": (i32, [vp, i32, i32, vp, vp, vp, vp, vp, vp]),
        "mtj_k_rng_uniforms": (i32, [ctypes.c_uint64, i32, i32, i32, vp, vp]),
        "mtj_nucleus_filter": (i32, [vp, vp, vp, i32, i32, vp, vp]),
        "mtj_k_prefill_attn": (i32, [vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, i32, vp, vp]),
        "mtj_k_all_reduce_buffer_bytes": (i64, [vp, i32]),
        "mtj_k_all_reduce": (i32, [vp, ctypes.POINTER(vp), i32, i32, i32, i32, vp, vp, vp, i32, vp]),
        "mtj_k_decode_attn": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, i64, vp, i32, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib, sig


lib, SIGNATURES = _load()


def check(code: int) -> None:
    if code != 0:
        raise MtjError(code, lib.mtj_last_error().decode("utf-8", "replace"))


def u32_array(values):
    arr = (ctypes.c_uint32 * len(values))(*[int(v) for v in values])
    return arr
