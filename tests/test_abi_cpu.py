"""CPU-side checks of the C ABI: the library loads, exports every declared
symbol and validates configs without touching a GPU."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    from mesh_transformer import _lib
    return _lib


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "mtj_b200.h")).read()
    names = set(re.findall(r"\b(mtj_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 15
    for n in sorted(names):
        assert hasattr(lib.lib, n), f"{n} is declared in include/mtj_b200.h but not exported"
    assert names == set(lib.SIGNATURES), "ctypes signatures and header disagree"


def _create(lib, **kw):
    base = dict(layers=2, d_model=256, n_heads=4, n_vocab=512, pe_rotary_dims=16, seq=128,
                cores_per_replica=1, rank=0, max_batch=2, max_gen=8, max_rows=128)
    base.update(kw)
    cfg = lib.MtjConfig(**base)
    h = ctypes.c_void_p()
    rc = lib.lib.mtj_create(ctypes.byref(cfg), ctypes.byref(h))
    return rc, h


def test_create_validates_like_the_reference_asserts(lib):
    rc, h = _create(lib)
    assert rc == 0
    assert lib.lib.mtj_weights_bytes(h) > 0 and lib.lib.mtj_workspace_bytes(h) > 0
    assert lib.lib.mtj_destroy(h) == 0
    # layers.py:172 / :239 / :238
    assert _create(lib, n_vocab=510, cores_per_replica=4, n_heads=4)[0] != 0
    assert _create(lib, n_heads=4, cores_per_replica=8)[0] != 0
    assert _create(lib, d_model=250)[0] != 0
    assert _create(lib, rank=3, cores_per_replica=2)[0] != 0
    assert _create(lib, mega_max_batch=5)[0] != 0
    rc, h = _create(lib, hilo_max_batch=-1, mega_max_batch=4, tc_decode_min_batch=8, wait_limit=1000)
    assert rc == 0 and lib.lib.mtj_destroy(h) == 0
    assert _create(lib, rank=3, cores_per_replica=2)[0] != 0
    assert b"cores_per_replica" in lib.lib.mtj_last_error()


def test_calls_before_binding_fail_cleanly(lib):
    rc, h = _create(lib)
    assert rc == 0
    assert lib.lib.mtj_prefill(h, None, None, 1, None) != 0
    assert lib.lib.mtj_decode_step(h, None, None, None, None, 1, None, None, None) != 0
    lib.lib.mtj_destroy(h)


def test_host_layer_rejects_configs_outside_the_path(lib):
    from mesh_transformer._runtime import validate_config
    ok = dict(layers=2, d_model=256, n_heads=4, n_vocab=512, norm="layernorm", pe="rotary",
              seq=128, cores_per_replica=1)
    validate_config(ok)
    with pytest.raises(NotImplementedError):
        validate_config(dict(ok, norm="rmsnorm"))
    with pytest.raises(NotImplementedError):
        validate_config(dict(ok, pe="t5"))
    with pytest.raises(AssertionError):
        validate_config(dict(ok, n_vocab=511, cores_per_replica=2))
