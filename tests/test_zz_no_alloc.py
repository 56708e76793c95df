"""The allocation-free decode attention entry point against the regular one.

Collected last on purpose: a failure here must not hide any other test in a
run that stops at the first failure.  It passes alone in a fresh process and
after the rest of the suite (the built-in scratch array keeps whatever an
earlier call left in it, and the entry point has to cope with that).
"""
import numpy as np
import pytest

from kernel_util import attention_reference, build_paged_kv, ptr

pytestmark = pytest.mark.gpu


def _case(cuda_device, seed, d_head, heads, batch, window, cur, pads, split):
    import torch
    rng = np.random.Generator(np.random.PCG64(seed))
    ring = (window + 63) // 64 + 1
    spans = [(max(p, cur - window + 1), cur + 1) for p in pads]
    table, kpool, vpool, keys, vals = build_paged_kv(rng, batch, heads, d_head, ring, spans)
    q = rng.standard_normal((batch, heads, d_head)).astype(np.float32)
    dev = cuda_device
    t = lambda a, dt=None: torch.from_numpy(a).to(dev) if dt is None else torch.from_numpy(a).to(dev).to(dt)
    return dict(q=q, keys=keys, vals=vals, ring=ring,
                q_d=t(q), k_d=t(kpool, torch.bfloat16), v_d=t(vpool, torch.bfloat16), tab_d=t(table),
                pad_d=t(np.array(pads, np.int32)), cur_d=t(np.array([cur], np.int32)))


@pytest.mark.parametrize("d_head,heads,batch,window,cur,pads,split", [
    (256, 16, 1, 2047, 2050, [0], 128),
    (64, 4, 2, 127, 150, [100, 0], 32),
])
def test_no_alloc_entry_point_matches_regular_one_twice(cuda_device, d_head, heads, batch, window, cur, pads, split):
    import torch
    from mesh_transformer._lib import check, lib
    ld = heads * d_head
    s = torch.cuda.current_stream().cuda_stream
    for call in range(2):                       # two calls in a row, different data each time
        c = _case(cuda_device, 100 + call, d_head, heads, batch, window, cur, pads, split)
        nbytes = lib.mtj_k_decode_attn_scratch_bytes(batch, heads, d_head, window, split)
        scratch = torch.zeros((nbytes + 256,), dtype=torch.uint8, device=cuda_device)
        sp = (scratch.data_ptr() + 255) // 256 * 256
        want = torch.zeros((batch, ld), dtype=torch.float32, device=cuda_device)
        got = torch.zeros_like(want)
        args = (ptr(c["q_d"]), ptr(c["k_d"]), ptr(c["v_d"]), ptr(c["tab_d"]), ptr(c["pad_d"]), ptr(c["cur_d"]),
                batch, heads, d_head, window, c["ring"], split)
        check(lib.mtj_k_decode_attn(*args, sp, nbytes, ptr(want), ld, s))
        check(lib.mtj_k_decode_attn_noalloc(*args, ptr(got), ld, s))
        torch.cuda.synchronize()
        w, g = want.cpu().numpy(), got.cpu().numpy()
        assert np.abs(g - w).max() <= 2e-3 * max(1.0, np.abs(w).max())
        for b in range(batch):
            ref = attention_reference(c["q"][b], c["keys"][b], c["vals"][b], d_head).reshape(-1)
            assert np.abs(g[b] - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())


def test_no_alloc_entry_point_rejects_shapes_beyond_its_array(cuda_device):
    import torch
    from mesh_transformer._lib import lib
    need = lib.mtj_k_decode_attn_scratch_bytes(64, 16, 256, 2047, 32)
    assert need > 4 * 1024 * 1024
    dummy = torch.zeros((64,), dtype=torch.float32, device=cuda_device)
    rc = lib.mtj_k_decode_attn_noalloc(ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy), ptr(dummy),
                                       64, 16, 256, 2047, 33, 32, ptr(dummy), 4096,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert b"built-in array holds" in lib.mtj_last_error()


def test_no_alloc_entry_point_on_a_second_device():
    """The built-in array and the kernels' shared-memory attribute exist per GPU: a process that drives two
    GPUs gets correct results on the second one too (d_head 256 needs the raised shared-memory limit)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from mesh_transformer._lib import check, lib
    d_head, heads, batch, window, cur, pads, split = 256, 4, 2, 300, 310, [0, 250], 64
    ld = heads * d_head
    for index in (0, 1):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            c = _case(dev, 7 + index, d_head, heads, batch, window, cur, pads, split)
            got = torch.zeros((batch, ld), dtype=torch.float32, device=dev)
            check(lib.mtj_k_decode_attn_noalloc(ptr(c["q_d"]), ptr(c["k_d"]), ptr(c["v_d"]), ptr(c["tab_d"]),
                                                ptr(c["pad_d"]), ptr(c["cur_d"]), batch, heads, d_head, window,
                                                c["ring"], split, ptr(got), ld,
                                                torch.cuda.current_stream(dev).cuda_stream))
            torch.cuda.synchronize(dev)
            g = got.cpu().numpy()
            for b in range(batch):
                ref = attention_reference(c["q"][b], c["keys"][b], c["vals"][b], d_head).reshape(-1)
                assert np.abs(g[b] - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())
