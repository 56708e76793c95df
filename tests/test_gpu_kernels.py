"""GPU parity of single kernel families through their C-ABI unit entry points."""
import numpy as np
import pytest

from kernel_util import attention_reference, build_paged_kv, ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d_head,heads,batch,window,cur,pads,split", [
    (256, 16, 1, 2047, 2047 + 5, [0], 128),          # GPT-J-6B shape, ring has wrapped
    (256, 2, 3, 300, 310, [0, 250, 310], 64),        # left pad, and a sequence that sees only itself
    (64, 4, 2, 127, 127, [100, 3], 32),              # tiny config
    (64, 4, 2, 127, 200, [0, 0], 8),                 # many splits
    # eight or more sequences take the multi-page streaming kernel
    (256, 4, 9, 2047, 2047 + 70, [0, 1500, 2100, 0, 77, 64, 2116, 1000, 2117], 128),
    (256, 2, 8, 300, 255, [0, 250, 255, 1, 63, 64, 65, 200], 64),      # window not yet full, cut pages
    (64, 4, 12, 127, 127, [100, 3, 0, 127, 64, 63, 1, 2, 90, 31, 32, 33], 32),
])
def test_decode_attention_matches_reference(cuda_device, d_head, heads, batch, window, cur, pads, split):
    import torch
    from mesh_transformer._lib import check, lib
    rng = np.random.Generator(np.random.PCG64(11))
    ring = (window + 63) // 64 + 1
    spans = [(max(p, cur - window + 1), cur + 1) for p in pads]
    table, kpool, vpool, keys, vals = build_paged_kv(rng, batch, heads, d_head, ring, spans)
    q = rng.standard_normal((batch, heads, d_head)).astype(np.float32)
    dev = cuda_device
    t = lambda a, dt=None: torch.from_numpy(a).to(dev) if dt is None else torch.from_numpy(a).to(dev).to(dt)
    q_d, k_d, v_d = t(q), t(kpool, torch.bfloat16), t(vpool, torch.bfloat16)
    tab_d, pad_d = t(table), t(np.array(pads, np.int32))
    cur_d = t(np.array([cur], np.int32))
    nbytes = lib.mtj_k_decode_attn_scratch_bytes(batch, heads, d_head, window, split)
    assert nbytes > 0
    scratch = torch.full((nbytes + 256,), 0x7f, dtype=torch.uint8, device=dev)   # dirty on purpose
    sp = (scratch.data_ptr() + 255) // 256 * 256
    out = torch.zeros((batch, heads * d_head + 8), dtype=torch.float32, device=dev)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        check(lib.mtj_k_decode_attn(ptr(q_d), ptr(k_d), ptr(v_d), ptr(tab_d), ptr(pad_d), ptr(cur_d),
                                    batch, heads, d_head, window, ring, split, sp, nbytes,
                                    ptr(out), heads * d_head + 8, s))
    got = out.cpu().numpy()[:, :heads * d_head].reshape(batch, heads, d_head)
    for b in range(batch):
        ref = attention_reference(q[b], keys[b], vals[b], d_head)
        assert np.abs(got[b] - ref).max() <= 2e-3 * max(1.0, np.abs(ref).max())
    assert float(out[:, heads * d_head:].abs().max()) == 0.0     # nothing written past the row


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 256), (256, 1792, 256), (254, 512, 1280),
                                   (2047, 4096, 4096), (100, 6300, 4096), (33, 384, 128), (700, 6300, 512), (193, 128, 64), (8, 512, 256), (32, 256, 4096), (64, 384, 1024),
                                   # few weight tiles and at most 64 token rows: K is split over a cluster of 2 or 4 blocks
                                   (16, 2048, 512), (50, 640, 2048), (8, 18000, 4096), (33, 200, 6144),
                                   # the GPT-J-6B in-projection slice of one of 8 / one of 2 shards at 32 sequences
                                   (32, 3584, 4096), (32, 14336, 4096),
                                   # block pairs on 256-row tiles: the last pair's second block lies entirely beyond N
                                   (300, 840, 128), (1000, 1288, 256)])
def test_tensor_core_gemm_matches_fp32_matmul(cuda_device, M, N, K):
    """tcgen05 GEMM against a plain fp32 matmul of the same bf16 values."""
    import torch
    from mesh_transformer._lib import check, lib
    g = torch.Generator(device=cuda_device)
    g.manual_seed(M * 7 + N)
    w = (torch.randn((N, K), generator=g, device=cuda_device) * 0.05).to(torch.bfloat16)
    x = torch.randn((M, K), generator=g, device=cuda_device).to(torch.bfloat16)
    bias = torch.randn((N,), generator=g, device=cuda_device)
    out = torch.full((M, N), float("nan"), device=cuda_device)
    check(lib.mtj_k_gemm_tc(ptr(w), ptr(x), ptr(bias), M, N, K, ptr(out), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    ref = x.float() @ w.float().T + bias
    err = (out - ref).abs().max().item()
    assert err <= 2e-3 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("heads,batch,T,pos0,pads,limits", [
    (2, 2, 200, 0, [0, 37], None),                    # two query tiles, the second partial; left padding
    (3, 1, 128, 64, [10], [150]),                     # a later chunk: keys from the cache before pos0, key limit
    (16, 1, 300, 0, [0], None),                       # the GPT-J-6B head count
    # more blocks than SMs: a block takes a long and a short query tile (odd tile count: the middle one alone)
    (16, 1, 1300, 0, [5], None),
    (8, 3, 900, 0, [0, 100, 899], [2000, 450, 2000]),  # paired tiles with left padding, empty tiles, a key limit
])
def test_tensor_core_prefill_attention_unit(cuda_device, heads, batch, T, pos0, pads, limits):
    """mtj_k_prefill_attn (d_head 256) against fp32 softmax attention over the same bf16 values."""
    import torch
    from mesh_transformer._lib import check, lib
    d_head = 256
    rng = np.random.Generator(np.random.PCG64(5 + heads))
    end = pos0 + T
    ring = (end + 63) // 64 + 1
    table, kpool, vpool, keys, vals = build_paged_kv(rng, batch, heads, d_head, ring, [(p, end) for p in pads])
    q = rng.standard_normal((batch, T, heads, d_head)).astype(np.float32)
    dev = cuda_device
    q_d = torch.from_numpy(q).to(dev).to(torch.bfloat16)
    qf = q_d.float().cpu().numpy()
    k_d = torch.from_numpy(kpool).to(dev).to(torch.bfloat16)
    v_d = torch.from_numpy(vpool).to(dev).to(torch.bfloat16)
    tab_d = torch.from_numpy(table).to(dev)
    pad_d = torch.from_numpy(np.array(pads, np.int32)).to(dev)
    lim_d = None if limits is None else torch.from_numpy(np.array(limits, np.int32)).to(dev)
    ld = heads * d_head + 8
    out = torch.zeros((batch * T, ld), dtype=torch.bfloat16, device=dev)
    status = torch.zeros((1,), dtype=torch.int32, device=dev)
    check(lib.mtj_k_prefill_attn(ptr(q_d), ptr(k_d), ptr(v_d), batch * ring, ptr(tab_d), ptr(pad_d),
                                 None if lim_d is None else ptr(lim_d), batch, T, pos0, heads, d_head, ring,
                                 ptr(out), ld, ptr(status), torch.cuda.current_stream().cuda_stream))
    got = out.float().cpu().numpy()
    assert int(status.item()) == 0
    assert float(np.abs(got[:, heads * d_head:]).max()) == 0.0
    got = got[:, :heads * d_head].reshape(batch, T, heads, d_head)
    for b in range(batch):
        for t in list(range(0, T, 7 if T < 512 else 29)) + [T - 1]:
            last = min(pos0 + t, limits[b] if limits is not None else 1 << 30)
            n = last - pads[b] + 1                                       # keys[b][i] sits at position pads[b] + i
            if n <= 0:
                assert np.abs(got[b, t]).max() == 0.0
                continue
            ref = attention_reference(qf[b, t], keys[b][:n], vals[b][:n], d_head)
            assert np.abs(got[b, t] - ref).max() <= 1.5e-2 * max(1.0, np.abs(ref).max()), (b, t)


def _exchange_buffers(lib, rt, world, rows_cap, dev):
    import ctypes
    import torch
    nbytes = lib.mtj_k_all_reduce_buffer_bytes(rt._h, rows_cap)
    bufs = [torch.zeros((nbytes + 256,), dtype=torch.uint8, device=dev) for _ in range(world)]
    base = [(b.data_ptr() + 255) // 256 * 256 for b in bufs]
    arr = (ctypes.c_void_p * world)(*base)
    d = rt.config["d_model"]
    flag_off = (2 * rows_cap * d * 4 + 255) // 256 * 256

    def view(r, dtype, off, count):
        start = base[r] - bufs[r].data_ptr() + off
        return bufs[r][start:start + count * 4].view(dtype)

    return bufs, arr, flag_off, view


def test_peer_all_reduce_unit_and_bounded_wait(cuda_device):
    """mtj_k_all_reduce on one GPU: rank 0 of a world of two, the peer's buffer being a second local
    allocation that the test fills by hand.  First the peer's flag is never published: the wait runs out
    after mtj_config.wait_limit polls, the kernel returns, mtj_check_device_status reports MTJ_ERR_TIMEOUT
    and nothing is faulted or hung.  Then the peer's data and flag are put in place and the same handle
    reduces correctly."""
    import torch
    torch.cuda.set_device(cuda_device)
    from mesh_transformer._lib import MtjError, check, lib
    from mesh_transformer._runtime import ShardRuntime
    from oracle import spec
    cfg = spec.tiny_config(1, seq=64)
    rt = ShardRuntime(cfg, max_batch=4, max_gen=2, wait_limit=20000)
    d, rows, cap, world = cfg["d_model"], 3, 4, 2
    bufs, arr, flag_off, view = _exchange_buffers(lib, rt, world, cap, cuda_device)
    g = torch.Generator(device=cuda_device)
    g.manual_seed(3)
    mine = torch.randn((rows, d), generator=g, device=cuda_device)
    theirs = torch.randn((rows, d), generator=g, device=cuda_device)
    x0 = torch.randn((rows, d), generator=g, device=cuda_device)
    x = x0.clone()
    stats = torch.zeros((rows, 2), device=cuda_device)
    s = torch.cuda.current_stream().cuda_stream

    # exchange 0: nobody publishes the peer's flag
    check(lib.mtj_k_all_reduce(rt._h, arr, 0, world, cap, rows, ptr(mine), ptr(x), ptr(stats), 1, s))
    with pytest.raises(MtjError) as err:
        rt.check_device_status()
    assert err.value.code == 5                                            # MTJ_ERR_TIMEOUT
    assert torch.equal(x, x0), "a timed-out exchange must leave x alone"
    rt.check_device_status()                                              # the error word was cleared
    seq = int(view(0, torch.int32, flag_off + 256, 1).item())
    assert seq == 1, "the exchange counter moves on after a timeout, so the ranks stay in step"
    assert int(view(1, torch.int32, flag_off, 1).item()) == 1            # rank 0 published its flag to the peer

    # exchange 1: the "peer" has written its partial sums into slot 1 and published flag 2
    view(1, torch.float32, cap * d * 4, rows * d).copy_(theirs.reshape(-1))
    view(0, torch.int32, flag_off + 4, 1).fill_(2)
    check(lib.mtj_k_all_reduce(rt._h, arr, 0, world, cap, rows, ptr(mine), ptr(x), ptr(stats), 1, s))
    rt.check_device_status()
    want = x0 + mine + theirs
    assert torch.allclose(x, want, atol=1e-6)
    assert torch.allclose(stats[:, 0], want.mean(-1), atol=1e-5)
    assert torch.allclose(stats[:, 1], 1.0 / torch.sqrt(want.var(-1, unbiased=False) + 1e-5), rtol=1e-4)
    # exchange 2, without accumulation: x = sum
    view(1, torch.float32, 0, rows * d).copy_(theirs.reshape(-1))
    view(0, torch.int32, flag_off + 4, 1).fill_(3)
    check(lib.mtj_k_all_reduce(rt._h, arr, 0, world, cap, rows, ptr(mine), ptr(x), ptr(stats), 0, s))
    rt.check_device_status()
    assert torch.allclose(x, mine + theirs, atol=1e-6)
    rt.close()
