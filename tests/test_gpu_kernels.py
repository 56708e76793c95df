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
                                   (2047, 4096, 4096), (100, 6300, 4096), (33, 384, 128), (700, 6300, 512), (193, 128, 64), (8, 512, 256), (32, 256, 4096), (64, 384, 1024)])
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
