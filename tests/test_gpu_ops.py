"""GPU numerics of the single-GPU kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_mm(a, b):
    return a.float() @ b.float().t()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 776, 520), (4096, 1024, 2048), (64, 8, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_matches_fp32_reference(M, N, K, dtype):
    from triton_distributed_b200 import ops
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(N, K, device="cuda", dtype=dtype) * 0.05
    c = ops.gemm(a, b)
    torch.cuda.synchronize()
    ref = _ref_mm(a, b)
    torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 1280, 5120), (8, 5120, 1024), (16, 384, 4096), (33, 1000, 520),
                                   (128, 512, 1024), (256, 256, 512)])
def test_gemm_skinny(M, N, K):
    from triton_distributed_b200 import ops
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    for splits in (0, 1, 3):
        y = ops.gemm_skinny(x, w, splits=splits)
        torch.cuda.synchronize()
        torch.testing.assert_close(y.float(), _ref_mm(x, w), rtol=2e-2, atol=2e-2)
    # the scratch must be left clean: a second call gives the same answer
    y2 = ops.gemm_skinny(x, w)
    torch.testing.assert_close(y2.float(), _ref_mm(x, w), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,I,K", [(8, 3200, 5120), (4, 256, 128), (40, 1000, 520)])
def test_gemm_skinny_swiglu(M, I, K):
    from triton_distributed_b200 import ops
    torch.manual_seed(2)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(2 * I, K, device="cuda", dtype=torch.bfloat16) * 0.03
    y = ops.gemm_skinny(x, w, swiglu=True)
    gu = _ref_mm(x, w)
    ref = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    torch.testing.assert_close(y.float(), ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("rows,hidden", [(8, 5120), (3, 128), (1000, 8192), (17, 16384)])
def test_rmsnorm(rows, hidden):
    from triton_distributed_b200 import ops
    torch.manual_seed(3)
    x = torch.randn(rows, hidden, device="cuda", dtype=torch.bfloat16)
    g = torch.randn(hidden, device="cuda", dtype=torch.bfloat16)
    y = ops.rmsnorm(x, g, 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    res = torch.randn_like(x)
    res0 = res.clone()
    y2 = ops.rmsnorm(x, g, 1e-6, residual=res)
    h = (x.float() + res0.float()).to(torch.bfloat16)
    torch.testing.assert_close(res, h)
    hf = h.float()
    ref2 = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float()
    torch.testing.assert_close(y2.float(), ref2, rtol=2e-2, atol=2e-2)


def _rope_ref(x, pos, theta=1e6):
    # x [T, H, 128] fp32, neox style
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=x.device, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


def test_qk_norm_rope_and_cache_write():
    from triton_distributed_b200 import ops
    torch.manual_seed(4)
    T, Hq, Hkv, D = 37, 8, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 4000, (T,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    ang = torch.arange(4096, device="cuda", dtype=torch.float32)[:, None] * inv[None, :]
    cos_sin = torch.cat([ang.cos(), ang.sin()], -1).contiguous()
    qg = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    kg = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    slots = torch.randperm(64, device="cuda")[:T].to(torch.int64)
    kc = torch.zeros(64, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = ops.qk_norm_rope(qkv, pos, cos_sin, Hq, Hkv, kc, vc, slots, qg, kg, 1e-6)
    x = qkv.float().view(T, Hq + 2 * Hkv, D)

    def norm(v, g):
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float()).to(torch.bfloat16).float()

    q_ref = _rope_ref(norm(x[:, :Hq], qg), pos)
    k_ref = _rope_ref(norm(x[:, Hq:Hq + Hkv], kg), pos)
    torch.testing.assert_close(q.float(), q_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(kc[slots].float(), k_ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(vc[slots], qkv.view(T, -1, D)[:, Hq + Hkv:])


def test_silu_mul_and_topk():
    from triton_distributed_b200 import ops
    torch.manual_seed(5)
    x = torch.randn(19, 2 * 1536, device="cuda", dtype=torch.bfloat16)
    y = ops.silu_mul(x)
    ref = torch.nn.functional.silu(x[:, :1536].float()) * x[:, 1536:].float()
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    logits = torch.randn(77, 256, device="cuda", dtype=torch.float32)
    ids, w = ops.topk_softmax(logits, 8)
    pw, pi = torch.topk(torch.softmax(logits, -1), 8, dim=-1)
    assert torch.equal(ids.long(), pi)
    torch.testing.assert_close(w, pw, rtol=1e-4, atol=1e-6)


def _paged_attn_ref(q, kc, vc, kv_lens, bt, scale, soft_cap=0.0):
    B, Hq, D = q.shape
    page, Hkv = kc.shape[1], kc.shape[2]
    G = Hq // Hkv
    out = torch.zeros(B, Hq, D, device=q.device)
    lse = torch.full((B, Hq), -float("inf"), device=q.device)
    for b in range(B):
        L = int(kv_lens[b])
        if L == 0:
            continue
        nb = (L + page - 1) // page
        k = kc[bt[b, :nb].long()].reshape(-1, Hkv, D)[:L].float()
        v = vc[bt[b, :nb].long()].reshape(-1, Hkv, D)[:L].float()
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("hd,lhd->hl", q[b].float(), k) * scale
        if soft_cap > 0:
            s = soft_cap * torch.tanh(s / soft_cap)
        lse[b] = torch.logsumexp(s, -1)
        out[b] = torch.einsum("hl,lhd->hd", torch.softmax(s, -1), v)
    return out, lse


@pytest.mark.parametrize("B,Hq,Hkv,page,max_len,splits,soft_cap", [
    (2, 8, 1, 16, 300, 1, 0.0), (3, 64, 8, 1, 777, 4, 0.0), (1, 32, 4, 64, 4096, 8, 30.0), (4, 16, 16, 32, 130, 3, 0.0),
    (2, 40, 2, 16, 500, 2, 0.0)])
def test_paged_decode_attention(B, Hq, Hkv, page, max_len, splits, soft_cap):
    from triton_distributed_b200 import ops
    torch.manual_seed(6)
    D = 128
    nblk_per = (max_len + page - 1) // page
    nblocks = B * nblk_per + 3
    kc = torch.randn(nblocks, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    perm = torch.randperm(nblocks, device="cuda")[: B * nblk_per].to(torch.int32).view(B, nblk_per)
    kv_lens = torch.randint(1, max_len + 1, (B,), device="cuda", dtype=torch.int32)
    kv_lens[0] = max_len
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    out, lse = ops.decode_attention(q, kc, vc, kv_lens, perm, scale, soft_cap, splits, return_lse=True)
    ref, ref_lse = _paged_attn_ref(q, kc, vc, kv_lens, perm, scale, soft_cap)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, ref_lse, rtol=1e-2, atol=1e-2)


def test_top_p_sampling_matches_sorted_reference():
    from triton_distributed_b200 import ops
    torch.manual_seed(7)
    B, V = 6, 151936
    logits = torch.randn(B, V, device="cuda") * 3
    temperature, top_p = 0.6, 0.95
    probs = torch.softmax(logits / temperature, -1)
    sp, si = torch.sort(probs, -1, descending=True)
    keep = (torch.cumsum(sp, -1) - sp) < top_p
    nucleus = torch.zeros_like(probs, dtype=torch.bool).scatter(1, si, keep)
    counts = torch.zeros(B, V, device="cuda")
    n_draws = 400
    for _ in range(n_draws):
        ids = ops.top_p_sample(logits, temperature, top_p)
        assert ids.shape == (B, 1) and ids.dtype == torch.int64
        assert bool(nucleus.gather(1, ids).all()), "sampled a token outside the nucleus"
        counts.scatter_add_(1, ids, torch.ones(B, 1, device="cuda"))
    # the most likely token must be drawn about as often as its renormalised probability says
    pn = probs * nucleus
    pn = pn / pn.sum(-1, keepdim=True)
    top = pn.argmax(-1, keepdim=True)
    want = pn.gather(1, top).squeeze(1)
    got = counts.gather(1, top).squeeze(1) / n_draws
    assert torch.all((got - want).abs() < 4 * torch.sqrt(want * (1 - want) / n_draws) + 0.02)
    # u = 0 picks the first kept index, and peaked logits are deterministic
    peaked = torch.full((2, 1000), -30.0, device="cuda")
    peaked[0, 123] = 10.0
    peaked[1, 999] = 10.0
    ids = ops.top_p_sample(peaked, 1.0, 0.9)
    assert ids.flatten().tolist() == [123, 999]
    # odd vocabulary: rows that are not 16-byte aligned take the scalar path; tiny rows leave some CTAs without work
    odd = torch.full((3, 1001), -30.0, device="cuda")
    odd[0, 1000] = 10.0
    odd[1, 5] = 10.0
    odd[2, 500] = 10.0
    assert ops.top_p_sample(odd, 1.0, 0.9).flatten().tolist() == [1000, 5, 500]
    tiny = torch.full((2, 10), -30.0, device="cuda")
    tiny[0, 9] = 5.0
    tiny[1, 0] = 5.0
    assert ops.top_p_sample(tiny, 0.7, 0.5).flatten().tolist() == [9, 0]


@pytest.mark.parametrize("M,K,Hq,Hkv,with_norm,with_scale", [(8, 5120, 8, 1, True, True), (3, 512, 2, 2, False, False),
                                                             (16, 1024, 64, 8, True, False)])
def test_gemm_skinny_qkv_heads_epilogue(M, K, Hq, Hkv, with_norm, with_scale):
    """The qkv projection that finishes every head in its epilogue (per-head RMSNorm, RoPE, q buffer, cache write),
    optionally with the input's RMSNorm folded in as a per-row scale, against the fp32 statement of the same chain."""
    from triton_distributed_b200 import ops
    torch.manual_seed(11)
    D, eps = 128, 1e-6
    N = (Hq + 2 * Hkv) * D
    h = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * K ** -0.5
    pos = torch.randint(0, 4000, (M,), device="cuda", dtype=torch.int32)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda", dtype=torch.float32) / D))
    ang = torch.arange(4096, device="cuda", dtype=torch.float32)[:, None] * inv[None, :]
    cos_sin = torch.cat([ang.cos(), ang.sin()], -1).contiguous()
    qg = torch.randn(D, device="cuda", dtype=torch.bfloat16) if with_norm else None
    kg = torch.randn(D, device="cuda", dtype=torch.bfloat16) if with_norm else None
    slots = torch.randperm(64, device="cuda")[:M].to(torch.int64)
    kc = torch.zeros(64, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = torch.zeros(M, Hq, D, device="cuda", dtype=torch.bfloat16)
    ep = ops.skinny_qkv_heads(pos, slots, cos_sin, Hq, Hkv, q, kc, vc, qg, kg, eps)
    x_in = h
    scale = torch.ones(M, 1, device="cuda")
    if with_scale:  # input = h * gain, rows scaled by 1 / rms(h) in the epilogue
        gain = torch.randn(K, device="cuda", dtype=torch.bfloat16)
        x_in = (h.float() * gain.float()).to(torch.bfloat16)
        sumsq = torch.zeros(16, device="cuda")
        sumsq[:M] = h.float().pow(2).sum(-1)
        ops.skinny_row_scale(sumsq, K, eps, base=ep)
        scale = torch.rsqrt(sumsq[:M] / K + eps)[:, None]
    for _ in range(2):
        ops.gemm_skinny(x_in, w, epilogue=ep)
    y = (x_in.float() @ w.float().t() * scale).view(M, Hq + 2 * Hkv, D)

    def norm(v, g):
        return v if g is None else v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * g.float()

    q_ref = _rope_ref(norm(y[:, :Hq], qg), pos)
    k_ref = _rope_ref(norm(y[:, Hq:Hq + Hkv], kg), pos)
    torch.testing.assert_close(q.float(), q_ref, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(kc[slots].float(), k_ref, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(vc[slots].float(), y[:, Hq + Hkv:], rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("M,N,K", [(8, 5120, 1024), (5, 384, 4096), (16, 1000, 520)])
def test_gemm_skinny_residual_and_row_scale_epilogues(M, N, K):
    """Producer side: h = x W^T + residual, h * gain and sum(h^2). Consumer side: (h * gain) W2^T scaled by 1 / rms(h),
    plain and with SwiGLU, i.e. an RMSNorm between two projections without a normalisation kernel."""
    from triton_distributed_b200 import ops
    torch.manual_seed(12)
    eps = 1e-6
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * K ** -0.5
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    res0 = res.clone()
    gain = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    xg = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    sumsq = torch.zeros(16, device="cuda")
    ops.gemm_skinny(x, w, epilogue=ops.skinny_residual(res, sumsq, gain, xg))
    h = (x.float() @ w.float().t() + res0.float())
    torch.testing.assert_close(res.float(), h, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(xg.float(), res.float() * gain.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(sumsq[:M], res.float().pow(2).sum(-1), rtol=1e-3, atol=1e-2)
    assert float(sumsq[M:].abs().sum()) == 0.0
    if N % 8 == 0:
        I = 256
        w2 = torch.randn(2 * I, N, device="cuda", dtype=torch.bfloat16) * N ** -0.5
        normed = (res.float() * torch.rsqrt(res.float().pow(2).mean(-1, keepdim=True) + eps) * gain.float())
        y = ops.gemm_skinny(xg, w2, epilogue=ops.skinny_row_scale(sumsq, N, eps))
        torch.testing.assert_close(y.float(), normed @ w2.float().t(), rtol=3e-2, atol=3e-2)
        act = ops.gemm_skinny(xg, w2, swiglu=True, epilogue=ops.skinny_row_scale(sumsq, N, eps))
        gu = normed @ w2.float().t()
        torch.testing.assert_close(act.float(), torch.nn.functional.silu(gu[:, :I]) * gu[:, I:], rtol=3e-2, atol=3e-2)


def test_embedding_with_norm_outputs():
    from triton_distributed_b200 import ops
    torch.manual_seed(13)
    V, H = 1000, 640
    table = torch.randn(V, H, device="cuda", dtype=torch.bfloat16)
    ids = torch.tensor([[3, 999], [0, 17]], device="cuda")
    gain = torch.randn(H, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(ops.embedding(ids, table), table[ids])
    xg = torch.empty(4, H, device="cuda", dtype=torch.bfloat16)
    ss = torch.zeros(16, device="cuda")
    out = ops.embedding(ids.reshape(-1), table, gamma=gain, scaled_out=xg, sumsq_out=ss)
    assert torch.equal(out, table[ids.reshape(-1)])
    torch.testing.assert_close(xg.float(), out.float() * gain.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(ss[:4], out.float().pow(2).sum(-1), rtol=1e-4, atol=1e-3)
