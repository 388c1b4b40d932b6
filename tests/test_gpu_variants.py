"""Every selectable variant of the attention kernels against fp32 PyTorch references: the three K/V pipelines of the
decode kernel with and without the in-kernel merge of the splits, and the tcgen05 prefill kernel on packed sequences
and on keys read in place from a cache-like slot array."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _paged_ref(q, kc, vc, kv_lens, bt, scale):
    B, Hq, D = q.shape
    page, Hkv = kc.shape[1], kc.shape[2]
    G = Hq // Hkv
    out = torch.zeros(B, Hq, D, device=q.device)
    lse = torch.zeros(B, Hq, device=q.device)
    for b in range(B):
        L = int(kv_lens[b])
        slots = (bt[b].long()[:, None] * page + torch.arange(page, device=q.device)[None, :]).reshape(-1)[:L]
        k = kc.view(-1, Hkv, D)[slots].float().repeat_interleave(G, dim=1)
        v = vc.view(-1, Hkv, D)[slots].float().repeat_interleave(G, dim=1)
        s = torch.einsum("hd,lhd->hl", q[b].float(), k) * scale
        lse[b] = torch.logsumexp(s, -1)
        out[b] = torch.einsum("hl,lhd->hd", torch.softmax(s, -1), v)
    return out, lse


@pytest.mark.parametrize("ring", [0, 3, 6])
@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("B,Hq,Hkv,page,max_len,splits", [(3, 64, 8, 1, 777, 4), (1, 32, 4, 64, 4096, 8), (2, 40, 2, 16, 500, 2),
                                                          (8, 8, 1, 64, 2100, 9), (2, 16, 16, 32, 130, 1)])
def test_decode_attention_pipelines_and_fused_merge(ring, fused, B, Hq, Hkv, page, max_len, splits):
    from triton_distributed_b200 import ops
    torch.manual_seed(6)
    D = 128
    nblk_per = (max_len + page - 1) // page
    nblocks = B * nblk_per + 3
    kc = torch.randn(nblocks, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.randperm(nblocks, device="cuda")[: B * nblk_per].to(torch.int32).view(B, nblk_per)
    kv_lens = torch.randint(1, max_len + 1, (B,), device="cuda", dtype=torch.int32)
    kv_lens[0] = max_len
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(D)
    ws: dict = {}
    for _ in range(2):  # the second call reuses the workspace and finds the tickets zeroed by the first
        out, lse = ops.decode_attention(q, kc, vc, kv_lens, bt, scale, 0.0, splits, return_lse=True, workspace=ws,
                                        fused_combine=fused, ring=ring)
        ref, ref_lse = _paged_ref(q, kc, vc, kv_lens, bt, scale)
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(lse, ref_lse, rtol=1e-2, atol=1e-2)
    if fused and splits > 1:
        assert int(ws["tickets"].abs().sum()) == 0


def _attn_ref(q, k, v, scale, causal):
    """q [lq, Hq, D], k / v [lk, Hkv, D] -> [lq, Hq, D] in fp32 with the bottom-right aligned causal mask."""
    lq, lk, G = q.shape[0], k.shape[0], q.shape[1] // k.shape[1]
    kk, vv = k.float().repeat_interleave(G, dim=1), v.float().repeat_interleave(G, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    if causal:
        qi = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
        ki = torch.arange(lk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1).nan_to_num(0.0), vv)


@pytest.mark.parametrize("lens_q,lens_k,Hq,Hkv,causal", [
    ([128], [128], 2, 1, True), ([300, 77], [300, 77], 8, 2, True), ([64, 200], [256, 333], 4, 4, True),
    ([130], [513], 4, 1, False), ([1024, 1], [1024, 700], 8, 8, True)])
def test_prefill_attention_matches_reference(lens_q, lens_k, Hq, Hkv, causal):
    """Packed variable-length sequences, GQA, and the bottom-right alignment of the causal mask when a sequence has
    more keys than queries."""
    from triton_distributed_b200 import ops
    torch.manual_seed(5)
    D = 128
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(lens_q), Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sum(lens_k), Hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sum(lens_k), Hkv, D, device="cuda", dtype=torch.bfloat16)
    scale = 1 / math.sqrt(D)
    out = ops.prefill_attention(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), scale, causal)
    ops.check_pipeline_status()
    for b, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qs, ks = int(cu_q[b]), int(cu_k[b])
        want = _attn_ref(q[qs:qs + lq], k[ks:ks + lk], v[ks:ks + lk], scale, causal)
        torch.testing.assert_close(out[qs:qs + lq].float(), want, rtol=3e-2, atol=3e-2)


def test_prefill_attention_reads_keys_in_place():
    """Keys of every sequence start at a fixed stride in a larger slot array (a cache whose sequences own contiguous
    runs of slots); rows beyond a sequence's length hold garbage that must not be read into the result."""
    from triton_distributed_b200 import ops
    torch.manual_seed(8)
    D, Hq, Hkv, stride = 128, 8, 2, 640
    lens_q, lens_k = [200, 64, 333], [200, 500, 333]
    B = len(lens_q)
    k = torch.randn(B * stride, Hkv, D, device="cuda", dtype=torch.bfloat16) * 30
    v = torch.randn(B * stride, Hkv, D, device="cuda", dtype=torch.bfloat16) * 30
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.arange(0, (B + 1) * stride, stride, dtype=torch.int32, device="cuda")
    q = torch.randn(sum(lens_q), Hq, D, device="cuda", dtype=torch.bfloat16)
    scale = 1 / math.sqrt(D)
    for b, lk in enumerate(lens_k):  # valid rows are well-scaled; everything else stays large
        k[b * stride:b * stride + lk].normal_()
        v[b * stride:b * stride + lk].normal_()
    out = ops.prefill_attention(q, k, v, cu_q, cu_k, max(lens_q), stride, scale, True,
                                seqlens_k=torch.tensor(lens_k, dtype=torch.int32, device="cuda"))
    ops.check_pipeline_status()
    for b, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qs, ks = int(cu_q[b]), b * stride
        want = _attn_ref(q[qs:qs + lq], k[ks:ks + lk], v[ks:ks + lk], scale, True)
        torch.testing.assert_close(out[qs:qs + lq].float(), want, rtol=3e-2, atol=3e-2)
