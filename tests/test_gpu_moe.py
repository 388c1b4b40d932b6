"""MoE kernels on one GPU: routing metadata against the CPU references, grouped GEMM against per-expert matmuls,
and the fused AG / RS forms with this GPU as the only rank."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,topk,E,bm,segments", [(37, 3, 8, 16, 1), (512, 8, 128, 128, 1), (64, 2, 4, 8, 4), (1024, 8, 256, 128, 8)])
def test_moe_sort_matches_reference(T, topk, E, bm, segments):
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import create_sort_plan, moe_sort, order_tiles
    torch.manual_seed(0)
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(T)]).to(torch.int32).cuda()
    plan = create_sort_plan(T * topk, topk, E, bm, segments)
    for _ in range(2):  # epochs
        moe_sort(ids, plan, tokens_per_rank=max(1, T // 4))
    torch.cuda.synchronize()
    m_pad, tiles = int(plan.totals[0]), int(plan.totals[1])
    if segments == 1:
        counts, _, gather, expert_index, want_pad = ref.calc_gather_scatter_index_ref(ids.cpu(), E, bm)
        assert m_pad == want_pad and tiles == want_pad // bm
        assert torch.equal(plan.sorted_ids[:m_pad].cpu(), gather)
        assert torch.equal(plan.tile_expert[:tiles].cpu(), expert_index)
        assert torch.equal(plan.group_count.cpu(), counts)
        world = 4
        _, _, s0, s1, order = ref.ag_moe_tile_schedule_ref(ids.cpu(), E, bm, 1, world) if T % world == 0 else (0, 0, None, None, None)
        if s0 is not None:
            assert torch.equal(plan.tile_seg_start[:tiles].cpu(), s0) and torch.equal(plan.tile_seg_end[:tiles].cpu(), s1)
            got = order_tiles(plan, 1, world)
            torch.cuda.synchronize()
            assert torch.equal(got[:tiles].cpu(), order)
    else:
        sorted_ids, expert_ids, barrier_ids, rank_blocks, npad = ref.moe_align_block_size_ref(ids.cpu(), E, bm, segments)
        assert m_pad == npad
        assert torch.equal(plan.sorted_ids[:m_pad].cpu(), sorted_ids)
        assert torch.equal(plan.tile_expert[:tiles].cpu(), expert_ids)
        assert torch.equal(plan.tile_seg_end[:tiles].cpu(), barrier_ids)
        assert torch.equal(plan.totals[2:].cpu(), torch.cumsum(rank_blocks, 0).to(torch.int32))
    assert int(plan.status[0]) == 0


@pytest.mark.parametrize("T,topk,E,N,K", [(64, 2, 4, 128, 64), (300, 4, 16, 384, 512), (1024, 8, 32, 200, 1032),
                                             (256, 4, 8, 512, 256), (200, 2, 4, 1000, 192)])  # the last two: 256-wide tiles
def test_grouped_gemm_matches_per_expert_matmul(T, topk, E, N, K):
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import grouped_gemm
    torch.manual_seed(1)
    a = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(T)]).to(torch.int32).cuda()
    out = grouped_gemm(a, w, ids)
    torch.cuda.synchronize()
    want = ref.grouped_gemm_ref(a.repeat_interleave(topk, 0), w, ids.reshape(-1).long())
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    # per-pair input and routing weights (the down-projection form)
    x = torch.randn(T * topk, K, device="cuda", dtype=torch.bfloat16)
    sc = torch.rand(T, topk, device="cuda")
    out2 = grouped_gemm(x, w, ids, a_per_pair=True, row_scale=sc)
    want2 = ref.grouped_gemm_ref(x, w, ids.reshape(-1).long()) * sc.reshape(-1, 1)
    torch.testing.assert_close(out2.float(), want2, rtol=2e-2, atol=2e-2)


def test_ag_group_gemm_and_moe_reduce_rs_world1(dist1):
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import (ag_group_gemm, create_ag_group_gemm_context, create_moe_rs_context,
                                                        moe_reduce_rs)
    from triton_distributed_b200.runtime.heap import get_heap
    torch.manual_seed(2)
    T, topk, E, K, N = 256, 4, 16, 512, 384
    a = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    w1 = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    logits = torch.randn(T, E, device="cuda")
    wt, ids = torch.topk(torch.softmax(logits, -1), topk, -1)
    ids = ids.to(torch.int32)
    ctx = create_ag_group_gemm_context(T, N, K, E, topk, torch.bfloat16, 0, 1)
    for _ in range(3):
        up = ag_group_gemm(a, w1, ctx, ids)
        torch.cuda.synchronize()
        get_heap().check_status("ag_group_gemm")
        torch.testing.assert_close(up.float(), ref.ag_group_gemm_ref(a, w1, ids).float(), rtol=2e-2, atol=2e-2)
    # the reference's [E, K, N] weight layout is accepted too
    up_t = ag_group_gemm(a, w1.transpose(1, 2).contiguous(), ctx, ids)
    torch.testing.assert_close(up_t, up)
    ctx.finalize()
    w2 = torch.randn(E, 640, N, device="cuda", dtype=torch.bfloat16) * 0.05
    rctx = create_moe_rs_context(dist1, 1, T, 640, E, topk, torch.bfloat16, torch.bfloat16)
    for _ in range(3):
        down = moe_reduce_rs(up, w2, ids, wt, rctx)
        torch.cuda.synchronize()
        get_heap().check_status("moe_reduce_rs")
        torch.testing.assert_close(down.float(), ref.moe_reduce_rs_ref(up, w2, ids, wt).float(), rtol=3e-2, atol=3e-2)
    rctx.finalize()


def _dequant_weight_blocks(w8, sw):
    E, N, K = w8.shape
    scale = sw.repeat_interleave(128, 1)[:, :N].repeat_interleave(128, 2)
    return w8.float() * scale


def test_fp8_ag_group_gemm_and_moe_reduce_rs_world1(dist1):
    """The block-scaled fp8 forms of both tensor-parallel MoE fusions against the dequantised fp32 products."""
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import (ag_group_gemm_fp8, create_ag_group_gemm_fp8_context,
                                                        create_moe_rs_context, moe_reduce_rs_fp8, quantize_fp8_rows,
                                                        quantize_fp8_weight_blocks)
    from triton_distributed_b200.runtime.heap import get_heap
    torch.manual_seed(12)
    T, topk, E, K, N, H = 256, 4, 16, 512, 384, 640
    a8, sa = quantize_fp8_rows(torch.randn(T, K, device="cuda") * torch.rand(T, 1, device="cuda") * 3)
    w8, sw = quantize_fp8_weight_blocks(torch.randn(E, N, K, device="cuda") * 0.05)
    wt, ids = torch.topk(torch.softmax(torch.randn(T, E, device="cuda"), -1), topk, -1)
    ids = ids.to(torch.int32)
    a_deq = ref.fp8_dequant_ref(a8, sa, dtype=torch.float32)
    want_up = ref.grouped_gemm_ref(a_deq.repeat_interleave(topk, 0), _dequant_weight_blocks(w8, sw), ids.reshape(-1).long())
    ctx = create_ag_group_gemm_fp8_context(T, N, K, E, topk, torch.bfloat16, 0, 1)
    for _ in range(3):
        up = ag_group_gemm_fp8(a8, sa, w8, sw, ctx, ids)
        torch.cuda.synchronize()
        get_heap().check_status("ag_group_gemm_fp8")
        torch.testing.assert_close(up.float(), want_up.float(), rtol=2e-2, atol=2e-2)
    ctx.finalize()
    x8, sx = quantize_fp8_rows(up.float())
    w28, sw2 = quantize_fp8_weight_blocks(torch.randn(E, H, N, device="cuda") * 0.05)
    x_deq = ref.fp8_dequant_ref(x8, sx, dtype=torch.float32)
    pairs = ref.grouped_gemm_ref(x_deq, _dequant_weight_blocks(w28, sw2), ids.reshape(-1).long()) * wt.reshape(-1, 1)
    want_down = pairs.view(T, topk, H).sum(1)
    rctx = create_moe_rs_context(dist1, 1, T, H, E, topk, torch.bfloat16, torch.bfloat16)
    for _ in range(3):
        down = moe_reduce_rs_fp8(x8, sx, w28, sw2, ids, wt, rctx)
        torch.cuda.synchronize()
        get_heap().check_status("moe_reduce_rs_fp8")
        torch.testing.assert_close(down.float(), want_down.float(), rtol=3e-2, atol=3e-2)
    rctx.finalize()


def test_ep_dispatch_combine_world1(dist1):
    from triton_distributed_b200 import ref
    from triton_distributed_b200.layers.nvidia import EPAll2AllLayer
    from triton_distributed_b200.runtime.heap import get_heap
    torch.manual_seed(3)
    T, H, E, topk = 96, 512, 16, 4
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    wt, ids = torch.topk(torch.softmax(torch.randn(T, E, device="cuda"), -1), topk, -1)
    ids = ids.to(torch.int32)
    for fp8 in (False, True):
        layer = EPAll2AllLayer(dist1, T, H, topk, 0, E, 1, 1, torch.bfloat16, fp8=fp8)
        for _ in range(3):
            res = layer.dispatch(x, ids)
            torch.cuda.synchronize()
            get_heap().check_status("ep dispatch")
            sorted_ids, tile_expert, totals, rows_per_expert = layer.recv_plan()
            assert int(rows_per_expert.sum()) == T * topk
            assert torch.equal(rows_per_expert.cpu(), torch.bincount(ids.reshape(-1).long().cpu(), minlength=E).to(torch.int32))
            if fp8:
                q, sc = res
                rows = ref.fp8_dequant_ref(q[: T * topk], sc[: T * topk], dtype=torch.bfloat16)
                expert_out = torch.zeros(layer.max_m, H, device="cuda", dtype=torch.bfloat16)
                expert_out[: T * topk] = rows
            else:
                expert_out = res
            out = layer.combine(expert_out, wt)
            torch.cuda.synchronize()
            get_heap().check_status("ep combine")
            torch.testing.assert_close(out.float(), x.float() * wt.sum(-1, keepdim=True), rtol=0.1 if fp8 else 2e-2,
                                       atol=0.1 if fp8 else 2e-2)
        layer.finalize()


@pytest.mark.parametrize("T,topk,E,N,K", [(64, 2, 4, 128, 128), (300, 4, 16, 384, 512), (1024, 8, 32, 200, 1024)])
def test_grouped_gemm_fp8_block_scaled(T, topk, E, N, K):
    """e4m3 operands, 1x128 activation scales and 128x128 weight scales, against the dequantised fp32 product."""
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import grouped_gemm_fp8, quantize_fp8_rows, quantize_fp8_weight_blocks
    torch.manual_seed(3)
    a = torch.randn(T, K, device="cuda") * torch.rand(T, 1, device="cuda") * 4   # rows of very different magnitude
    w = torch.randn(E, N, K, device="cuda") * 0.05
    a8, sa = quantize_fp8_rows(a)
    w8, sw = quantize_fp8_weight_blocks(w)
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(T)]).to(torch.int32).cuda()
    out = grouped_gemm_fp8(a8, sa, w8, sw, ids)
    torch.cuda.synchronize()
    want = ref.grouped_gemm_fp8_ref(a8.repeat_interleave(topk, 0), sa.repeat_interleave(topk, 0), w8, sw, ids.reshape(-1).long())
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    # and it is close to the unquantised product (fp8 has 3 mantissa bits: a few percent of the row norm)
    exact = ref.grouped_gemm_ref(a.repeat_interleave(topk, 0), w, ids.reshape(-1).long())
    err = (out.float() - exact).norm() / exact.norm()
    assert err < 0.06, f"relative error {err:.3f} against the bf16 product"
    # per-pair rows with routing weights (the down-projection form)
    x = torch.randn(T * topk, K, device="cuda")
    x8, sx = quantize_fp8_rows(x)
    sc = torch.rand(T, topk, device="cuda")
    out2 = grouped_gemm_fp8(x8, sx, w8, sw, ids, a_per_pair=True, row_scale=sc)
    want2 = ref.grouped_gemm_fp8_ref(x8, sx, w8, sw, ids.reshape(-1).long()) * sc.reshape(-1, 1)
    torch.testing.assert_close(out2.float(), want2, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("fp8,fp8_experts", [(False, False), (True, False), (True, True)])
def test_ep_moe_layer_world1(dist1, fp8, fp8_experts):
    """Expert-parallel MoE layer with the GPU as its own only peer: dispatch -> grouped GEMMs -> weighted combine,
    in bf16, with fp8 dispatch, and with the block-scaled fp8 up-projection on the dispatched bytes."""
    from triton_distributed_b200.layers.nvidia import EP_MoE
    from triton_distributed_b200.runtime.heap import get_heap
    E, topk, H, I, T = 8, 2, 256, 384, 64
    torch.manual_seed(11)
    gate = torch.randn(E, H, device="cuda", dtype=torch.bfloat16)  # wide logits: no near-ties between experts
    wgu = torch.randn(E, 2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.05
    wdn = torch.randn(E, H, I, device="cuda", dtype=torch.bfloat16) * 0.05
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    ep = EP_MoE(0, 1, dist1, E, topk, H, T, torch.bfloat16, True, fp8_dispatch=fp8, fp8_experts=fp8_experts)
    ep._init_parameters(gate, wgu, wdn)
    want = ep.torch_fwd(x, wgu, wdn)
    for _ in range(2):
        got = ep.dist_triton_fwd(x)
        torch.cuda.synchronize()
        get_heap().check_status("ep_moe")
        torch.testing.assert_close(got.float(), want.float(), rtol=0.12 if fp8 else 5e-2, atol=0.3 if fp8 else 0.1)
    ep.finalize()


@pytest.mark.parametrize("T,I", [(5, 128), (300, 384), (4096, 1536)])
def test_silu_mul_fp8_matches_gate_then_block_quant(T, I):
    """The fused SwiGLU + e4m3 block quantisation against silu_mul followed by the PyTorch quantiser: scales agree to
    rounding, and the dequantised values agree within one e4m3 step."""
    from triton_distributed_b200 import ops
    from triton_distributed_b200.kernels.nvidia import quantize_fp8_rows
    torch.manual_seed(14)
    x = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
    q, s = ops.silu_mul_fp8(x)
    xf = x.float()
    act = torch.nn.functional.silu(xf[:, :I]) * xf[:, I:]
    q_ref, s_ref = quantize_fp8_rows(act)
    torch.testing.assert_close(s, s_ref, rtol=1e-4, atol=1e-8)
    deq = (q.float().view(T, I // 128, 128) * s[:, :, None]).view(T, I)
    torch.testing.assert_close(deq, act, rtol=0.07, atol=1e-3)
    deq_ref = (q_ref.float().view(T, I // 128, 128) * s_ref[:, :, None]).view(T, I)
    assert (deq - deq_ref).abs().max() <= 0.07 * act.abs().max()
