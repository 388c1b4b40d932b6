"""Multi-rank GPU checks, run as ``torchrun --nproc-per-node N tests/dist_cases.py [case ...]``.

Every case compares a fused kernel with the ``torch.distributed`` (NCCL) + ``torch.matmul`` composition
that the reference uses as its golden (``test/nvidia/test_ag_gemm.py:71-137``, ``test_gemm_rs.py:38-51``,
``test_allreduce.py:95-136``, ``test_fast_allgather.py``). A case passes only if it passes on every rank
and no kernel recorded an expired wait. Exit code = number of failed cases.
"""
from __future__ import annotations

import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from triton_distributed_b200 import _lib  # noqa: E402
from triton_distributed_b200 import utils as U  # noqa: E402
from triton_distributed_b200.kernels.allreduce import to_allreduce_method  # noqa: E402
from triton_distributed_b200.kernels.nvidia import (ag_gemm, all_reduce, all_reduce_rmsnorm, create_ag_gemm_context,  # noqa: E402
                                                    create_allreduce_ctx, create_fast_allgather_context,
                                                    create_gemm_rs_context, fast_allgather, gemm_rs)
from triton_distributed_b200.runtime.heap import get_heap  # noqa: E402

CASES = {}


def case(fn):
    CASES[fn.__name__] = fn
    return fn


def _rank_world():
    return dist.get_rank(), dist.get_world_size()


@case
def heap_peer_views():
    rank, world = _rank_world()
    heap = get_heap()
    views = heap.create_tensors((world, 256), torch.float32)
    # every rank writes its row into every peer's copy through the peer mapping (copy engine / elementwise kernels)
    for k in range(world):
        views[k][rank].fill_(float(rank + 1))
    torch.cuda.synchronize()
    heap.barrier_all()
    torch.cuda.synchronize()
    want = torch.arange(1, world + 1, device="cuda", dtype=torch.float32)[:, None].expand(world, 256)
    assert torch.equal(views[rank], want), "peer writes did not land"
    if heap.has_multicast:
        mc = heap.multicast_tensor(views[rank])
        assert mc.data_ptr() != views[rank].data_ptr()
    heap.barrier_all()
    torch.cuda.synchronize()
    heap.free(views[rank])


@case
def primitives_put_get_notify():
    rank, world = _rank_world()
    heap = get_heap()
    n = 4096
    src = heap.create_tensor((n,), torch.int32)
    dst = heap.create_tensor((n,), torch.int32)
    sig = heap.create_tensor((32,), torch.int32)
    flags = heap.create_tensor((32,), torch.int32)
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    for it in range(1, 4):
        src.copy_(torch.arange(n, device="cuda", dtype=torch.int32) + rank * 100000 + it)
        heap.barrier_all()
        _lib.call("b200_test_ring_put", heap.ctx, _lib.ptr(src), _lib.ptr(dst), _lib.ptr(sig), n, it, _lib.ptr(ok), _lib.stream_ptr())
        torch.cuda.synchronize()
        prev = (rank - 1) % world
        assert int(ok.item()) == 1
        assert torch.equal(dst, torch.arange(n, device="cuda", dtype=torch.int32) + prev * 100000 + it), "ring put"
        heap.barrier_all()
    dst.zero_()
    heap.barrier_all()
    _lib.call("b200_test_ring_get", heap.ctx, _lib.ptr(src), _lib.ptr(dst), n, _lib.ptr(flags), 1, _lib.ptr(ok), _lib.stream_ptr())
    torch.cuda.synchronize()
    prev = (rank - 1) % world
    assert int(ok.item()) == 1 and torch.equal(dst, torch.arange(n, device="cuda", dtype=torch.int32) + prev * 100000 + 3), "ring get"
    counter = heap.create_tensor((8,), torch.int32)
    heap.barrier_all()
    _lib.call("b200_test_notify_add", heap.ctx, _lib.ptr(counter), 0, world, _lib.ptr(ok), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(ok.item()) == 1
    heap.barrier_all()
    torch.cuda.synchronize()
    if rank == 0:
        assert int(counter[0].item()) == world, "notify add"
    if heap.has_multicast:
        buf = heap.create_tensor((1024,), torch.float32)
        buf.fill_(float(rank + 1))
        out = torch.zeros(1024, device="cuda")
        mflags = heap.create_tensor((32,), torch.int32)
        heap.barrier_all()
        _lib.call("b200_test_multimem", heap.ctx, _lib.ptr(buf), 256, _lib.ptr(mflags), 1, _lib.ptr(out), _lib.ptr(ok), _lib.stream_ptr())
        torch.cuda.synchronize()
        assert int(ok.item()) == 1 and torch.all(out == world * (world + 1) / 2), "multimem ld_reduce"
        heap.barrier_all()
        torch.cuda.synchronize()
        heap.free(mflags), heap.free(buf)
    for t in (counter, flags, sig, dst, src):
        heap.free(t)


@case
def shmem_device_api():
    """broadcast / fcollect / putmem_signal_warp / int_p / barrier_all_warp / team queries in one collective kernel."""
    rank, world = _rank_world()
    heap = get_heap()
    n4 = 512
    n = n4 * 4
    bcast = heap.create_tensor((n,), torch.float32)
    coll = heap.create_tensor((world, n), torch.float32)
    ring = heap.create_tensor((n,), torch.float32)
    sig = heap.create_tensor((2,), torch.int32)
    word = heap.create_tensor((world,), torch.int32)
    flags = heap.create_tensor((16,), torch.int32)
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    base = torch.arange(n, device="cuda", dtype=torch.float32)
    for it in range(1, 4):
        root = it % world
        src = base + 1000.0 * rank + it
        heap.barrier_all()
        _lib.call("b200_test_shmem_api", heap.ctx, _lib.ptr(src), _lib.ptr(bcast), _lib.ptr(coll), _lib.ptr(ring), _lib.ptr(sig),
                  _lib.ptr(word), _lib.ptr(flags), n4, root, it, _lib.ptr(ok), _lib.stream_ptr())
        torch.cuda.synchronize()
        assert int(ok.item()) == 1, "shmem api probe reported a failed wait"
        assert torch.equal(bcast, base + 1000.0 * root + it), "broadcast"
        for r in range(world):
            assert torch.equal(coll[r], base + 1000.0 * r + it), f"fcollect slot {r}"
        assert torch.equal(ring, base + 1000.0 * ((rank - 1) % world) + it), "putmem_signal_warp"
        assert word.tolist() == [it + r for r in range(world)], "int_p"
        heap.barrier_all()
    torch.cuda.synchronize()
    for t in (flags, word, sig, ring, coll, bcast):
        heap.free(t)


@case
def fast_allgather_modes():
    rank, world = _rank_world()
    heap = get_heap()
    ctx = create_fast_allgather_context(rank, 0, world, 1, max_buffer_size=4 << 20)
    modes = ["pull", "push2d", "push2d_ll"] + (["push2d_ll_multimem"] if heap.has_multicast else [])
    for per_rank in (64, 4096, 65536):
        buf = heap.create_tensor((world, per_rank), torch.float32)
        for it, mode in enumerate(modes * 2):
            buf.zero_()
            buf[rank] = torch.arange(per_rank, device="cuda", dtype=torch.float32) + 1000 * rank + it
            heap.barrier_all()
            fast_allgather(buf, ctx, mode=mode)
            torch.cuda.synchronize()
            want = torch.arange(per_rank, device="cuda", dtype=torch.float32)[None, :] + 1000 * torch.arange(
                world, device="cuda", dtype=torch.float32)[:, None] + it
            assert torch.equal(buf, want), f"fast_allgather {mode} {per_rank}"
            heap.barrier_all()
        torch.cuda.synchronize()
        heap.free(buf)
    ctx.finalize()


@case
def allreduce_methods():
    rank, world = _rank_world()
    heap = get_heap()
    ctx = create_allreduce_ctx(8 << 20, rank, world, world)
    methods = ["one_shot", "two_shot", "double_tree"] + (["one_shot_multimem", "two_shot_multimem"] if heap.has_multicast else [])
    tol = {torch.bfloat16: 3e-2, torch.float16: 1e-2, torch.float32: 1e-3}
    for dtype in (torch.bfloat16, torch.float16, torch.float32):
        for n in (8 * world, 4096 * world, 1 << 20, (3 << 20) + 16 * world):
            for m in methods:
                torch.manual_seed(rank + n)
                x = torch.randn(n, device="cuda", dtype=dtype)
                ref = x.clone().float()
                dist.all_reduce(ref)
                for _ in range(2):
                    y = all_reduce(x, None, to_allreduce_method(m), ctx)
                torch.cuda.synchronize()
                torch.testing.assert_close(y.float(), ref, rtol=tol[dtype], atol=tol[dtype] * 4, msg=lambda s: f"{m} {dtype} n={n}: {s}")
    y = all_reduce(torch.ones(1024, device="cuda", dtype=torch.float32), None, None, ctx)  # auto method
    assert torch.all(y == world)
    ctx.finalize()


@case
def allreduce_fused_rmsnorm():
    rank, world = _rank_world()
    heap = get_heap()
    ctx = create_allreduce_ctx(32 << 20, rank, world, world)
    methods = ["one_shot", "two_shot"] + (["one_shot_multimem", "two_shot_multimem"] if heap.has_multicast else [])
    if os.environ.get("B200DIST_AR_LL", "0") == "1":
        methods.append(None)  # the automatic choice, which the opt-in packet path takes over for small inputs
    for rows, hidden in ((8, 5120), (8 * world, 8192), (3, 1024), (64 * world, 8192)):
        for m in methods:
            torch.manual_seed(rank * 7 + rows)
            x = torch.randn(rows, hidden, device="cuda", dtype=torch.bfloat16)
            torch.manual_seed(rows)
            res = torch.randn(rows, hidden, device="cuda", dtype=torch.bfloat16)
            g = torch.randn(hidden, device="cuda", dtype=torch.bfloat16)
            s = x.clone().float()
            dist.all_reduce(s)
            h_ref = (s.to(torch.bfloat16).float() + res.float())  # tolerance covers the reference's extra rounding
            res_in = res.clone()
            y, h = all_reduce_rmsnorm(x, res_in, g, 1e-6, ctx, to_allreduce_method(m) if m else None)
            torch.cuda.synchronize()
            torch.testing.assert_close(h.float(), h_ref, rtol=3e-2, atol=6e-2, msg=lambda s_: f"residual {m} {rows}x{hidden}: {s_}")
            hf = h.float()
            y_ref = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float()
            torch.testing.assert_close(y.float(), y_ref, rtol=2e-2, atol=2e-2, msg=lambda s_: f"normed {m} {rows}x{hidden}: {s_}")
            # all ranks must hold identical results
            hh = [torch.empty_like(h) for _ in range(world)]
            dist.all_gather(hh, h.contiguous())
            assert all(torch.equal(hh[0], t) for t in hh), f"ranks disagree on the residual ({m})"
    ctx.finalize()


def _ag_gemm_case(Mr, N, K, dtype, iters=3, straggler=False, method=None):
    rank, world = _rank_world()
    torch.manual_seed(1234 + rank)
    b = (torch.randn(N, K, device="cuda", dtype=dtype) * 0.05)
    ctx = create_ag_gemm_context(torch.empty(Mr, K, device="cuda", dtype=dtype), b, rank, world, max_M=Mr * world)
    if method is not None:
        ctx.all_gather_method = method
    for it in range(iters):
        a = torch.randn(Mr, K, device="cuda", dtype=dtype)
        full = torch.empty(Mr * world, K, device="cuda", dtype=dtype)
        dist.all_gather_into_tensor(full, a)
        ref = full.float() @ b.float().t()
        opt = (it % world, 2_000_000_000) if straggler else None
        c = ag_gemm(a, b, ctx, straggler_option=opt)
        torch.cuda.synchronize()
        torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-2, msg=lambda s: f"ag_gemm Mr={Mr} N={N} K={K} it={it}: {s}")
    ctx.finalize()


@case
def ag_gemm_shapes():
    _ag_gemm_case(128, 256, 256, torch.bfloat16)
    _ag_gemm_case(512, 1024, 2048, torch.bfloat16)
    _ag_gemm_case(999, 776, 520, torch.bfloat16)   # ragged: blocks straddle ranks
    _ag_gemm_case(64, 512, 1024, torch.float16)
    _ag_gemm_case(1024, 7168, 8192, torch.bfloat16, iters=2)
    _ag_gemm_case(512, 1024, 2048, torch.bfloat16, method="sm_pull_fused")
    _ag_gemm_case(999, 776, 520, torch.bfloat16, iters=4, method="sm_pull_fused")
    _ag_gemm_case(999, 776, 520, torch.bfloat16, iters=5, method="sm_push_fused")  # odd and even parities reused


@case
def ag_gemm_straggler():
    _ag_gemm_case(512, 1024, 1024, torch.bfloat16, iters=4, straggler=True)


def _gemm_rs_case(M, N, K, dtype, iters=3, nvls=None):
    rank, world = _rank_world()
    torch.manual_seed(4321 + rank)
    ctx = create_gemm_rs_context(M, N, rank, world, world, dtype)
    if nvls is not None:
        ctx.nvls = nvls
    b = torch.randn(N, K, device="cuda", dtype=dtype) * 0.05
    for it in range(iters):
        a = torch.randn(M, K, device="cuda", dtype=dtype) * 0.5 * (rank + 1)
        full = (a.float() @ b.float().t())
        ref = torch.empty(M // world, N, device="cuda", dtype=torch.float32)
        dist.reduce_scatter_tensor(ref, full)
        out = gemm_rs(a, b, ctx)
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), ref, rtol=6e-2, atol=6e-2 * world, msg=lambda s: f"gemm_rs M={M} N={N} K={K} nvls={ctx.nvls} it={it}: {s}")
    ctx.finalize()


@case
def gemm_rs_shapes():
    world = dist.get_world_size()
    _gemm_rs_case(128 * world, 256, 256, torch.bfloat16)
    _gemm_rs_case(512 * world, 1024, 512, torch.bfloat16)
    _gemm_rs_case(100 * world, 776, 520, torch.bfloat16)  # ragged: tiles straddle owners
    _gemm_rs_case(world, 512, 1024, torch.bfloat16)       # one row per rank (decode-like)
    _gemm_rs_case(64 * world, 512, 256, torch.float16)
    _gemm_rs_case(8192, 8192, 3584, torch.bfloat16, iters=2)
    if get_heap().has_multicast:  # the same shapes with the reduction inside the switch, and both modes on one context
        for nvls in (True, False):
            _gemm_rs_case(512 * world, 1024, 512, torch.bfloat16, nvls=nvls)
            _gemm_rs_case(100 * world, 776, 520, torch.bfloat16, nvls=nvls)
            _gemm_rs_case(64 * world, 512, 256, torch.float16, nvls=nvls)
        _gemm_rs_case(8192, 8192, 3584, torch.bfloat16, iters=2, nvls=True)


@case
def moe_tp_ag_group_gemm_and_reduce_rs():
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import (ag_group_gemm, create_ag_group_gemm_context, create_moe_rs_context,
                                                        moe_reduce_rs, select_experts)
    rank, world = _rank_world()
    group = U.TP_GROUP()
    for (Tr, topk, E, K, N, H) in ((64, 2, 8, 256, 128, 256), (256, 8, 32, 1024, 384, 1024), (100, 4, 16, 520, 200, 776)):
        T = Tr * world
        torch.manual_seed(100 + rank)
        a = torch.randn(Tr, K, device="cuda", dtype=torch.bfloat16)
        logits = torch.randn(Tr, E, device="cuda")
        torch.manual_seed(7)
        w1 = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.05   # this rank's N shard (same values on all ranks is fine)
        w2 = torch.randn(E, H, N, device="cuda", dtype=torch.bfloat16) * 0.05   # K shard of the down projection
        ids, wt = select_experts(group, world, topk, torch.bfloat16, "cuda", logits)
        ids_ref, wt_ref = ref.select_experts_ref(logits, topk, group)
        assert torch.equal(ids, ids_ref)
        ctx = create_ag_group_gemm_context(T, N, K, E, topk, torch.bfloat16, rank, world)
        rctx = create_moe_rs_context(group, world, T, H, E, topk, torch.bfloat16, torch.bfloat16)
        for it in range(3):
            up = ag_group_gemm(a, w1, ctx, ids)
            torch.cuda.synchronize()
            torch.testing.assert_close(up.float(), ref.ag_group_gemm_ref(a, w1, ids, group).float(), rtol=2e-2, atol=2e-2,
                                       msg=lambda s_: f"ag_group_gemm Tr={Tr} it={it}: {s_}")
            x = (up * (0.5 + rank)).contiguous()
            want_down = ref.moe_reduce_rs_ref(x, w2, ids, wt, group).float()
            for nvls in ([False, True] if get_heap().has_multicast else [False]):  # slots at the owner / sum in the switch
                rctx.nvls = nvls
                down = moe_reduce_rs(x, w2, ids, wt, rctx)
                torch.cuda.synchronize()
                torch.testing.assert_close(down.float(), want_down, rtol=5e-2, atol=5e-2 * world,
                                           msg=lambda s_: f"moe_reduce_rs Tr={Tr} nvls={nvls} it={it}: {s_}")
            rctx.nvls = False
        ctx.finalize()
        if K % 128 == 0 and N % 128 == 0:
            # block-scaled fp8 forms of both fusions against the bf16 oracles fed with the dequantised operands
            from triton_distributed_b200.kernels.nvidia import (ag_group_gemm_fp8, create_ag_group_gemm_fp8_context,
                                                                moe_reduce_rs_fp8, quantize_fp8_rows,
                                                                quantize_fp8_weight_blocks)

            def deq_w(w8_, sw_):
                n_ = w8_.shape[1]
                return (w8_.float() * sw_.repeat_interleave(128, 1)[:, :n_].repeat_interleave(128, 2)).to(torch.bfloat16)

            a8, sa = quantize_fp8_rows(a.float())
            w18, sw1 = quantize_fp8_weight_blocks(w1.float())
            w28, sw2 = quantize_fp8_weight_blocks(w2.float())
            a_deq = ref.fp8_dequant_ref(a8, sa, dtype=torch.bfloat16)
            fctx = create_ag_group_gemm_fp8_context(T, N, K, E, topk, torch.bfloat16, rank, world)
            for it in range(3):
                up8 = ag_group_gemm_fp8(a8, sa, w18, sw1, fctx, ids)
                torch.cuda.synchronize()
                torch.testing.assert_close(up8.float(), ref.ag_group_gemm_ref(a_deq, deq_w(w18, sw1), ids, group).float(),
                                           rtol=3e-2, atol=3e-2, msg=lambda s_: f"ag_group_gemm_fp8 Tr={Tr} it={it}: {s_}")
                x8, sx = quantize_fp8_rows(up8.float() * (0.5 + rank))
                x_deq = ref.fp8_dequant_ref(x8, sx, dtype=torch.bfloat16)
                down8 = moe_reduce_rs_fp8(x8, sx, w28, sw2, ids, wt, rctx)
                torch.cuda.synchronize()
                torch.testing.assert_close(down8.float(), ref.moe_reduce_rs_ref(x_deq, deq_w(w28, sw2), ids, wt, group).float(),
                                           rtol=5e-2, atol=5e-2 * world, msg=lambda s_: f"moe_reduce_rs_fp8 Tr={Tr} it={it}: {s_}")
            fctx.finalize()
        rctx.finalize()


@case
def ep_all_to_all_dispatch_combine():
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia import all_to_all_post_process, create_all_to_all_context, fast_all_to_all
    from triton_distributed_b200.layers.nvidia import EPAll2AllLayer
    rank, world = _rank_world()
    group = U.TP_GROUP()
    for (T, H, E, topk) in ((64, 256, 8 * world, 2), (128, 7168, 32 * world, 8)):
        torch.manual_seed(50 + rank)
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        logits = torch.randn(T, E, device="cuda")
        wt, ids = torch.topk(torch.softmax(logits, -1), topk, -1)
        ids = ids.to(torch.int32)
        # --- sorted-rows all-to-all (reference low-latency API) ---
        flat = ids.reshape(-1).long()
        order = torch.argsort(flat, stable=True)
        send = x.repeat_interleave(topk, 0)[order].contiguous()
        cum = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(torch.bincount(flat, minlength=E), 0)]).to(torch.int32)
        scale = torch.rand(send.shape[0], device="cuda")
        actx = create_all_to_all_context(T * topk, H, rank, E, world, E // world, torch.bfloat16)
        for it in range(3):
            splits, recv, rscale = fast_all_to_all(actx, send, cum, scale)
            torch.cuda.synchronize()
            want_splits, want_recv, want_scale = ref.fast_all_to_all_ref(send, cum, T * topk, group, scale[:, None])
            assert torch.equal(splits, want_splits), "splits"
            got, gscale = all_to_all_post_process(actx, splits, recv, rscale)
            want, wscale = ref.all_to_all_post_process_ref(T * topk, want_splits, want_recv, want_scale)
            assert torch.equal(got, want), f"fast_all_to_all rows it={it}"
            assert torch.equal(gscale, wscale.view(-1)), "scales"
        actx.finalize()
        # --- fused dispatch / combine layer ---
        for fp8 in (False, True):
            layer = EPAll2AllLayer(group, T, H, topk, rank, E, world, world, torch.bfloat16, fp8=fp8)
            for it in range(2):
                res = layer.dispatch(x, ids)
                torch.cuda.synchronize()
                sorted_ids, tile_expert, totals, rows_per_expert = layer.recv_plan()
                m_pad = int(totals[0])
                sel = sorted_ids[:m_pad]
                valid = sel < world * layer.max_m
                want_rows, want_expert, origin = ref.ep_dispatch_ref(x, ids, E, group)
                assert int(valid.sum()) == want_rows.shape[0], "received row count"
                exp_of_row = tile_expert[: m_pad // 128].repeat_interleave(128)[valid]
                assert torch.equal(exp_of_row, want_expert), "expert grouping"
                if fp8:
                    q, sc = res
                    rows = ref.fp8_dequant_ref(q[sel[valid].long()], sc[sel[valid].long()], dtype=torch.float32)
                    wq, ws = ref.fp8_quant_ref(want_rows)
                    torch.testing.assert_close(rows, ref.fp8_dequant_ref(wq, ws, dtype=torch.float32), rtol=0.13, atol=1e-3)  # one e4m3 ulp: tie rounding differs between converters
                    expert_out = torch.zeros(world * layer.max_m, H, device="cuda", dtype=torch.bfloat16)
                    expert_out[sel[valid].long()] = rows.to(torch.bfloat16)
                    tol = 0.1
                else:
                    assert torch.equal(res[sel[valid].long()], want_rows), "dispatched rows"
                    expert_out = res
                    tol = 2e-2
                back = layer.combine(expert_out, wt)
                torch.cuda.synchronize()
                torch.testing.assert_close(back.float(), x.float() * wt.sum(-1, keepdim=True), rtol=tol, atol=tol)
                if not fp8:
                    back2 = layer.combine(expert_out)
                    torch.testing.assert_close(back2.float(), x.float() * topk, rtol=2e-2, atol=2e-2 * topk)
            layer.finalize()


@case
def sp_flash_decode_and_allgather_layer():
    import math
    from triton_distributed_b200 import ref
    from triton_distributed_b200.layers.nvidia import AllGatherLayer, SpGQAFlashDecodeAttention
    rank, world = _rank_world()
    group = U.TP_GROUP()
    heap = get_heap()
    Hq, Hkv, D, page = 64, 8, 128, 16
    # packets over plain stores, packets over multimem, and the bulk exchange (forced for every batch size)
    for use_mc, bulk_rows in ([(False, None), (True, None), (False, 0)] if heap.has_multicast else [(False, None), (False, 0)]):
        layer = SpGQAFlashDecodeAttention(rank, 0, world, 1, Hq, Hkv, D, D, page_size=page, scale=1 / math.sqrt(D),
                                          max_allowed_batch=8, use_multicast=use_mc, bulk_rows=bulk_rows)
        for B, per_rank_len in ((1, 512), (8, 1000), (3, 37)):
            torch.manual_seed(9)  # same q on every rank
            q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
            torch.manual_seed(100 + rank)
            nb = (per_rank_len + page - 1) // page
            kc = torch.randn(B * nb, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
            vc = torch.randn_like(kc)
            bt = torch.randperm(B * nb, device="cuda").to(torch.int32).view(B, nb)
            lens = torch.randint(1, per_rank_len + 1, (B,), device="cuda", dtype=torch.int32)
            if rank == world - 1:
                lens[0] = 0  # a rank without tokens for sequence 0 must drop out of the merge
            all_lens = torch.empty(world, B, device="cuda", dtype=torch.int32)
            dist.all_gather_into_tensor(all_lens, lens, group=group)
            for it in range(2):
                out = layer(q, kc, vc, all_lens, bt)
                torch.cuda.synchronize()
                want = ref.sp_flash_decode_ref(q, kc, vc, lens, bt, 1 / math.sqrt(D), 0.0, group)
                torch.testing.assert_close(out.float(), want, rtol=5e-2, atol=2e-2, msg=lambda s_: f"sp decode B={B} mc={use_mc} bulk={bulk_rows} it={it}: {s_}")
        layer.finalize()
    ag = AllGatherLayer(1, world, rank, max_buffer_size=1 << 20)
    for fn in (ag.forward_pull, ag.forward_push_2d, ag.forward_push_2d_ll, ag.forward_push_2d_ll_multimem, ag.forward_push_numa_2d_ll):
        for n in (17 * 4, 4096):
            local = torch.arange(n, device="cuda", dtype=torch.float32) + 10000 * rank
            heap.barrier_all()
            got = fn(local).clone()
            torch.cuda.synchronize()
            want = ref.fast_allgather_ref(local, group)
            assert torch.equal(got, want), f"AllGatherLayer {fn.__name__}"
    ag.finalize()


@case
def reduce_scatter_op_and_moe_layers():
    from triton_distributed_b200.kernels.nvidia import create_reduce_scater_2d_ctx, reduce_scatter_2d_op
    from triton_distributed_b200.layers.nvidia import EP_MoE, TP_MoE
    rank, world = _rank_world()
    group = U.TP_GROUP()
    ctx = create_reduce_scater_2d_ctx(64 * world, 512, rank, world, world, torch.bfloat16)
    for it in range(3):
        torch.manual_seed(rank + it)
        x = torch.randn(64 * world, 512, device="cuda", dtype=torch.bfloat16)
        want = torch.empty(64, 512, device="cuda", dtype=torch.float32)
        dist.reduce_scatter_tensor(want, x.float(), group=group)
        got = reduce_scatter_2d_op(x, ctx)
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2 * world)
    ctx.finalize()
    # TP-MoE layer: sequence-sharded fused path vs the torch forward on replicated activations
    E, topk, H, I, T = 16, 4, 512, 256 * world, 64 * world
    torch.manual_seed(3)
    gate = torch.randn(E, H, device="cuda", dtype=torch.bfloat16)
    wgu = torch.randn(E, 2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.05
    wdn = torch.randn(E, H, I, device="cuda", dtype=torch.bfloat16) * 0.05
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    il = I // world
    sl = slice(rank * il, (rank + 1) * il)
    tp = TP_MoE(rank, world, group, topk, True)
    tp._init_parameters(gate, torch.cat([wgu[:, :I][:, sl], wgu[:, I:][:, sl]], dim=1), wdn[:, :, sl])
    tp._init_ctx(T)
    want = tp.torch_fwd(x)
    per = T // world
    for it in range(2):
        got = tp.dist_triton_fwd(x[rank * per:(rank + 1) * per].contiguous())
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want[rank * per:(rank + 1) * per].float(), rtol=5e-2, atol=0.1 * world)
    tp.finalize()
    # the same layer with both projections on the block-scaled fp8 fused kernels
    tp8 = TP_MoE(rank, world, group, topk, True, fp8=True)
    tp8._init_parameters(gate, torch.cat([wgu[:, :I][:, sl], wgu[:, I:][:, sl]], dim=1), wdn[:, :, sl])
    tp8._init_ctx(T)
    for it in range(2):
        got = tp8.dist_triton_fwd(x[rank * per:(rank + 1) * per].contiguous())
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want[rank * per:(rank + 1) * per].float(), rtol=0.12, atol=0.3 * world)
    tp8.finalize()
    # EP-MoE layer: every rank owns E / world whole experts
    for fp8, fp8_experts in ((False, False), (True, False), (True, True)):
        ep = EP_MoE(rank, world, group, E, topk, H, per, torch.bfloat16, True, fp8_dispatch=fp8, fp8_experts=fp8_experts)
        el = E // world
        ep._init_parameters(gate, wgu[rank * el:(rank + 1) * el].contiguous(), wdn[rank * el:(rank + 1) * el].contiguous())
        xl = x[rank * per:(rank + 1) * per].contiguous()
        want_l = ep.torch_fwd(xl, wgu, wdn)
        for it in range(2):
            got = ep.dist_triton_fwd(xl)
            torch.cuda.synchronize()
            torch.testing.assert_close(got.float(), want_l.float(), rtol=0.12 if fp8 else 5e-2, atol=(0.3 if fp8 else 0.1) * world)
        ep.finalize()


@case
def sp_ag_attention_prefill():
    from triton_distributed_b200.kernels.nvidia import create_sp_ag_attention_context_intra_node, fused_sp_ag_attn_intra_node
    from triton_distributed_b200.kernels.nvidia.sp_ag_attention_intra_node import zigzag_positions
    rank, world = _rank_world()
    Hq, Hkv, D = 8, 2, 128
    lens = [16 * world, 48 * world]
    torch.manual_seed(21)
    q = [torch.randn(L, Hq, D, device="cuda", dtype=torch.bfloat16) for L in lens]
    k = [torch.randn(L, Hkv, D, device="cuda", dtype=torch.bfloat16) for L in lens]
    v = [torch.randn(L, Hkv, D, device="cuda", dtype=torch.bfloat16) for L in lens]
    ctx = create_sp_ag_attention_context_intra_node(len(lens), Hq, Hkv, max(lens), max(lens) // world, D, torch.bfloat16,
                                                    torch.bfloat16, rank, world)
    pos = [zigzag_positions(L, rank, world, "cuda") for L in lens]
    q_sh = torch.cat([qq[p] for qq, p in zip(q, pos)])
    k_sh = torch.cat([kk[p] for kk, p in zip(k, pos)])
    v_sh = torch.cat([vv[p] for vv, p in zip(v, pos)])
    cu_q = torch.tensor([0] + [sum(l // world for l in lens[:i + 1]) for i in range(len(lens))], dtype=torch.int32)
    cu_k = torch.tensor([0] + [sum(lens[:i + 1]) for i in range(len(lens))], dtype=torch.int32)
    out = fused_sp_ag_attn_intra_node(ctx, q_sh, k_sh, v_sh, None, cu_q, cu_k, max(lens) // world, max(lens), rank, world)
    torch.cuda.synchronize()
    for i, L in enumerate(lens):
        full = torch.nn.functional.scaled_dot_product_attention(q[i].float().transpose(0, 1)[None], k[i].float().transpose(0, 1)[None],
                                                                v[i].float().transpose(0, 1)[None], is_causal=True, enable_gqa=True)[0].transpose(0, 1)
        torch.testing.assert_close(out[cu_q[i]:cu_q[i + 1]].float(), full[pos[i]], rtol=3e-2, atol=3e-2)
    ctx.finalize()


def main() -> int:
    U.initialize_distributed(seed=0, heap_bytes=int(os.environ.get("B200DIST_TEST_HEAP", 3 << 30)))
    rank, world = _rank_world()
    heap = get_heap()
    names = sys.argv[1:] or list(CASES)
    if rank == 0:
        print(f"[dist_cases] world={world} heap mode={heap.mode} multicast={heap.has_multicast}", flush=True)
    failed = 0
    # Verdicts travel over a gloo group so that a rank whose case failed early cannot collide with the NCCL
    # collectives its peers are still issuing; a watchdog ends the process if a case stalls.
    import datetime
    import threading
    verdict_group = dist.new_group(list(range(world)), backend="gloo", timeout=datetime.timedelta(seconds=120))
    case_budget_s = int(os.environ.get("B200DIST_CASE_TIMEOUT_S", "120"))
    for name in names:
        ok, err = True, ""
        dog = threading.Timer(case_budget_s, lambda n=name: (print(f"CASE {n} STALLED on rank {rank}: giving up", flush=True), os._exit(3)))
        dog.daemon = True
        dog.start()
        try:
            CASES[name]()
            torch.cuda.synchronize()
            heap.check_status(name)
        except Exception:  # noqa: BLE001
            ok, err = False, traceback.format_exc()
        verdicts = [None] * world
        try:
            dist.all_gather_object(verdicts, (ok, err), group=verdict_group)
        except Exception:  # noqa: BLE001
            print(f"CASE {name} FAIL (rank {rank}: verdict exchange failed)\n{err}", flush=True)
            os._exit(2)
        finally:
            dog.cancel()
        all_ok = all(v[0] for v in verdicts)
        if rank == 0:
            print(f"CASE {name} {'PASS' if all_ok else 'FAIL'}", flush=True)
            if not all_ok:
                for r, v in enumerate(verdicts):
                    if not v[0]:
                        print(f"--- rank {r} ---\n{v[1]}", flush=True)
        failed += 0 if all_ok else 1
        if not all_ok:
            break  # state after a failed collective case is not trustworthy
    U.finalize_distributed()
    return failed


if __name__ == "__main__":
    sys.exit(main())
