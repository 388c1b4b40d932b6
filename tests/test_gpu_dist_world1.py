"""Symmetric heap, primitives and fused collectives on ONE GPU (world size 1): every kernel runs its
real code path with itself as the only peer, which checks the tcgen05 mainloop, flag epochs and
buffer layouts without needing a second device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_heap_alloc_free_and_views(dist1):
    from triton_distributed_b200.runtime.heap import get_heap
    heap = get_heap()
    assert heap.world == 1 and heap.mode in ("vmm", "ipc")
    a = heap.create_tensor((1024, 64), torch.bfloat16)
    b = heap.create_tensor((7,), torch.float32)
    assert a.is_cuda and a.shape == (1024, 64) and float(a.abs().sum()) == 0.0
    a.fill_(1.5)
    b.fill_(2.0)
    torch.cuda.synchronize()
    assert float(a.float().sum()) == 1.5 * a.numel() and float(b.sum()) == 14.0
    views = heap.create_tensors((16,), torch.int32)
    assert len(views) == 1 and views[0].data_ptr() >= heap.base[0]
    live = heap.live_bytes()
    heap.free(a)
    assert heap.live_bytes() < live
    a2 = heap.create_tensor((1024, 64), torch.bfloat16)  # reuses the hole, zero-filled again
    assert float(a2.abs().sum()) == 0.0
    for t in (a2, b, views[0]):
        heap.free(t)
    heap.barrier_all()
    torch.cuda.synchronize()
    heap.check_status()


def test_bounded_wait_reports_timeout_instead_of_hanging(dist1):
    """A wait on a flag that nobody sets must come back with an error status."""
    from triton_distributed_b200 import _lib
    from triton_distributed_b200.runtime.heap import SymmTimeoutError, get_heap
    heap = get_heap()
    flags = heap.create_tensor((32,), torch.int32)
    ok = torch.ones(1, dtype=torch.int32, device="cuda")
    heap.set_timeout_ms(50)
    try:
        _lib.call("b200_test_wait", heap.ctx, _lib.ptr(flags), 4, 1, _lib.ptr(ok), _lib.stream_ptr())
        torch.cuda.synchronize()
        assert int(ok.item()) == 0
        with pytest.raises(SymmTimeoutError):
            heap.check_status("wait probe")
        # the context is still usable and a satisfied wait succeeds
        flags.fill_(1)
        _lib.call("b200_test_wait", heap.ctx, _lib.ptr(flags), 4, 1, _lib.ptr(ok), _lib.stream_ptr())
        torch.cuda.synchronize()
        assert int(ok.item()) == 1
        heap.check_status()
    finally:
        heap.set_timeout_ms(10000)
        heap.free(flags)


def test_grid_barrier_rounds(dist1):
    from triton_distributed_b200 import _lib
    from triton_distributed_b200.runtime.heap import get_heap
    heap = get_heap()
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad = torch.zeros(1, dtype=torch.int32, device="cuda")
    ctas, rounds, base = 64, 20, 0
    for _ in range(3):
        acc = torch.zeros(rounds, dtype=torch.int32, device="cuda")
        _lib.call("b200_test_grid_barrier", heap.ctx, _lib.ptr(counter), _lib.ptr(acc), rounds, ctas,
                  ctypes.c_uint32(base), _lib.ptr(bad), _lib.stream_ptr())
        base += rounds
    torch.cuda.synchronize()
    assert int(bad.item()) == 0
    heap.check_status()


@pytest.mark.parametrize("method", ["sm_push_fused", "sm_pull_fused"])
@pytest.mark.parametrize("Mr,N,K", [(256, 512, 256), (1000, 776, 520), (64, 256, 128)])
def test_ag_gemm_world1(dist1, Mr, N, K, method):
    from triton_distributed_b200.kernels.nvidia import ag_gemm, create_ag_gemm_context
    from triton_distributed_b200.runtime.heap import get_heap
    torch.manual_seed(0)
    a = torch.randn(Mr, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    ctx = create_ag_gemm_context(a, b, 0, 1, max_M=1024)
    ctx.all_gather_method = method
    for it in range(3):  # epochs / parity buffers across calls
        a2 = a * (it + 1)
        c = ag_gemm(a2, b, ctx)
        torch.cuda.synchronize()
        get_heap().check_status("ag_gemm")
        torch.testing.assert_close(c.float(), a2.float() @ b.float().t(), rtol=2e-2, atol=2e-2 * (it + 1))
    assert ctx.phase == 3
    ctx.finalize()


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1000, 776, 520), (8, 256, 1024)])
def test_gemm_rs_world1(dist1, M, N, K):
    from triton_distributed_b200.kernels.nvidia import create_gemm_rs_context, gemm_rs
    from triton_distributed_b200.runtime.heap import get_heap
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    ctx = create_gemm_rs_context(1024, N, 0, 1, 1, torch.bfloat16)
    for it in range(3):
        out = gemm_rs(a, b, ctx)
        torch.cuda.synchronize()
        get_heap().check_status("gemm_rs")
        torch.testing.assert_close(out.float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-2)
    ctx.finalize()


@pytest.mark.parametrize("method", ["one_shot", "two_shot", "double_tree"])
def test_allreduce_world1(dist1, method):
    from triton_distributed_b200.kernels.allreduce import to_allreduce_method
    from triton_distributed_b200.kernels.nvidia import all_reduce, all_reduce_rmsnorm, create_allreduce_ctx
    from triton_distributed_b200.runtime.heap import get_heap
    ctx = create_allreduce_ctx(1 << 20, 0, 1, 1)
    for n in (8, 4096, 300000):  # the last one is chunked
        x = torch.randn(n, device="cuda", dtype=torch.bfloat16)
        y = all_reduce(x, None, to_allreduce_method(method), ctx)
        torch.cuda.synchronize()
        get_heap().check_status("all_reduce")
        assert torch.equal(x, y)
    x = torch.randn(8, 5120, device="cuda", dtype=torch.bfloat16)
    res = torch.randn_like(x)
    g = torch.randn(5120, device="cuda", dtype=torch.bfloat16)
    res0 = res.clone()
    y, h = all_reduce_rmsnorm(x, res, g, 1e-6, ctx, to_allreduce_method(method))
    torch.cuda.synchronize()
    get_heap().check_status("all_reduce_rmsnorm")
    href = (x.float() + res0.float()).to(torch.bfloat16)
    torch.testing.assert_close(h, href)
    hf = href.float()
    torch.testing.assert_close(y.float(), hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * g.float(),
                               rtol=2e-2, atol=2e-2)
    ctx.finalize()


@pytest.mark.parametrize("mode", ["pull", "push2d", "push2d_ll"])
def test_fast_allgather_world1(dist1, mode):
    from triton_distributed_b200.kernels.nvidia import create_fast_allgather_context, fast_allgather
    from triton_distributed_b200.runtime.heap import get_heap
    heap = get_heap()
    ctx = create_fast_allgather_context(0, 0, 1, 1, max_buffer_size=1 << 20)
    buf = heap.create_tensor((4096,), torch.float32)
    buf.copy_(torch.arange(4096, device="cuda", dtype=torch.float32))
    fast_allgather(buf, ctx, mode=mode)
    torch.cuda.synchronize()
    heap.check_status("fast_allgather")
    assert torch.equal(buf, torch.arange(4096, device="cuda", dtype=torch.float32))
    heap.free(buf)
    ctx.finalize()


@pytest.mark.parametrize("bulk_rows", [None, 0])
def test_sp_flash_decode_world1(dist1, bulk_rows):
    import math
    from triton_distributed_b200 import ref
    from triton_distributed_b200.layers.nvidia import SpGQAFlashDecodeAttention
    from triton_distributed_b200.runtime.heap import get_heap
    torch.manual_seed(0)
    B, Hq, Hkv, D, page, L = 4, 32, 4, 128, 16, 700
    layer = SpGQAFlashDecodeAttention(0, 0, 1, 1, Hq, Hkv, D, D, page_size=page, scale=1 / math.sqrt(D), max_allowed_batch=4,
                                      bulk_rows=bulk_rows)
    nb = (L + page - 1) // page
    kc = torch.randn(B * nb, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    bt = torch.randperm(B * nb, device="cuda").to(torch.int32).view(B, nb)
    lens = torch.randint(1, L + 1, (1, B), device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    for splits in (-1, 1, 5):
        out = layer(q, kc, vc, lens, bt, kv_split=splits)
        torch.cuda.synchronize()
        get_heap().check_status("sp decode")
        want, _ = ref.paged_decode_attention_ref(q, kc, vc, lens[0], bt, 1 / math.sqrt(D))
        torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)
    layer.finalize()


@pytest.mark.parametrize("zigzag", [True, False])
def test_sp_ag_attention_world1(dist1, zigzag):
    """Context-parallel prefill with one rank: the K/V scatter kernel writes rows in global order (the identity here) and
    the zig-zag split turns every sequence into two causal problems with prefixes of different length."""
    from triton_distributed_b200.kernels.nvidia import create_sp_ag_attention_context_intra_node, fused_sp_ag_attn_intra_node
    torch.manual_seed(3)
    Hq, Hkv, D = 8, 2, 128
    lens = [64, 384, 130 * 2]
    q = torch.randn(sum(lens), Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sum(lens), Hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sum(lens), Hkv, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    ctx = create_sp_ag_attention_context_intra_node(len(lens), Hq, Hkv, max(lens), max(lens), D, torch.bfloat16, torch.bfloat16, 0, 1)
    for _ in range(2):
        out = fused_sp_ag_attn_intra_node(ctx, q, k, v, None, cu, cu, max(lens), max(lens), 0, 1, True, zigzag)
    torch.cuda.synchronize()
    for b, L in enumerate(lens):
        s = slice(int(cu[b]), int(cu[b + 1]))
        want = torch.nn.functional.scaled_dot_product_attention(
            q[s].float().transpose(0, 1)[None], k[s].float().transpose(0, 1)[None], v[s].float().transpose(0, 1)[None],
            is_causal=True, enable_gqa=True)[0].transpose(0, 1)
        torch.testing.assert_close(out[s].float(), want, rtol=3e-2, atol=3e-2)
    ctx.finalize()


def test_shmem_device_api_world1(dist1):
    """broadcast / fcollect / putmem_signal_warp / int_p / barrier_all_warp with the GPU as its own only peer."""
    from triton_distributed_b200 import _lib
    from triton_distributed_b200.runtime.heap import get_heap
    heap = get_heap()
    n4 = 256
    n = n4 * 4
    bcast, ring = heap.create_tensor((n,), torch.float32), heap.create_tensor((n,), torch.float32)
    coll = heap.create_tensor((1, n), torch.float32)
    sig, word, flags = heap.create_tensor((2,), torch.int32), heap.create_tensor((1,), torch.int32), heap.create_tensor((16,), torch.int32)
    ok = torch.zeros(1, dtype=torch.int32, device="cuda")
    for it in (1, 2):
        src = torch.arange(n, device="cuda", dtype=torch.float32) + it
        _lib.call("b200_test_shmem_api", heap.ctx, _lib.ptr(src), _lib.ptr(bcast), _lib.ptr(coll), _lib.ptr(ring), _lib.ptr(sig),
                  _lib.ptr(word), _lib.ptr(flags), n4, 0, it, _lib.ptr(ok), _lib.stream_ptr())
        torch.cuda.synchronize()
        assert int(ok.item()) == 1
        assert torch.equal(bcast, src) and torch.equal(coll[0], src) and torch.equal(ring, src) and int(word[0]) == it
    heap.check_status()
    for t in (flags, word, sig, coll, ring, bcast):
        heap.free(t)
