"""Worker body of the CPU multi-process tests: world_size ranks over gloo, fp32, seed 0."""
from __future__ import annotations

import os
import sys
import traceback

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _ag_gemm(rank, world):
    from triton_distributed_b200 import ref
    g = torch.Generator().manual_seed(0)
    A = torch.randn(world * 256, 512, generator=g)
    B = torch.randn(world, 1024 // world, 512, generator=g) * 0.02  # B_rank [N / world, K]
    a_local = A[rank * 256:(rank + 1) * 256]
    c = ref.ag_gemm_ref(a_local, B[rank])
    gathered = [torch.empty_like(a_local) for _ in range(world)]
    dist.all_gather(gathered, a_local)
    want = torch.cat(gathered) @ B[rank].t()
    torch.testing.assert_close(c, want, rtol=1e-5, atol=1e-5)
    assert c.shape == (world * 256, 1024 // world)


def _gemm_rs(rank, world):
    from triton_distributed_b200 import ref
    g = torch.Generator().manual_seed(0)
    A = torch.randn(512, 2048, generator=g)
    B = torch.randn(512, 2048, generator=g) * 0.02
    kper = 2048 // world
    a, b = A[:, rank * kper:(rank + 1) * kper], B[:, rank * kper:(rank + 1) * kper]
    out = ref.gemm_rs_ref(a.contiguous(), b.contiguous())
    full = A @ B.t()
    per = 512 // world
    torch.testing.assert_close(out, full[rank * per:(rank + 1) * per], rtol=1e-4, atol=1e-4)


def _all_reduce(rank, world):
    from triton_distributed_b200 import ref
    x = torch.full((8, 64), float(rank + 1))
    assert torch.all(ref.all_reduce_ref(x) == world * (world + 1) / 2)
    gam = torch.ones(64)
    y, h = ref.all_reduce_rmsnorm_ref(x, torch.ones(8, 64), gam, 1e-6)
    assert torch.allclose(h, torch.full((8, 64), world * (world + 1) / 2 + 1))
    assert torch.allclose(y, torch.ones(8, 64), atol=1e-4)
    ag = ref.fast_allgather_ref(torch.full((4,), float(rank)))
    assert ag.shape == (world, 4) and torch.equal(ag[:, 0], torch.arange(world, dtype=torch.float32))


def _ep_all_to_all(rank, world):
    """64 tokens/rank, hidden 256, 8 experts, top-2 from softmax of N(0,1) logits; checked against all_to_all_single
    semantics (rows grouped by destination) and dispatch∘combine == topk-sum."""
    from triton_distributed_b200 import ref
    torch.manual_seed(rank)
    T, H, E, topk = 64, 256, 8, 2
    x = torch.randn(T, H)
    logits = torch.randn(T, E)
    w, ids = torch.topk(torch.softmax(logits, -1), topk, -1)
    # low-latency all-to-all: rows sorted by expert
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    send = x.repeat_interleave(topk, 0)[order]
    counts = torch.bincount(flat, minlength=E)
    cum = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(counts, 0)]).to(torch.int32)
    splits, recv, _ = ref.fast_all_to_all_ref(send, cum, max_m=T * topk)
    out, _ = ref.all_to_all_post_process_ref(T * topk, splits, recv)
    # golden: gloo all_to_all via all_gather of padded per-destination chunks
    e_local = E // world
    chunks = []
    for d in range(world):
        lo, hi = int(cum[d * e_local]), int(cum[(d + 1) * e_local])
        chunks.append(send[lo:hi])
    sizes = torch.tensor([c.shape[0] for c in chunks])
    all_sizes = [torch.empty_like(sizes) for _ in range(world)]
    dist.all_gather(all_sizes, sizes)
    padded = torch.zeros(world, T * topk, H)
    for d, c in enumerate(chunks):
        padded[d, : c.shape[0]] = c
    allp = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(allp, padded)
    want = torch.cat([allp[s][rank, : int(all_sizes[s][rank])] for s in range(world)])
    torch.testing.assert_close(out, want, rtol=0, atol=0)
    assert int(splits.sum()) == want.shape[0]
    # dispatch -> identity experts -> combine == topk * x ; weighted combine == sum_k w x
    recv_rows, recv_expert, origin = ref.ep_dispatch_ref(x, ids, E)
    assert torch.all(recv_expert >= 0) and torch.all(recv_expert < e_local)
    back = ref.ep_combine_ref(recv_rows, origin, T, topk)
    torch.testing.assert_close(back, x * topk, rtol=1e-5, atol=1e-5)
    backw = ref.ep_combine_ref(recv_rows, origin, T, topk, topk_weight=w)
    torch.testing.assert_close(backw, x * w.sum(-1, keepdim=True), rtol=1e-5, atol=1e-5)


def _moe_tp(rank, world):
    from triton_distributed_b200 import ref
    torch.manual_seed(0)
    T, K, N, E, topk = 32 * world, 64, 48, 8, 2
    a = torch.randn(T, K)
    w1 = torch.randn(E, N, K) * 0.1
    logits = torch.randn(T, E)
    per = T // world
    ids, wt = ref.select_experts_ref(logits[rank * per:(rank + 1) * per], topk)
    assert ids.shape == (T, topk)
    up = ref.ag_group_gemm_ref(a[rank * per:(rank + 1) * per], w1, ids)
    want = torch.stack([a[t] @ w1[ids[t, k]].t() for t in range(T) for k in range(topk)])
    torch.testing.assert_close(up, want, rtol=1e-4, atol=1e-4)
    # down projection with K sharded over ranks
    kper = N // world
    w2 = torch.randn(E, 40, N) * 0.1
    out = ref.moe_reduce_rs_ref(up[:, rank * kper:(rank + 1) * kper].contiguous(), w2[:, :, rank * kper:(rank + 1) * kper].contiguous(), ids, wt)
    full = torch.stack([sum(wt[t, k] * (up[t * topk + k] @ w2[ids[t, k]].t()) for k in range(topk)) for t in range(T)])
    torch.testing.assert_close(out, full[rank * per:(rank + 1) * per], rtol=1e-3, atol=1e-3)


def _sp_decode(rank, world):
    from triton_distributed_b200 import ref
    torch.manual_seed(0)
    B, Hq, Hkv, D, page, Ltot = 2, 8, 2, 32, 4, 64 * world
    q = torch.randn(B, Hq, D)
    K = torch.randn(B, Ltot, Hkv, D)
    V = torch.randn(B, Ltot, Hkv, D)
    per = Ltot // world
    nb = per // page
    kc = K[:, rank * per:(rank + 1) * per].reshape(B * nb, page, Hkv, D)
    vc = V[:, rank * per:(rank + 1) * per].reshape(B * nb, page, Hkv, D)
    bt = torch.arange(B * nb, dtype=torch.int32).view(B, nb)
    lens = torch.tensor([per, per // 2 if rank == world - 1 else per], dtype=torch.int32)
    out = ref.sp_flash_decode_ref(q, kc, vc, lens, bt, D ** -0.5)
    for b in range(B):
        L = per * world if b == 0 else per * (world - 1) + per // 2
        k = K[b, :L].repeat_interleave(Hq // Hkv, 1)
        v = V[b, :L].repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("hd,lhd->hl", q[b], k) * D ** -0.5
        want = torch.einsum("hl,lhd->hd", torch.softmax(s, -1), v)
        torch.testing.assert_close(out[b], want, rtol=1e-4, atol=1e-4)


def _failure_detection(rank, world):
    """A rank that never joins a collective must surface as an error on the others, not as a hang."""
    import datetime
    pg = dist.new_group(list(range(world)), timeout=datetime.timedelta(seconds=2), backend="gloo")
    t = torch.ones(4)
    if rank == 0:
        return  # skips the collective
    try:
        dist.all_reduce(t, group=pg)
    except Exception:
        return
    raise AssertionError("all_reduce with a missing rank did not fail")


CASES = {"ag_gemm": _ag_gemm, "gemm_rs": _gemm_rs, "all_reduce": _all_reduce, "ep_all_to_all": _ep_all_to_all,
         "moe_tp": _moe_tp, "sp_decode": _sp_decode, "failure_detection": _failure_detection}


def worker(rank: int, world: int, port: int, name: str, errq) -> None:
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        CASES[name](rank, world)
        if name != "failure_detection":
            dist.barrier()
        errq.put((rank, None))
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
    finally:
        try:
            if name != "failure_detection":
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
