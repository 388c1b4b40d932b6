"""Fused collectives against their NCCL (+ torch) compositions on N GPUs of one node.

  allreduce   bf16 sizes 8 KB ... 256 MB: every method of this library and its automatic choice vs ``dist.all_reduce``;
              fused all-reduce + residual + RMSNorm (hidden 8192) vs ``dist.all_reduce`` + torch residual / norm
  ep_a2a      expert-parallel dispatch + combine, 128 tokens per rank, hidden 7168, 32 experts per rank, top-8, fp8
              e4m3 rows with one fp32 scale per 128 channels vs two ``all_to_all_single`` calls per direction
  sp_decode   sequence-parallel flash-decode, 64 query / 8 KV heads, head dim 128, batch {1, 8, 32}, total KV length
              {32K, 128K, 1M} split over the ranks vs local decode attention + ``all_gather_into_tensor`` + combine
  tp_moe      Qwen3-235B-shaped tensor-parallel MoE (128 experts, top-8, hidden 4096, intermediate 1536 / world,
              8192 tokens): all-gather + grouped GEMM and grouped GEMM + top-k reduce + reduce-scatter vs the
              same grouped GEMM kernel around NCCL collectives

Every number is device-timed with CUDA events, L2 flushed before each call, reported as the maximum over ranks of the
per-rank minimum over iterations, one JSON line per row on rank 0.

Run: ``python -m torch.distributed.run --nproc-per-node N -m triton_distributed_b200.benchmark.bench_collectives --ops allreduce ep_a2a``
Role in the reference: the perf modes of ``test/nvidia/test_allreduce.py``, ``test_all_to_all.py``, ``test_sp_decode_attn.py``,
``test_ag_moe.py`` and ``test_moe_reduce_rs.py``.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch
import torch.distributed as dist

from .. import ops, utils
from ..kernels.allreduce import to_allreduce_method
from ..kernels.nvidia import (ag_group_gemm, all_reduce, all_reduce_rmsnorm, create_ag_group_gemm_context, create_allreduce_ctx,
                              create_moe_rs_context, grouped_gemm, moe_reduce_rs, select_experts)

LINK_GBS = 770.0   # measured peer copy per direction on this pool
HBM_GBS = 6531.9   # measured copy bandwidth


def _time(fn, iters, warmup, group):
    _, _, ts = utils.perf_func_cold(fn, iters, warmup)
    return utils.max_over_ranks(min(ts), group) * 1e3  # us


def bench_allreduce(args, group, rows):
    rank, world = dist.get_rank(), dist.get_world_size()
    heap = utils.get_heap()
    ctx = create_allreduce_ctx(min(512 << 20, max(args.ar_max_bytes, 64 << 20)), rank, world, world)
    methods = ["one_shot", "two_shot"] + (["one_shot_multimem", "two_shot_multimem"] if heap.has_multicast else [])
    nbytes = 8 << 10
    while nbytes <= args.ar_max_bytes:
        n = nbytes // 2
        x = torch.randn(n, device="cuda", dtype=torch.bfloat16)
        y = torch.empty_like(x)
        row = {"op": "allreduce", "world": world, "bytes": nbytes}
        row["nccl_us"] = _time(lambda: dist.all_reduce(y.copy_(x), group=group), args.iters, args.warmup, group)
        row["copy_us"] = _time(lambda: y.copy_(x), args.iters, args.warmup, group)  # the baseline's extra copy, for reference
        row["auto_us"] = _time(lambda: all_reduce(x, y, None, ctx), args.iters, args.warmup, group)
        for m in methods:
            if m.startswith("one_shot") and nbytes > (8 << 20):
                continue  # one-shot moves world x the data: not a candidate for large messages
            row[m + "_us"] = _time(lambda: all_reduce(x, y, to_allreduce_method(m), ctx), args.iters, args.warmup, group)
        # bytes that must cross a rank's links in the bandwidth-optimal algorithm: 2 (world - 1) / world of the message
        row["roofline_us"] = 2.0 * (world - 1) / world * nbytes / (LINK_GBS * 1e3)
        row["speedup"] = (row["nccl_us"] - row["copy_us"]) / row["auto_us"]
        rows.append(row)
        nbytes *= 4
    hidden = 8192
    for tokens in getattr(args, "ar_tokens", (8, 128, 2048, 8192)):
        x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
        g = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
        buf = torch.empty_like(x)

        def base():
            buf.copy_(x)
            dist.all_reduce(buf, group=group)
            h = buf + res
            hf = h.float()
            return (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * g, h

        row = {"op": "allreduce_residual_rmsnorm", "world": world, "tokens": tokens, "hidden": hidden}
        row["nccl_torch_us"] = _time(base, args.iters, args.warmup, group)
        row["ours_us"] = _time(lambda: all_reduce_rmsnorm(x, res.clone(), g, 1e-6, ctx, None), args.iters, args.warmup, group)
        row["speedup"] = row["nccl_torch_us"] / row["ours_us"]
        rows.append(row)
    ctx.finalize()


def bench_ep_a2a(args, group, rows):
    from ..layers.nvidia import EPAll2AllLayer
    rank, world = dist.get_rank(), dist.get_world_size()
    T, H, topk = args.ep_tokens, 7168, 8
    E = 32 * world
    torch.manual_seed(50 + rank)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    wt, ids = torch.topk(torch.softmax(logits, -1), topk, -1)
    ids = ids.to(torch.int32)
    layer = EPAll2AllLayer(group, T, H, topk, rank, E, world, world, torch.bfloat16, fp8=True)
    back = torch.randn(world * layer.max_m, H, device="cuda", dtype=torch.bfloat16)

    def ours():
        layer.dispatch(x, ids)
        return layer.combine(back, wt)

    # NCCL composition: the rows of every destination rank in one all_to_all_single (fp8 payload + scales), and the
    # bf16 rows back. Splits are exchanged once outside the timed region (the library path computes them in-kernel).
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    dest = (flat[order] // 32)
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    q8 = torch.randint(0, 255, (T * topk, H), device="cuda", dtype=torch.uint8)
    s32 = torch.rand(T * topk, H // 128, device="cuda")
    r8 = torch.empty(sum(rc), H, device="cuda", dtype=torch.uint8)
    rs32 = torch.empty(sum(rc), H // 128, device="cuda")
    ret_send = torch.randn(sum(rc), H, device="cuda", dtype=torch.bfloat16)
    ret_recv = torch.empty(T * topk, H, device="cuda", dtype=torch.bfloat16)

    def nccl():
        dist.all_to_all_single(r8, q8, rc, sc, group=group)
        dist.all_to_all_single(rs32, s32, rc, sc, group=group)
        dist.all_to_all_single(ret_recv, ret_send, sc, rc, group=group)
        return (ret_recv.view(T, topk, H).float() * wt[..., None]).sum(1).to(torch.bfloat16)

    row = {"op": "ep_dispatch_combine_fp8", "world": world, "tokens_per_rank": T, "hidden": H, "experts": E, "topk": topk}
    row["ours_us"] = _time(ours, args.iters, args.warmup, group)
    row["ours_dispatch_us"] = _time(lambda: layer.dispatch(x, ids), args.iters, args.warmup, group)
    row["nccl_a2a_us"] = _time(nccl, args.iters, args.warmup, group)
    out_bytes = T * topk * (H + H // 128 * 4) * (world - 1) / world   # dispatch payload leaving a rank (uniform routing)
    back_bytes = T * topk * H * 2 * (world - 1) / world
    row["roofline_us"] = (out_bytes + back_bytes) / (LINK_GBS * 1e3)
    row["speedup"] = row["nccl_a2a_us"] / row["ours_us"]
    rows.append(row)
    layer.finalize()


def bench_sp_decode(args, group, rows):
    from ..layers.nvidia import SpGQAFlashDecodeAttention
    rank, world = dist.get_rank(), dist.get_world_size()
    Hq, Hkv, D, page = 64, 8, 128, 64
    scale = 1 / math.sqrt(D)
    for B in getattr(args, "sp_batches", (1, 8, 32)):
        for total_kv in getattr(args, "sp_kv", (32 << 10, 128 << 10, 1 << 20)):
            per_rank = total_kv // world
            if B * per_rank * Hkv * D * 2 * 2 > (40 << 30):
                continue  # keep the KV cache of one rank below 40 GB
            nb = (per_rank + page - 1) // page
            kc = torch.randn(B * nb, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
            vc = torch.randn_like(kc)
            bt = torch.arange(B * nb, device="cuda", dtype=torch.int32).view(B, nb)
            lens = torch.full((B,), per_rank, device="cuda", dtype=torch.int32)
            all_lens = lens[None].expand(world, B).contiguous()
            q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
            layer = SpGQAFlashDecodeAttention(rank, 0, world, 1, Hq, Hkv, D, D, page_size=page, scale=scale, max_allowed_batch=B)
            S = ops.choose_kv_splits(B, Hkv, Hq // Hkv, per_rank)
            gathered_o = torch.empty(world, B * Hq, D, device="cuda", dtype=torch.float32)
            gathered_l = torch.empty(world, B * Hq, device="cuda", dtype=torch.float32)

            def base():
                o, lse = ops.decode_attention(q, kc, vc, lens, bt, scale, 0.0, S, return_lse=True)
                dist.all_gather_into_tensor(gathered_o, o.float().view(B * Hq, D), group=group)
                dist.all_gather_into_tensor(gathered_l, lse.view(B * Hq), group=group)
                return ops.combine_partials(gathered_o, gathered_l, torch.bfloat16)

            row = {"op": "sp_flash_decode", "world": world, "batch": B, "total_kv": total_kv}
            row["ours_us"] = _time(lambda: layer(q, kc, vc, all_lens, bt), args.iters, args.warmup, group)
            row["local_nccl_us"] = _time(base, args.iters, args.warmup, group)
            kv_bytes = 2.0 * B * per_rank * Hkv * D * 2
            row["roofline_us"] = kv_bytes / (HBM_GBS * 1e3)
            row["kv_tbs"] = kv_bytes / row["ours_us"] / 1e6
            row["speedup"] = row["local_nccl_us"] / row["ours_us"]
            rows.append(row)
            layer.finalize()
            del kc, vc
            torch.cuda.empty_cache()


def bench_tp_moe(args, group, rows):
    rank, world = dist.get_rank(), dist.get_world_size()
    E, topk, H, I, T = 128, 8, 4096, 1536, args.moe_tokens
    il = I // world
    Tr = T // world
    torch.manual_seed(100 + rank)
    a = torch.randn(Tr, H, device="cuda", dtype=torch.bfloat16)
    logits = torch.randn(Tr, E, device="cuda")
    torch.manual_seed(7)
    w1 = torch.randn(E, 2 * il, H, device="cuda", dtype=torch.bfloat16) * 0.02
    w2 = torch.randn(E, H, il, device="cuda", dtype=torch.bfloat16) * 0.02
    ids, wt = select_experts(group, world, topk, torch.bfloat16, "cuda", logits)
    ctx = create_ag_group_gemm_context(T, 2 * il, H, E, topk, torch.bfloat16, rank, world)
    rctx = create_moe_rs_context(group, world, T, H, E, topk, torch.bfloat16, torch.bfloat16)
    full = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)

    def base_up():
        dist.all_gather_into_tensor(full, a, group=group)
        return grouped_gemm(full, w1, ids)

    row = {"op": "ag_group_gemm", "world": world, "tokens": T, "experts": E, "topk": topk, "N": 2 * il, "K": H}
    row["ours_us"] = _time(lambda: ag_group_gemm(a, w1, ctx, ids), args.iters, args.warmup, group)
    row["nccl_grouped_us"] = _time(base_up, args.iters, args.warmup, group)
    row["speedup"] = row["nccl_grouped_us"] / row["ours_us"]
    rows.append(row)

    act = torch.randn(T * topk, il, device="cuda", dtype=torch.bfloat16) * 0.1
    out = torch.empty(Tr, H, device="cuda", dtype=torch.bfloat16)

    def base_down():
        y = grouped_gemm(act, w2, ids, a_per_pair=True, row_scale=wt)
        red = y.view(T, topk, H).sum(1)
        dist.reduce_scatter_tensor(out, red, group=group)
        return out

    row = {"op": "moe_reduce_rs", "world": world, "tokens": T, "experts": E, "topk": topk, "N": H, "K": il}
    row["ours_us"] = _time(lambda: moe_reduce_rs(act, w2, ids, wt, rctx), args.iters, args.warmup, group)
    if rctx.heap.has_multicast and world > 1:   # the other reduction mode of the same kernel, for the record
        rctx.nvls = not rctx.nvls
        row["nvls_us" if rctx.nvls else "slots_us"] = _time(lambda: moe_reduce_rs(act, w2, ids, wt, rctx), args.iters, args.warmup, group)
        rctx.nvls = not rctx.nvls
    row["grouped_nccl_us"] = _time(base_down, args.iters, args.warmup, group)
    row["speedup"] = row["grouped_nccl_us"] / row["ours_us"]
    rows.append(row)
    ctx.finalize()
    # block-scaled fp8 forms (the down-projection needs its K shard to be a multiple of 128)
    from ..kernels.nvidia import (ag_group_gemm_fp8, create_ag_group_gemm_fp8_context, moe_reduce_rs_fp8, quantize_fp8_rows,
                                  quantize_fp8_weight_blocks)
    a8, sa = quantize_fp8_rows(a.float())
    w18, sw1 = quantize_fp8_weight_blocks(w1.float())
    fctx = create_ag_group_gemm_fp8_context(T, 2 * il, H, E, topk, torch.bfloat16, rank, world)
    row = {"op": "ag_group_gemm_fp8", "world": world, "tokens": T, "experts": E, "topk": topk, "N": 2 * il, "K": H}
    row["ours_us"] = _time(lambda: ag_group_gemm_fp8(a8, sa, w18, sw1, fctx, ids), args.iters, args.warmup, group)
    row["bf16_fused_us"] = rows[-2]["ours_us"]
    rows.append(row)
    fctx.finalize()
    if il % 128 == 0:
        x8, sx = quantize_fp8_rows(act.float())
        w28, sw2 = quantize_fp8_weight_blocks(w2.float())
        row = {"op": "moe_reduce_rs_fp8", "world": world, "tokens": T, "experts": E, "topk": topk, "N": H, "K": il}
        row["ours_us"] = _time(lambda: moe_reduce_rs_fp8(x8, sx, w28, sw2, ids, wt, rctx), args.iters, args.warmup, group)
        row["bf16_fused_us"] = rows[-2]["ours_us"]
        rows.append(row)
    rctx.finalize()


BENCHES = {"allreduce": bench_allreduce, "ep_a2a": bench_ep_a2a, "sp_decode": bench_sp_decode, "tp_moe": bench_tp_moe}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ops", nargs="+", choices=list(BENCHES), default=list(BENCHES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ar-max-bytes", type=int, default=256 << 20)
    ap.add_argument("--ep-tokens", type=int, default=128)
    ap.add_argument("--moe-tokens", type=int, default=8192)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    group = utils.initialize_distributed(seed=0, heap_bytes=int(os.environ.get("B200DIST_BENCH_HEAP", 8 << 30)))
    rank = dist.get_rank()
    rows: list[dict] = []
    for name in args.ops:
        BENCHES[name](args, group, rows)
        utils.get_heap().check_status(name)
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                json.dump(rows, f, indent=1)
    utils.finalize_distributed()


if __name__ == "__main__":
    main()
