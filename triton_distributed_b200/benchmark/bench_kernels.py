"""Run ONE named fused kernel on a single GPU (world size 1: the GPU is its own only peer) for profiling and timing.

Every kernel executes its real code path (flag epochs, slot buffers, communication warps), so an
``ncu -k regex:<kernel>`` capture of this script shows the same instruction mix as a multi-rank run minus the NVLink
traffic. Sizes are small (a few hundred MB at most) so that a ``--set full`` capture ends by itself.

Example: ``python -m triton_distributed_b200.benchmark.bench_kernels --op ag_gemm --iters 3``
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from .. import ops, utils
from ..utils import perf_func_cold

OPS = ["ag_gemm", "gemm_rs", "grouped_gemm", "grouped_gemm_fp8", "ag_group_gemm", "moe_reduce_rs", "allreduce_rmsnorm", "ep_dispatch_combine",
       "decode_attn", "sp_decode", "moe_sort", "sampling", "rmsnorm", "qk_norm_rope"]


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", choices=OPS, required=True)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--m", type=int, default=4096, help="rows of the ag_gemm / gemm_rs problem")
    ap.add_argument("--n", type=int, default=0, help="ag_gemm / gemm_rs: N (0 = the Llama-3-70B TP8 default)")
    ap.add_argument("--k", type=int, default=0, help="ag_gemm / gemm_rs: K (0 = the Llama-3-70B TP8 default)")
    ap.add_argument("--kv-len", type=int, default=16384, help="KV length of the decode_attn / sp_decode problem")
    ap.add_argument("--splits", type=int, default=0, help="decode_attn: KV splits (0 = the library's choice)")
    args = ap.parse_args()
    os.environ.setdefault("RANK", "0"), os.environ.setdefault("LOCAL_RANK", "0"), os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"), os.environ.setdefault("MASTER_PORT", "29571")
    group = utils.initialize_distributed(seed=0, heap_bytes=2 << 30)
    from ..kernels import nvidia as K
    from ..layers.nvidia import EPAll2AllLayer, SpGQAFlashDecodeAttention
    dt = torch.bfloat16
    dev = "cuda"
    info = {}
    if args.op == "ag_gemm":
        M, N, K_ = args.m, args.n or 3584, args.k or 8192
        a = torch.randn(M, K_, device=dev, dtype=dt)
        b = torch.randn(N, K_, device=dev, dtype=dt) * 0.02
        ctx = K.create_ag_gemm_context(a, b, 0, 1, M)
        fn = lambda: K.ag_gemm(a, b, ctx)
        info = {"flops": 2.0 * M * N * K_}
    elif args.op == "gemm_rs":
        M, N, K_ = args.m, args.n or 8192, args.k or 3584
        a = torch.randn(M, K_, device=dev, dtype=dt)
        b = torch.randn(N, K_, device=dev, dtype=dt) * 0.02
        ctx = K.create_gemm_rs_context(M, N, 0, 1, 1, dt)
        fn = lambda: K.gemm_rs(a, b, ctx)
        info = {"flops": 2.0 * M * N * K_}
    elif args.op == "grouped_gemm_fp8":
        T, topk, E, H, I = 4096, 8, 128, 4096, 384
        ids = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(T)]).to(torch.int32)
        a8, sa = K.quantize_fp8_rows(torch.randn(T, H, device=dev))
        w8, sw = K.quantize_fp8_weight_blocks(torch.randn(E, I, H, device=dev) * 0.02)
        plan = K.create_sort_plan(T * topk, topk, E, 128, 1)
        fn = lambda: K.grouped_gemm_fp8(a8, sa, w8, sw, ids, plan=plan)
        info = {"flops": 2.0 * T * topk * I * H}
    elif args.op in ("grouped_gemm", "ag_group_gemm", "moe_reduce_rs"):
        T, topk, E, H, I = 4096, 8, 128, 4096, 384
        ids = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(T)]).to(torch.int32)
        wt = torch.rand(T, topk, device=dev)
        x = torch.randn(T, H, device=dev, dtype=dt)
        w1 = torch.randn(E, I, H, device=dev, dtype=dt) * 0.02
        if args.op == "grouped_gemm":
            fn = lambda: K.grouped_gemm(x, w1, ids)
            info = {"flops": 2.0 * T * topk * I * H}
        elif args.op == "ag_group_gemm":
            ctx = K.create_ag_group_gemm_context(T, I, H, E, topk, dt, 0, 1)
            fn = lambda: K.ag_group_gemm(x, w1, ctx, ids)
            info = {"flops": 2.0 * T * topk * I * H}
        else:
            act = torch.randn(T * topk, I // 2, device=dev, dtype=dt)
            w2 = torch.randn(E, H, I // 2, device=dev, dtype=dt) * 0.02
            ctx = K.create_moe_rs_context(group, 1, T, H, E, topk, dt, dt)
            fn = lambda: K.moe_reduce_rs(act, w2, ids, wt, ctx)
            info = {"flops": 2.0 * T * topk * H * (I // 2)}
    elif args.op == "allreduce_rmsnorm":
        rows, hidden = 8192, 8192
        x = torch.randn(rows, hidden, device=dev, dtype=dt)
        res = torch.randn(rows, hidden, device=dev, dtype=dt)
        g = torch.ones(hidden, device=dev, dtype=dt)
        ctx = K.create_allreduce_ctx(512 << 20, 0, 1, 1)
        fn = lambda: K.all_reduce_rmsnorm(x, res, g, 1e-6, ctx, K.allreduce.AllReduceMethod.TwoShot)
        info = {"bytes": 5.0 * rows * hidden * 2}
    elif args.op == "ep_dispatch_combine":
        T, H, E, topk = 4096, 7168, 256, 8
        x = torch.randn(T, H, device=dev, dtype=dt)
        ids = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(T)]).to(torch.int32)
        wt = torch.rand(T, topk, device=dev)
        layer = EPAll2AllLayer(group, T, H, topk, 0, E, 1, 1, dt, fp8=True)
        back = torch.zeros(layer.max_m, H, device=dev, dtype=dt)

        def fn():
            layer.dispatch(x, ids)
            return layer.combine(back, wt)
        info = {"bytes": T * H * 2.0 + T * topk * H * 1.0 + T * topk * H * 2.0 * 2 + T * H * 2.0}
    elif args.op in ("decode_attn", "sp_decode"):
        B, Hq, Hkv, D, page, L = 8, 64, 8, 128, 64, args.kv_len
        nb = L // page
        kc = torch.randn(B * nb, page, Hkv, D, device=dev, dtype=dt)
        vc = torch.randn_like(kc)
        bt = torch.arange(B * nb, device=dev, dtype=torch.int32).view(B, nb)
        lens = torch.full((B,), L, device=dev, dtype=torch.int32)
        q = torch.randn(B, Hq, D, device=dev, dtype=dt)
        info = {"bytes": 2.0 * kc.numel() * 2}
        if args.op == "decode_attn":
            S = args.splits or ops.choose_kv_splits(B, Hkv, Hq // Hkv, L)
            info["splits"] = S
            fn = lambda: ops.decode_attention(q, kc, vc, lens, bt, 1 / math.sqrt(D), 0.0, S)
        else:
            layer = SpGQAFlashDecodeAttention(0, 0, 1, 1, Hq, Hkv, D, D, page_size=page, scale=1 / math.sqrt(D), max_allowed_batch=B)
            fn = lambda: layer(q, kc, vc, lens[None], bt)
    elif args.op == "moe_sort":
        T, topk, E = 8192, 8, 128
        ids = torch.stack([torch.randperm(E, device=dev)[:topk] for _ in range(T)]).to(torch.int32)
        plan = K.create_sort_plan(T * topk, topk, E, 128, 1)
        fn = lambda: K.moe_sort(ids, plan)
    elif args.op == "sampling":
        logits = torch.randn(8, 151936, device=dev) * 3
        fn = lambda: ops.top_p_sample(logits, 0.6, 0.95)
    elif args.op == "rmsnorm":
        x = torch.randn(16384, 8192, device=dev, dtype=dt)
        g = torch.ones(8192, device=dev, dtype=dt)
        fn = lambda: ops.rmsnorm(x, g, 1e-6)
        info = {"bytes": 2.0 * x.numel() * 2}
    else:  # qk_norm_rope
        T, Hq, Hkv, D = 16384, 64, 8, 128
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev, dtype=dt)
        pos = torch.arange(T, device=dev, dtype=torch.int32) % 4096
        inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
        ang = torch.arange(4096, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        cs = torch.cat([ang.cos(), ang.sin()], -1).contiguous()
        kcache = torch.zeros(T, Hkv, D, device=dev, dtype=dt)
        vcache = torch.zeros_like(kcache)
        g = torch.ones(D, device=dev, dtype=dt)
        fn = lambda: ops.qk_norm_rope(qkv, pos, cs, Hq, Hkv, kcache, vcache, None, g, g)
        info = {"bytes": 2.0 * qkv.numel() * 2}
    _, ms, ts = perf_func_cold(fn, args.iters, args.warmup)
    utils.get_heap().check_status(args.op)
    out = {"op": args.op, "ms_min": min(ts), "ms_mean": ms}
    if "flops" in info:
        out["tflops"] = info["flops"] / min(ts) / 1e9
    if "bytes" in info:
        out["gbs"] = info["bytes"] / min(ts) / 1e6
    if "splits" in info:
        out["splits"] = info["splits"]
    print(json.dumps(out), flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
