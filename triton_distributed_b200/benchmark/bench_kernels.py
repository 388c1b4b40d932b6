"""Run ONE named fused kernel on a single GPU (world size 1: the GPU is its own only peer) for profiling and timing.

Every kernel executes its real code path (flag epochs, slot buffers, communication warps), so an
``ncu -k regex:<kernel>`` capture of this script shows the same instruction mix as a multi-rank run minus the NVLink
traffic. Sizes are small (a few hundred MB at most) so that a ``--set full`` capture ends by itself.

Example: ``python -m triton_distributed_b200.benchmark.bench_kernels --op ag_gemm --iters 3``

``--op decode_step`` is different: it builds the first ``--layers`` layers of Qwen3-32B, captures one decode step of
``Engine`` (batch 8, prompt 2048) in a CUDA graph and prints the device time per kernel name from ``torch.profiler``
over a few replays (a timeline, not ncu). It also runs under torchrun on several GPUs.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from .. import ops, utils
from ..utils import perf_func_cold

OPS = ["decode_step", "prefill_attn", "gemm_skinny_fused", "ag_gemm", "gemm_rs", "grouped_gemm", "grouped_gemm_fp8", "ag_group_gemm", "moe_reduce_rs", "allreduce_rmsnorm", "ep_dispatch_combine",
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
    ap.add_argument("--layers", type=int, default=8, help="decode_step: transformer layers to build (64 = the full model)")
    ap.add_argument("--out", default=None, help="decode_step: text file for the table (rank 0)")
    ap.add_argument("--model", default="Qwen/Qwen3-32B", help="decode_step: architecture name (see models/config.py)")
    args = ap.parse_args()
    if args.op == "decode_step":
        return decode_step_table(args)
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
    elif args.op == "prefill_attn":
        B, S, Hq, Hkv, D = 8, args.kv_len if args.kv_len <= 8192 else 2048, 64, 8, 128
        q = torch.randn(B * S, Hq, D, device=dev, dtype=dt)
        k = torch.randn(B * S, Hkv, D, device=dev, dtype=dt)
        v = torch.randn_like(k)
        cu = torch.arange(0, (B + 1) * S, S, device=dev, dtype=torch.int32)
        fn = lambda: ops.prefill_attention(q, k, v, cu, cu, S, S, 1 / math.sqrt(D), True)
        info = {"flops": 4.0 * B * Hq * S * S * D / 2}
    elif args.op == "gemm_skinny_fused":
        M, H, Hq, Hkv, D = 8, 5120, 64, 8, 128
        x = torch.randn(M, H, device=dev, dtype=dt)
        w = torch.randn((Hq + 2 * Hkv) * D, H, device=dev, dtype=dt) * 0.02
        pos = torch.randint(0, 2000, (M,), device=dev, dtype=torch.int32)
        inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))
        ang = torch.arange(4096, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        cs = torch.cat([ang.cos(), ang.sin()], -1).contiguous()
        kcache = torch.zeros(64, Hkv, D, device=dev, dtype=dt)
        vcache = torch.zeros_like(kcache)
        qo = torch.zeros(M, Hq, D, device=dev, dtype=dt)
        g = torch.ones(D, device=dev, dtype=dt)
        ss = torch.full((16,), float(H), device=dev)
        ep = ops.skinny_row_scale(ss, H, 1e-6, base=ops.skinny_qkv_heads(pos, None, cs, Hq, Hkv, qo, kcache, vcache, g, g, 1e-6))
        fn = lambda: ops.gemm_skinny(x, w, epilogue=ep)
        info = {"bytes": 2.0 * w.numel()}
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
    utils.finalize_distributed()


def decode_step_table(args) -> None:
    """Device time per kernel of one captured decode step (see the module docstring)."""
    import torch.distributed as dist

    from ..models import Engine, ModelConfig
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29547")):
        os.environ.setdefault(k, v)
    group = utils.initialize_distributed(seed=0, heap_bytes=1 << 30)
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = ModelConfig(model_name=args.model, max_length=2048 + 256, rank=rank, world_size=world,
                      num_layers_override=args.layers)
    eng = Engine(cfg, temperature=0.6, top_p=0.95, group=group)
    prompt = torch.randint(0, eng.model.arch.vocab_size, (8, 2048), device="cuda")
    eng.prepare_decode(eng.prefill(prompt))
    for _ in range(4):
        eng.decode_one()
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    steps = max(args.iters, 4)
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(steps):
            eng.decode_one()
        torch.cuda.synchronize()
    if rank == 0:
        rows = []
        for e in prof.key_averages():
            t = getattr(e, "device_time_total", 0) or getattr(e, "cuda_time_total", 0)
            if t > 0 and e.device_type.name == "CUDA":
                rows.append((t / steps, e.count / steps, e.key[:90]))
        rows.sort(reverse=True)
        lines = [f"world={world} layers={args.layers}: total kernel us/step {sum(r[0] for r in rows):.1f}"]
        lines += [f"{t:10.1f} us/step  {c:7.1f} calls/step  {t / max(c, 1e-9):8.2f} us/call  {k}" for t, c, k in rows[:25]]
        print("\n".join(lines), flush=True)
        if args.out:
            os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
            with open(args.out, "w") as f:
                f.write("\n".join(lines) + "\n")
    if eng.graph is not None:
        eng.graph.reset()
        eng.graph = None
    torch.cuda.synchronize()
    utils.finalize_distributed()


if __name__ == "__main__":
    main()
