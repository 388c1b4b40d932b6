"""Tutorial 04 - expert-parallel dispatch and combine with fp8 rows (DeepSeek-style inference all-to-all).

Every rank routes its tokens to top-k of E experts; expert e lives on rank e // (E / world). ``EPAll2AllLayer.dispatch``
sorts the (token, k) pairs by expert, quantises every row to e4m3 with one fp32 scale per 128 channels (scale = amax /
448) and writes it straight into the expert rank's receive buffer; ``combine`` returns every expert's output row to
the token's rank and sums the k copies with the routing weights. Both are one kernel each, with no host polling.

The script runs an identity "expert" (dequantise, multiply by the local expert's index + 1), and checks the result
against the same computation done on one rank with plain PyTorch.

    bash launch.sh --nproc 8 tutorials/04_ep_all2all_fp8.py

Reference counterpart: ``tutorials/04-deepseek-infer-all2all.py``.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from triton_distributed_b200 import utils
from triton_distributed_b200.layers.nvidia import EPAll2AllLayer


def quant_dequant(x: torch.Tensor) -> torch.Tensor:
    """bf16 [T, H] -> what a receiver reconstructs from e4m3 rows with per-128 scales."""
    T, H = x.shape
    g = x.float().view(T, H // 128, 128)
    scale = g.abs().amax(-1, keepdim=True) / 448.0
    q = (g / scale.clamp_min(1e-30)).to(torch.float8_e4m3fn).float()
    return (q * scale).view(T, H)


def main() -> None:
    for k, v in (("RANK", "0"), ("LOCAL_RANK", "0"), ("WORLD_SIZE", "1"), ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29574")):
        os.environ.setdefault(k, v)
    group = utils.initialize_distributed(seed=0, heap_bytes=2 << 30)
    rank, world = dist.get_rank(), dist.get_world_size()
    T, H, topk, e_local = 128, 7168, 8, 32
    E = e_local * world
    torch.manual_seed(100 + rank)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    weight, ids = torch.topk(torch.softmax(torch.randn(T, E, device="cuda"), -1), topk, -1)
    ids = ids.to(torch.int32)
    layer = EPAll2AllLayer(group, T, H, topk, rank, E, world, world, torch.bfloat16, fp8=True)

    rows, scales = layer.dispatch(x, ids)                      # e4m3 [world * max_m, H], fp32 [world * max_m, H / 128]
    sorted_ids, tile_expert, totals, rows_per_expert = layer.recv_plan()   # rows grouped by local expert (device side)
    # the "expert": dequantise and scale by (local expert index + 1); a real model runs a grouped GEMM over recv_plan()
    deq = (rows.float().view(rows.shape[0], H // 128, 128) * scales[..., None]).view(rows.shape[0], H)
    factor = torch.zeros(rows.shape[0], device="cuda")
    n_tiles = int(totals[1])
    for t in range(n_tiles):                                    # host loop for clarity only
        idx = sorted_ids[t * 128:(t + 1) * 128].long()
        idx = idx[idx < rows.shape[0]]
        factor[idx] = float(tile_expert[t]) + 1.0
    expert_out = (deq * factor[:, None]).to(torch.bfloat16)
    out = layer.combine(expert_out, weight)                     # [T, H]
    torch.cuda.synchronize()
    utils.get_heap().check_status("ep all-to-all")

    local_index = (ids % e_local).float() + 1.0                 # what every chosen expert multiplies by
    want = quant_dequant(x)[:, None, :] * (local_index * weight)[..., None]
    want = want.sum(1)
    # e4m3 has a 6 % step: a value that sits on a rounding boundary may land one step away from the PyTorch cast, so the
    # check is on the error norm and on the fraction of elements that agree closely, not element by element
    err = (out.float() - want).norm() / want.norm()
    close = torch.isclose(out.float(), want, rtol=3e-2, atol=3e-2).float().mean()
    assert err < 1e-2 and close > 0.99, (float(err), float(close))
    utils.dist_print(f"tutorial 04: {T} tokens/rank x top-{topk} over {E} experts on {world} rank(s): dispatch + combine match",
                     allowed_ranks=[0])
    layer.finalize()
    utils.finalize_distributed()


if __name__ == "__main__":
    main()
