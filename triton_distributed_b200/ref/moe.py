"""Reference semantics of the MoE building blocks: routing, index/sort metadata, grouped GEMMs fused with
all-gather / reduce-scatter, expert-parallel all-to-all, and fp8 block quantisation."""
from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def _rank(group) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def _all_gather_cat(t: torch.Tensor, group) -> torch.Tensor:
    world = _world(group)
    if world == 1:
        return t
    outs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(outs, t.contiguous(), group=group)
    return torch.cat(outs, dim=0)


# ------------------------------------------------------------------------------------------------
# routing and index metadata
# ------------------------------------------------------------------------------------------------
def select_experts_ref(router_logits: torch.Tensor, topk: int, group=None, renormalize: bool = False):
    """softmax -> top-k on the local tokens, then all-gather: (ids int32 [T, topk], weights fp32 [T, topk])."""
    probs = torch.softmax(router_logits.float(), dim=-1)
    w, ids = torch.topk(probs, topk, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return _all_gather_cat(ids.to(torch.int32), group), _all_gather_cat(w, group)


def calc_gather_scatter_index_ref(chosen_experts: torch.Tensor, num_experts: int, alignment: int = 1):
    """Sort the (token, k) pairs by expert (stable), padding every expert's run to a multiple of `alignment`.

    Returns (tokens_by_expert [E], scatter_index [T, topk] = position of each pair in the sorted order,
    gather_index [M_pad] = flat pair index at each position (pad = T * topk), expert_index [M_pad / alignment]
    = expert of every `alignment`-row tile, M_pad)."""
    T, topk = chosen_experts.shape
    flat = chosen_experts.reshape(-1).long().cpu()
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + alignment - 1) // alignment * alignment
    starts = torch.cumsum(padded, 0) - padded
    m_pad = int(padded.sum())
    gather = torch.full((m_pad,), T * topk, dtype=torch.int32)
    scatter = torch.empty(T * topk, dtype=torch.int32)
    order = torch.argsort(flat, stable=True)
    pos_in_expert = torch.arange(T * topk) - torch.repeat_interleave(torch.cumsum(counts, 0) - counts, counts)
    dest = starts[flat[order]] + pos_in_expert
    gather[dest] = order.to(torch.int32)
    scatter[order] = dest.to(torch.int32)
    expert_index = torch.repeat_interleave(torch.arange(num_experts), padded // alignment).to(torch.int32)
    dev = chosen_experts.device
    return (counts.to(torch.int32).to(dev), scatter.view(T, topk).to(dev), gather.to(dev), expert_index.to(dev), m_pad)


def moe_align_block_size_ref(topk_ids: torch.Tensor, num_experts: int, block_m: int, num_ranks: int = 1):
    """Row-wise MoE+RS metadata: every source-rank block of ``T / num_ranks`` tokens is sorted by expert on its own and
    every expert run is padded to `block_m`.

    Returns (sorted_token_ids [M_pad] flat pair indices (pad = T * topk), expert_ids [tiles], block_barrier_ids [tiles]
    = source rank of every tile, rank_block_num [num_ranks] tiles per rank, num_tokens_post_pad)."""
    T, topk = topk_ids.shape
    per = T // num_ranks
    ids_all, experts_all, ranks_all, per_rank_tiles = [], [], [], []
    for r in range(num_ranks):
        blk = topk_ids[r * per:(r + 1) * per]
        _, _, gather, expert_index, _ = calc_gather_scatter_index_ref(blk, num_experts, block_m)
        gather = gather.clone().long().cpu()
        valid = gather < per * topk
        gather[valid] += r * per * topk
        gather[~valid] = T * topk
        ids_all.append(gather)
        experts_all.append(expert_index.cpu())
        ranks_all.append(torch.full((expert_index.numel(),), r, dtype=torch.int32))
        per_rank_tiles.append(expert_index.numel())
    dev = topk_ids.device
    sorted_ids = torch.cat(ids_all).to(torch.int32).to(dev)
    return (sorted_ids, torch.cat(experts_all).to(torch.int32).to(dev), torch.cat(ranks_all).to(dev),
            torch.tensor(per_rank_tiles, dtype=torch.int32, device=dev), int(sorted_ids.numel()))


def ag_moe_tile_schedule_ref(topk_ids: torch.Tensor, num_experts: int, block_m: int, rank: int, world: int):
    """AG+MoE metadata: pairs sorted by expert (stable, so by source rank inside an expert), runs padded to `block_m`.
    A tile needs the token shards of ranks seg_start..seg_end; its stage is the step of a ring starting at `rank` after
    which all of them have arrived: ``(seg_end - rank) mod world``, or ``world - 1`` when the range runs past
    ``rank - 1`` (the last shard to arrive). Tiles are issued stage-major, in their
    original (expert-major) order inside a stage.

    Returns (gather_index [M_pad], tile_expert [tiles], tile_seg_start, tile_seg_end, tile_order [tiles])."""
    T, topk = topk_ids.shape
    per = T // world
    _, _, gather, expert_index, _ = calc_gather_scatter_index_ref(topk_ids, num_experts, block_m)
    g = gather.cpu().long().view(-1, block_m)
    valid = g < T * topk
    src = torch.where(valid, (g // topk) // per, torch.full_like(g, -1))
    seg_end = src.max(dim=1).values
    seg_start = torch.where(valid, src, torch.full_like(src, world)).min(dim=1).values
    stage = (seg_end - rank) % world
    stage = torch.where((seg_start - rank) % world > stage, torch.full_like(stage, world - 1), stage)
    order = torch.argsort(stage, stable=True)
    dev = topk_ids.device
    return (gather, expert_index, seg_start.to(torch.int32).to(dev), seg_end.to(torch.int32).to(dev),
            order.to(torch.int32).to(dev))


# ------------------------------------------------------------------------------------------------
# grouped GEMMs
# ------------------------------------------------------------------------------------------------
def grouped_gemm_ref(a_rows: torch.Tensor, w: torch.Tensor, expert_of_row: torch.Tensor) -> torch.Tensor:
    """out[i] = a_rows[i] @ w[expert_of_row[i]].T with w [E, N, K]."""
    out = torch.zeros((a_rows.shape[0], w.shape[1]), dtype=torch.float32, device=a_rows.device)
    for e in range(w.shape[0]):
        m = expert_of_row == e
        if bool(m.any()):
            out[m] = a_rows[m].float() @ w[e].float().t()
    return out


def dequant_fp8_rows(a8: torch.Tensor, a_scale: torch.Tensor) -> torch.Tensor:
    """e4m3 [T, K] with fp32 scales [T, K / 128] -> fp32 [T, K]."""
    T, K = a8.shape
    return (a8.float().view(T, K // 128, 128) * a_scale[:, :, None]).view(T, K)


def dequant_fp8_weight_blocks(w8: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """e4m3 [E, N, K] with fp32 scales [E, ceil(N / 128), K / 128] (one per 128 x 128 block) -> fp32 [E, N, K]."""
    E, N, K = w8.shape
    s = w_scale.repeat_interleave(128, dim=1)[:, :N].repeat_interleave(128, dim=2)
    return w8.float() * s


def grouped_gemm_fp8_ref(a8_rows: torch.Tensor, a_scale_rows: torch.Tensor, w8: torch.Tensor, w_scale: torch.Tensor,
                         expert_of_row: torch.Tensor) -> torch.Tensor:
    """Block-scaled fp8 grouped GEMM in fp32: out[i] = dequant(a8_rows[i]) @ dequant(w8[expert_of_row[i]]).T."""
    return grouped_gemm_ref(dequant_fp8_rows(a8_rows, a_scale_rows), dequant_fp8_weight_blocks(w8, w_scale), expert_of_row)


def ag_group_gemm_ref(a_local: torch.Tensor, w: torch.Tensor, full_topk_ids: torch.Tensor, group=None) -> torch.Tensor:
    """TP-MoE up-projection: tokens all-gathered, every (token, k) pair multiplied by its expert's weight shard.
    a_local [T / world, K]; w [E, N_local, K]; returns [T * topk, N_local] with row t * topk + k."""
    a = _all_gather_cat(a_local, group)
    topk = full_topk_ids.shape[1]
    rows = a.repeat_interleave(topk, dim=0)
    return grouped_gemm_ref(rows, w, full_topk_ids.reshape(-1).long()).to(a_local.dtype)


def moe_reduce_rs_ref(x: torch.Tensor, w: torch.Tensor, topk_ids: torch.Tensor, topk_weight: torch.Tensor, group=None):
    """TP-MoE down-projection: x [T * topk, K_local] times w [E, N, K_local], scaled by the routing weight, summed over
    the k choices of a token and reduce-scattered over ranks -> [T / world, N]."""
    T, topk = topk_ids.shape
    out = grouped_gemm_ref(x, w, topk_ids.reshape(-1).long()) * topk_weight.reshape(-1, 1).float()
    tok = out.view(T, topk, -1).sum(1)
    world = _world(group)
    if world > 1:
        dist.all_reduce(tok, group=group)
        per = T // world
        tok = tok[_rank(group) * per:(_rank(group) + 1) * per]
    return tok.to(x.dtype)


# ------------------------------------------------------------------------------------------------
# fp8 block quantisation (1 x 128 blocks, scale = amax / 448, as in the reference's all-to-all tutorial)
# ------------------------------------------------------------------------------------------------
def fp8_quant_ref(x: torch.Tensor, block: int = 128):
    """x [T, H] -> (q e4m3 [T, H], scale fp32 [T, H / block]) with x ~= q * scale."""
    T, H = x.shape
    xb = x.float().view(T, H // block, block)
    scale = xb.abs().amax(-1) / 448.0
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = (xb / safe[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(T, H)
    return q, scale


def fp8_dequant_ref(q: torch.Tensor, scale: torch.Tensor, block: int = 128, dtype=torch.bfloat16) -> torch.Tensor:
    T, H = q.shape
    return (q.float().view(T, H // block, block) * scale[..., None]).view(T, H).to(dtype)


# ------------------------------------------------------------------------------------------------
# expert-parallel all-to-all
# ------------------------------------------------------------------------------------------------
def fast_all_to_all_ref(send: torch.Tensor, send_split_cumsum: torch.Tensor, max_m: int, group=None,
                        send_scale: torch.Tensor | None = None):
    """Low-latency all-to-all: `send` [n, H] is sorted by (global) expert, `send_split_cumsum` [E + 1] delimits the
    experts. Rank d receives, from every source s, the rows of its own experts, at rows ``s * max_m ...`` of the
    receive buffer. Returns (recv_splits int32 [world, E_local], recv_buf [world * max_m, H], recv_scale | None)."""
    world, rank = _world(group), _rank(group)
    E = send_split_cumsum.numel() - 1
    e_local = E // world
    splits = (send_split_cumsum[1:] - send_split_cumsum[:-1]).to(torch.int32)
    all_splits = _all_gather_cat(splits[None], group)              # [world(src), E]
    all_cum = _all_gather_cat(send_split_cumsum[None].to(torch.int64), group)
    recv = torch.zeros((world * max_m, send.shape[1]), dtype=send.dtype, device=send.device)
    recv_scale = None
    if send_scale is not None:
        recv_scale = torch.zeros((world * max_m, *send_scale.shape[1:]), dtype=send_scale.dtype, device=send.device)
    # gather every source's send buffer (padded to a common length) and cut out what is addressed to this rank
    n_max = int(_all_gather_cat(torch.tensor([send.shape[0]], device=send.device), group).max())
    pad = torch.zeros((n_max, send.shape[1]), dtype=send.dtype, device=send.device)
    pad[: send.shape[0]] = send
    bufs = _all_gather_cat(pad[None], group)
    if send_scale is not None:
        spad = torch.zeros((n_max, *send_scale.shape[1:]), dtype=send_scale.dtype, device=send.device)
        spad[: send.shape[0]] = send_scale
        sbufs = _all_gather_cat(spad[None], group)
    for s in range(world):
        lo = int(all_cum[s, rank * e_local])
        hi = int(all_cum[s, (rank + 1) * e_local])
        recv[s * max_m: s * max_m + hi - lo] = bufs[s, lo:hi]
        if send_scale is not None:
            recv_scale[s * max_m: s * max_m + hi - lo] = sbufs[s, lo:hi]
    recv_splits = all_splits[:, rank * e_local:(rank + 1) * e_local].contiguous()
    return recv_splits, recv, recv_scale


def all_to_all_post_process_ref(max_m: int, recv_splits: torch.Tensor, recv_buf: torch.Tensor,
                                scale_buf: torch.Tensor | None = None):
    """Compact the per-source segments of the receive buffer into one tensor (source-major)."""
    per_src = recv_splits.sum(dim=1)
    rows = [recv_buf[s * max_m: s * max_m + int(n)] for s, n in enumerate(per_src)]
    out = torch.cat(rows)
    sc = None
    if scale_buf is not None:
        sc = torch.cat([scale_buf[s * max_m: s * max_m + int(n)] for s, n in enumerate(per_src)])
    return out, sc


def ep_dispatch_ref(x: torch.Tensor, topk_ids: torch.Tensor, num_experts: int, group=None):
    """Expert-parallel dispatch: every (token, k) pair travels to the rank that owns expert ``topk_ids[t, k]``.
    Returns (recv [n_recv, H] grouped by local expert then source rank then source order, recv_expert [n_recv] local
    expert id, origin [n_recv, 3] = (source rank, token, k))."""
    world, rank = _world(group), _rank(group)
    e_local = num_experts // world
    T, topk = topk_ids.shape
    xs = _all_gather_cat(x[None], group)                                  # [world, T, H] (equal T per rank)
    ids = _all_gather_cat(topk_ids[None].to(torch.int64), group)          # [world, T, topk]
    rows, experts, origin = [], [], []
    for e in range(rank * e_local, (rank + 1) * e_local):
        for s in range(world):
            tk = torch.nonzero(ids[s] == e)                               # in (token, k) order
            if tk.numel():
                rows.append(xs[s, tk[:, 0]])
                experts.append(torch.full((tk.shape[0],), e - rank * e_local, dtype=torch.int32, device=x.device))
                origin.append(torch.cat([torch.full((tk.shape[0], 1), s, device=x.device), tk], dim=1))
    if not rows:
        return (x.new_zeros((0, x.shape[1])), torch.zeros(0, dtype=torch.int32, device=x.device),
                torch.zeros((0, 3), dtype=torch.int64, device=x.device))
    return torch.cat(rows), torch.cat(experts), torch.cat(origin)


def ep_combine_ref(expert_out: torch.Tensor, origin: torch.Tensor, num_tokens: int, topk: int, group=None,
                   topk_weight: torch.Tensor | None = None) -> torch.Tensor:
    """Inverse of dispatch: rows return to their source rank and the k copies of a token are summed (weighted by
    `topk_weight` [T, topk] of the SOURCE rank when given). Returns [T, H] fp32."""
    world, rank = _world(group), _rank(group)
    n_max = int(_all_gather_cat(torch.tensor([expert_out.shape[0]], device=expert_out.device), group).max())
    pad = torch.zeros((n_max, expert_out.shape[1]), dtype=torch.float32, device=expert_out.device)
    pad[: expert_out.shape[0]] = expert_out.float()
    opad = torch.full((n_max, 3), -1, dtype=torch.int64, device=expert_out.device)
    opad[: origin.shape[0]] = origin
    outs = _all_gather_cat(pad[None], group)
    origins = _all_gather_cat(opad[None], group)
    res = torch.zeros((num_tokens, expert_out.shape[1]), dtype=torch.float32, device=expert_out.device)
    for d in range(world):
        mine = origins[d, :, 0] == rank
        if bool(mine.any()):
            tok, k = origins[d, mine, 1], origins[d, mine, 2]
            rows = outs[d, mine]
            if topk_weight is not None:
                rows = rows * topk_weight[tok, k].float()[:, None]
            res.index_add_(0, tok, rows)
    return res
