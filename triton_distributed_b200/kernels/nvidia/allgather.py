"""Copy-engine all-gather producers.

API parity with ``python/triton_dist/kernels/nvidia/allgather.py`` (``AllGatherMethod`` :46-53,
``get_auto_all_gather_method`` :57-71, ``cp_engine_producer_all_gather_intra_node`` :263-290). The fused AG-GEMM of
this library pulls with SM warps inside the GEMM kernel; these producers remain for callers that want the
reference's structure (a side stream of peer-to-peer memcpys that raise one flag per source rank).
"""
from __future__ import annotations

import enum

import torch


class AllGatherMethod(enum.Enum):
    Auto = 0
    All2All_IntraNode = 1     # full-mesh pull
    Ring1D_IntraNode = 2
    Ring2D_IntraNode = 3
    All2All_InterNode = 4
    Ring2D_InterNode = 5
    Ring3D_InterNode = 6


def get_auto_all_gather_method(num_ranks: int, num_local_ranks: int) -> AllGatherMethod:
    """Behind an NVSwitch every peer is one hop away: the full-mesh pull is always the choice on one node."""
    if num_ranks != num_local_ranks:
        raise NotImplementedError("single node only")
    return AllGatherMethod.All2All_IntraNode


def cp_engine_producer_all_gather_intra_node(rank: int, num_ranks: int, local_tensor: torch.Tensor,
                                             remote_tensor_buffers: list[torch.Tensor], barrier_buffers: list[torch.Tensor],
                                             stream: torch.cuda.Stream, for_correctness: bool = False,
                                             all_gather_method: AllGatherMethod = AllGatherMethod.Auto, signal_value: int = 1):
    """Pull every peer's shard into the local gather buffer with copy-engine memcpys on `stream`, raising
    ``barrier_buffers[rank][src] = signal_value`` after each. ``remote_tensor_buffers[k]`` is rank k's gather buffer
    ``[num_ranks * M_per_rank, K]`` (peer views of one symmetric allocation); slot `rank` of every buffer is expected
    to hold that rank's shard already."""
    m = local_tensor.shape[0]
    with torch.cuda.stream(stream):
        for k in range(1, num_ranks):
            src = (rank + k) % num_ranks
            if for_correctness:
                torch.cuda._sleep(100_000)
            remote_tensor_buffers[rank][src * m:(src + 1) * m].copy_(remote_tensor_buffers[src][src * m:(src + 1) * m])
            barrier_buffers[rank][src:src + 1].fill_(signal_value)


def cp_engine_producer_all_gather_inter_node(*args, **kwargs):
    raise NotImplementedError("inter-node all-gather is out of scope: this library spans one NVSwitch node")
