"""NVIDIA kernel library (exports follow ``python/triton_dist/kernels/nvidia/__init__.py:25-85``)."""
from .allgather_gemm import ag_gemm, create_ag_gemm_context, gemm_non_persistent, gemm_persistent
from .allreduce import all_reduce, all_reduce_rmsnorm, create_allreduce_ctx, get_auto_allreduce_method
from .common_ops import BarrierAllContext, barrier_all_on_stream, set_signal, wait_eq
from .flash_decode import (get_triton_combine_kv_algo_info, gqa_fwd_batch_decode, gqa_fwd_batch_decode_aot,
                           gqa_fwd_batch_decode_intra_rank, gqa_fwd_batch_decode_intra_rank_aot,
                           gqa_fwd_batch_decode_persistent, gqa_fwd_batch_decode_persistent_aot,
                           kernel_gqa_fwd_batch_decode_split_kv_persistent,
                           kernel_inter_rank_gqa_fwd_batch_decode_combine_kv)
from .gemm_reduce_scatter import create_gemm_rs_context, gemm_rs
from .low_latency_allgather import create_fast_allgather_context, fast_allgather
from .allgather_group_gemm import (ag_group_gemm, ag_group_gemm_fp8, create_ag_group_gemm_context,
                                   create_ag_group_gemm_fp8_context, grouped_gemm)
from .grouped_gemm_fp8 import (grouped_gemm_fp8, grouped_gemm_fp8_planned, quantize_fp8_rows,
                               quantize_fp8_weight_blocks)
from .moe_reduce_rs import (create_moe_rs_context, create_moe_rs_context_colwise, moe_reduce_rs, moe_reduce_rs_colwise,
                            moe_reduce_rs_fp8, moe_reduce_rs_rowise, select_experts)
from .moe_utils import (calc_gather_index_from_scatter_index, calc_gather_scatter_index, calc_gather_scatter_index_triton,
                        calc_scatter_index_torch, create_sort_plan, histogram_by_expert, histogram_by_expert_torch,
                        histogram_by_expert_triton, moe_sort, order_tiles, reduce_topk, reduce_topk_non_tma, reduce_topk_tma)
from .gemm_perf_model import estimate_gemm_sol_time_ms, get_dram_gbps, get_tensorcore_tflops
from .comm_perf_model import (estimate_all_gather_time_ms, estimate_reduce_scatter_time_ms, fused_roofline_ms,
                              get_nic_gbps_per_gpu)
from .low_latency_all_to_all import all_to_all_post_process, create_all_to_all_context, fast_all_to_all
from .allgather import (AllGatherMethod, cp_engine_producer_all_gather_inter_node, cp_engine_producer_all_gather_intra_node,
                        get_auto_all_gather_method)
from .reduce_scatter import create_reduce_scater_2d_ctx, reduce_scatter_2d_op, ring_reduce
from .sp_ag_attention_intra_node import (create_sp_ag_attention_context_inter_node, create_sp_ag_attention_context_intra_node,
                                         fused_sp_ag_attn_inter_node, fused_sp_ag_attn_intra_node)
