"""Reference semantics of every distributed op in plain PyTorch.

These functions run on any device and any ``torch.distributed`` backend (gloo on CPU included). They are
the oracle for the CUDA kernels and the executable statement of what each fused op means:
the same compositions the reference uses as goldens (``test/nvidia/test_ag_gemm.py:71-137``,
``test_gemm_rs.py:38-51``, ``test_all_to_all.py:184-241``, ``test_ag_moe.py:39-70``,
``test_moe_reduce_rs.py:76-152``, ``test_sp_decode_attn.py:82-133``).
"""
from .collectives import (ag_gemm_ref, all_reduce_ref, all_reduce_rmsnorm_ref, fast_allgather_ref, gemm_rs_ref)
from .moe import (ag_group_gemm_ref, grouped_gemm_ref, grouped_gemm_fp8_ref, dequant_fp8_rows, dequant_fp8_weight_blocks, all_to_all_post_process_ref, ep_combine_ref, ep_dispatch_ref, fast_all_to_all_ref,
                  fp8_dequant_ref, fp8_quant_ref, moe_align_block_size_ref, moe_reduce_rs_ref, select_experts_ref,
                  ag_moe_tile_schedule_ref, calc_gather_scatter_index_ref)
from .attention import paged_decode_attention_ref, combine_partials_ref, sp_flash_decode_ref

__all__ = [n for n in dir() if n.endswith("_ref")]
