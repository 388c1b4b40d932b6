"""Host-side logic that needs no GPU: index/sort metadata references, weights I/O, sampling, helpers."""
import json

import pytest
import torch


def test_gather_scatter_index_is_a_stable_sort_with_padding():
    from triton_distributed_b200 import ref
    torch.manual_seed(0)
    T, topk, E, align = 37, 3, 8, 16
    ids = torch.stack([torch.randperm(E)[:topk] for _ in range(T)]).to(torch.int32)
    counts, scatter, gather, expert_index, m_pad = ref.calc_gather_scatter_index_ref(ids, E, align)
    assert int(counts.sum()) == T * topk and m_pad % align == 0 and gather.numel() == m_pad
    flat = ids.reshape(-1)
    valid = gather < T * topk
    assert int(valid.sum()) == T * topk
    # every tile holds one expert; rows of an expert keep their original order
    for tile in range(m_pad // align):
        rows = gather[tile * align:(tile + 1) * align]
        rows = rows[rows < T * topk].long()
        assert torch.all(flat[rows] == expert_index[tile])
        assert torch.all(rows[1:] > rows[:-1])
    # scatter is the inverse of gather
    assert torch.equal(gather[scatter.reshape(-1).long()].long(), torch.arange(T * topk))


def test_moe_align_per_rank_blocks():
    from triton_distributed_b200 import ref
    torch.manual_seed(1)
    T, topk, E, bm, ranks = 64, 2, 4, 8, 4
    ids = torch.randint(0, E, (T, topk), dtype=torch.int32)
    sorted_ids, expert_ids, barrier_ids, rank_blocks, npad = ref.moe_align_block_size_ref(ids, E, bm, ranks)
    assert npad == sorted_ids.numel() == expert_ids.numel() * bm and int(rank_blocks.sum()) == expert_ids.numel()
    per = T // ranks * topk
    for tile in range(expert_ids.numel()):
        rows = sorted_ids[tile * bm:(tile + 1) * bm]
        rows = rows[rows < T * topk].long()
        assert torch.all(ids.reshape(-1)[rows] == expert_ids[tile])
        assert torch.all(rows // per == barrier_ids[tile])
    assert sorted(sorted_ids[sorted_ids < T * topk].tolist()) == list(range(T * topk))


def test_ag_moe_schedule_orders_tiles_by_arrival_stage():
    from triton_distributed_b200 import ref
    torch.manual_seed(2)
    T, topk, E, bm, world = 128, 2, 4, 16, 4
    ids = torch.randint(0, E, (T, topk), dtype=torch.int32)
    for rank in range(world):
        gather, tile_expert, s0, s1, order = ref.ag_moe_tile_schedule_ref(ids, E, bm, rank, world)
        stage = (s1.long() - rank) % world
        stage = torch.where((s0.long() - rank) % world > stage, torch.full_like(stage, world - 1), stage)
        assert torch.all(stage[order.long()][1:] >= stage[order.long()][:-1])
        assert sorted(order.tolist()) == list(range(tile_expert.numel()))
        per = T // world
        for tile in range(tile_expert.numel()):
            rows = gather[tile * bm:(tile + 1) * bm]
            rows = rows[rows < T * topk].long()
            src = (rows // topk) // per
            assert int(src.min()) == int(s0[tile]) and int(src.max()) == int(s1[tile])


def test_fp8_block_quant_roundtrip():
    from triton_distributed_b200 import ref
    torch.manual_seed(3)
    x = torch.randn(16, 512) * 3
    q, s = ref.fp8_quant_ref(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (16, 4)
    back = ref.fp8_dequant_ref(q, s, dtype=torch.float32)
    assert (back - x).abs().max() <= x.abs().max() * 0.07
    # quantisation of an already representable tensor is exact
    q2, s2 = ref.fp8_quant_ref(back)
    torch.testing.assert_close(ref.fp8_dequant_ref(q2, s2, dtype=torch.float32), back, rtol=1e-5, atol=1e-5)


def test_combine_partials_skips_empty_and_matches_full_softmax():
    from triton_distributed_b200 import ref
    torch.manual_seed(4)
    s = torch.randn(5, 3, 40)
    v = torch.randn(5, 40, 8)
    full = torch.softmax(s.reshape(5, 120)[:, :], -1)  # three parts of 40 keys each -> one softmax over 120
    vv = torch.cat([v, v * 2, v * 3], 1)
    want = torch.einsum("bl,bld->bd", full, vv)
    parts_o, parts_l = [], []
    for r, scale in enumerate((1, 2, 3)):
        sr = s[:, r]
        parts_l.append(torch.logsumexp(sr, -1))
        parts_o.append(torch.einsum("bl,bld->bd", torch.softmax(sr, -1), v * scale))
    parts_o.append(torch.zeros(5, 8))
    parts_l.append(torch.full((5,), float("-inf")))
    out, lse = ref.combine_partials_ref(torch.stack(parts_o), torch.stack(parts_l))
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(lse, torch.logsumexp(s.reshape(5, 120), -1), rtol=1e-5, atol=1e-5)


def test_checkpoint_writer_and_sliced_reader(tmp_path):
    from triton_distributed_b200.models import ARCHS
    from triton_distributed_b200.models.weights import (RandomSource, SafetensorsSource, hf_param_shapes,
                                                       read_arch_from_checkpoint, write_random_checkpoint)
    arch = ARCHS["tiny-qwen3"]
    write_random_checkpoint(str(tmp_path), arch, torch.bfloat16, seed=5, max_shard_bytes=2 << 20)
    idx = json.load(open(tmp_path / "model.safetensors.index.json"))
    assert set(idx["weight_map"]) == set(hf_param_shapes(arch))
    assert read_arch_from_checkpoint(str(tmp_path)) == arch
    src = SafetensorsSource(str(tmp_path), device="cpu")
    rnd = RandomSource(arch, torch.bfloat16, seed=5, device="cpu", consistent=True)
    name = "model.layers.1.mlp.down_proj.weight"
    assert torch.equal(src.get(name, cols=slice(128, 256)), rnd.get(name, cols=slice(128, 256)))
    assert torch.equal(src.get("model.layers.0.self_attn.q_proj.weight", rows=slice(0, 128)),
                       rnd.get("model.layers.0.self_attn.q_proj.weight", rows=slice(0, 128)))
    assert torch.all(src.get("model.norm.weight") == 1)
    # per-slice random source: right shapes, deterministic
    fast = RandomSource(arch, torch.bfloat16, seed=5, device="cpu", consistent=False)
    a = fast.get(name, cols=slice(0, 64))
    assert a.shape == (arch.hidden_size, 64) and torch.equal(a, fast.get(name, cols=slice(0, 64)))


def test_sample_token_cpu_paths():
    from triton_distributed_b200.models import sample_token
    logits = torch.full((2, 1, 50), -20.0)
    logits[0, 0, 7] = 5.0
    logits[1, 0, 33] = 5.0
    assert sample_token(logits, temperature=0.0).flatten().tolist() == [7, 33]
    torch.manual_seed(0)
    assert sample_token(logits, temperature=0.6, top_p=0.9).flatten().tolist() == [7, 33]


def test_allreduce_method_names_and_auto_choice():
    from triton_distributed_b200.kernels.allreduce import AllReduceMethod, get_allreduce_methods, to_allreduce_method
    from triton_distributed_b200.kernels.nvidia.allreduce import get_auto_allreduce_method
    assert set(get_allreduce_methods()) >= {"double_tree", "one_shot", "two_shot", "one_shot_multimem", "two_shot_multimem"}
    assert to_allreduce_method("two_shot_multimem") is AllReduceMethod.TwoShot_Multimem
    with pytest.raises(ValueError):
        to_allreduce_method("ring")
    assert get_auto_allreduce_method(8 << 10, has_multicast=True, world=8) is AllReduceMethod.OneShot
    assert get_auto_allreduce_method(8 << 20, has_multicast=True, world=8) is AllReduceMethod.TwoShot_Multimem
    assert get_auto_allreduce_method(8 << 20, has_multicast=True, world=2) is AllReduceMethod.OneShot   # same bytes as two-shot
    assert get_auto_allreduce_method(2 << 20, has_multicast=True, world=4) is AllReduceMethod.OneShot
    assert get_auto_allreduce_method(8 << 20, has_multicast=True, world=4) is AllReduceMethod.TwoShot_Multimem
    assert get_auto_allreduce_method(32 << 20, has_multicast=True, world=2) is AllReduceMethod.TwoShot
    assert get_auto_allreduce_method(8 << 10, has_multicast=False, world=8) is AllReduceMethod.OneShot
    assert get_auto_allreduce_method(8 << 20, has_multicast=False, world=8) is AllReduceMethod.TwoShot


def test_trace_merge_and_helpers(capsys):
    from triton_distributed_b200 import utils
    a = {"traceEvents": [{"ph": "X", "pid": 1, "tid": 2, "name": "k"}, {"ph": "M", "pid": 1, "args": {"name": "proc"}}], "meta": 1}
    b = {"traceEvents": [{"ph": "X", "pid": 1, "tid": 2, "name": "k"}]}
    m = utils.merge_traces([a, b])
    assert len(m["traceEvents"]) == 3 and m["meta"] == 1
    assert m["traceEvents"][2]["pid"] == 1 + 100_000_000 and m["traceEvents"][1]["args"]["name"] == "proc_rank0"
    utils.assert_allclose(torch.ones(4), torch.ones(4), 1e-3, 1e-3, verbose=False)
    with pytest.raises(RuntimeError, match="mismatches"):
        utils.assert_allclose(torch.ones(4), torch.zeros(4), 1e-3, 1e-3)
    utils.dist_print("hello", allowed_ranks="all", prefix=True)
    assert "hello" in capsys.readouterr().out


def test_native_library_builds_and_reports_errors():
    """The shared object loads without a driver; entry points that need one fail with a message, not a crash."""
    import ctypes
    from triton_distributed_b200 import _lib
    lib = _lib.load()
    assert lib.b200_symm_ctx_size() >= 96
    lib.b200_gemm_skinny_scratch_floats.restype = ctypes.c_longlong
    assert lib.b200_gemm_skinny_scratch_floats(8, 1280, 0) == 10 * 16 * 128
    assert lib.b200_allreduce_ws_factor(0, 8, 0) == 8 and lib.b200_allreduce_ws_factor(3, 8, 1) == 3
    if not torch.cuda.is_available():
        h = ctypes.c_void_p()
        rc = lib.b200_heap_create(0, 0, 1, ctypes.c_uint64(1 << 20), 0, ctypes.byref(h))
        assert rc != 0 and lib.b200_last_error()
        from triton_distributed_b200 import ops
        with pytest.raises(RuntimeError, match="CUDA"):
            ops.gemm(torch.zeros(2, 8), torch.zeros(2, 8))


def test_fp8_block_quantisers_round_trip_and_reference():
    """1x128 activation scales and 128x128 weight scales: amax / 448 without epsilon, zero blocks stay zero, and the
    dequantised grouped product stays within fp8's precision of the exact one."""
    import torch
    from triton_distributed_b200 import ref
    from triton_distributed_b200.kernels.nvidia.grouped_gemm_fp8 import quantize_fp8_rows, quantize_fp8_weight_blocks
    torch.manual_seed(0)
    a = torch.randn(12, 256)
    a[3] = 0
    w = torch.randn(3, 200, 256) * 0.05
    a8, sa = quantize_fp8_rows(a)
    w8, sw = quantize_fp8_weight_blocks(w)
    assert a8.dtype == torch.float8_e4m3fn and sa.shape == (12, 2) and sw.shape == (3, 2, 2)
    assert torch.all(sa[3] == 0) and torch.all(ref.dequant_fp8_rows(a8, sa)[3] == 0)
    torch.testing.assert_close(sa[0, 0], a[0, :128].abs().max() / 448.0)
    assert (ref.dequant_fp8_rows(a8, sa) - a).abs().max() <= a.abs().max() * 0.07
    e = torch.randint(0, 3, (12,))
    got = ref.grouped_gemm_fp8_ref(a8, sa, w8, sw, e)
    exact = ref.grouped_gemm_ref(a, w, e)
    assert (got - exact).norm() / exact.norm() < 0.06


def test_scatter_gather_index_helpers_and_public_names():
    """The torch index helpers invert each other, and the package exports every name of the reference's
    kernels.nvidia surface that has a counterpart here."""
    import torch
    from triton_distributed_b200.kernels import nvidia as K
    ids = torch.tensor([[1, 0], [0, 2], [2, 1], [1, 1]], dtype=torch.int32)
    scatter = K.calc_scatter_index_torch(ids, 3)
    assert sorted(scatter.reshape(-1).tolist()) == list(range(8))
    experts_sorted = torch.empty(8, dtype=torch.int32)
    experts_sorted[scatter.reshape(-1).long()] = ids.reshape(-1)
    assert torch.equal(experts_sorted, torch.sort(ids.reshape(-1), stable=True).values)
    gather = K.calc_gather_index_from_scatter_index(scatter)
    assert torch.equal(gather[scatter.reshape(-1).long()], torch.arange(8, dtype=torch.int32))
    assert torch.equal(K.histogram_by_expert_torch(ids, 3), torch.tensor([2, 4, 2], dtype=torch.int32))
    for name in ["create_ag_gemm_context", "ag_gemm", "gemm_persistent", "create_gemm_rs_context", "gemm_rs", "AllGatherMethod",
                 "get_auto_all_gather_method", "create_ag_group_gemm_context", "ag_group_gemm", "select_experts",
                 "create_moe_rs_context", "moe_reduce_rs_rowise", "moe_reduce_rs_colwise", "create_all_to_all_context",
                 "fast_all_to_all", "all_to_all_post_process", "create_fast_allgather_context", "fast_allgather",
                 "gqa_fwd_batch_decode", "gqa_fwd_batch_decode_intra_rank", "gqa_fwd_batch_decode_persistent",
                 "fused_sp_ag_attn_intra_node", "fused_sp_ag_attn_inter_node", "create_allreduce_ctx", "all_reduce",
                 "get_auto_allreduce_method", "BarrierAllContext", "wait_eq", "set_signal", "create_reduce_scater_2d_ctx",
                 "reduce_scatter_2d_op", "ring_reduce", "calc_gather_scatter_index_triton", "reduce_topk_tma",
                 "estimate_gemm_sol_time_ms", "get_tensorcore_tflops", "estimate_all_gather_time_ms", "grouped_gemm_fp8",
                 "create_ag_group_gemm_fp8_context", "ag_group_gemm_fp8", "moe_reduce_rs_fp8", "moe_reduce_rs",
                 "quantize_fp8_rows", "quantize_fp8_weight_blocks"]:
        assert hasattr(K, name), name


def test_ag_gemm_gather_choice_follows_world_size_and_bytes():
    """`auto` pushes only when at least four ranks take part and at most 64 MB leave a rank."""
    import torch
    from triton_distributed_b200.kernels.nvidia.allgather_gemm import AllGatherGEMMTensorParallelContext as Ctx

    def ctx(world, K=8192):
        return Ctx(rank=0, num_ranks=world, num_local_ranks=world, max_M=8192, N_per_rank=1024, K=K, dtype=torch.bfloat16,
                   heap=None, symm_workspaces=[], symm_ready=None, blk_cnt=None, blk_flag=None, sync=None)
    assert ctx(2).method_for(64) == "sm_push_fused"      # one peer: pushed rows arrive as one stream
    assert ctx(8).method_for(128) == "sm_push_fused"      # M = 1024: 14.7 MB out
    assert ctx(8).method_for(512) == "sm_push_fused"      # M = 4096: 58.7 MB out
    assert ctx(8).method_for(1024) == "sm_pull_fused"     # M = 8192: 117 MB out
    c = ctx(8)
    c.all_gather_method = "sm_pull_fused"
    assert c.method_for(128) == "sm_pull_fused"


def test_bench_reference_arm_reports_unavailable_and_exits_zero():
    """`bench.py --impl reference` must answer with one JSON line and exit 0 even where the reference cannot run."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                           "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-500:]
    line = [l for l in proc.stdout.splitlines() if l.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]


def test_allreduce_method_resolution_and_split_heuristics():
    """Host-side choices that need no GPU: which native all-reduce a reference method name maps to (with and without
    an NVLS mapping), the workspace factors, and the KV split heuristic's bounds."""
    import types

    import pytest

    from triton_distributed_b200 import ops
    from triton_distributed_b200.kernels.allreduce import AllReduceMethod, get_allreduce_methods, to_allreduce_method
    from triton_distributed_b200.kernels.nvidia import allreduce as ar

    def ctx(mc):
        return types.SimpleNamespace(heap=types.SimpleNamespace(has_multicast=mc), world_size=8, max_ctas=128)

    assert ar._resolve(AllReduceMethod.OneShot, 1 << 10, ctx(False)) == 0
    assert ar._resolve(AllReduceMethod.OneShot_TMA, 1 << 10, ctx(False)) == 0
    assert ar._resolve(AllReduceMethod.TwoShot, 1 << 24, ctx(False)) == 1
    assert ar._resolve(AllReduceMethod.DoubleTree, 1 << 10, ctx(False)) == 0      # small: one-shot
    assert ar._resolve(AllReduceMethod.DoubleTree, 1 << 24, ctx(False)) == 1      # large: two-shot
    assert ar._resolve(None, 1 << 10, ctx(True)) == 0 and ar._resolve(None, 1 << 24, ctx(True)) == 3      # one-shot push, NVLS two-shot
    assert ar._resolve(None, 1 << 20, ctx(True)) == 0 and ar._resolve(None, (1 << 20) + 16, ctx(True)) == 3
    assert ar._resolve(None, 1 << 10, ctx(False)) == 0 and ar._resolve(None, 1 << 24, ctx(False)) == 1
    with pytest.raises(RuntimeError):
        ar._resolve(AllReduceMethod.TwoShot_Multimem, 1 << 20, ctx(False))
    assert ar._ws_factor(0, 8, False) == 8 and ar._ws_factor(2, 8, False) == 1
    assert ar._ws_factor(1, 8, False) == 2 and ar._ws_factor(1, 8, True) == 3
    assert all(to_allreduce_method(n).name.lower().replace("_", "") == n.replace("_", "") for n in get_allreduce_methods())
    with pytest.raises(ValueError):
        to_allreduce_method("ring")
    for batch, hkv, group, kv in [(1, 1, 8, 128), (8, 8, 8, 2048), (8, 1, 8, 2048), (32, 8, 8, 1 << 20), (1, 8, 8, 1 << 20)]:
        s = ops.choose_kv_splits(batch, hkv, group, kv)
        assert 1 <= s <= 64 and (s == 1 or kv // s >= 128)


def test_bench_withholds_its_result_when_a_wait_expired(capsys):
    """A kernel whose bounded wait ran out returns early with incomplete data and leaves the status word set.
    bench.py must then fail instead of printing a tokens/s line; with a clean status it prints exactly one line."""
    import importlib.util
    import json
    import os

    import pytest

    from triton_distributed_b200.runtime.heap import SymmHeap, SymmTimeoutError
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class FakeHeap:
        rank = 0
        check_status = SymmHeap.check_status

        def __init__(self, code):
            self.code, self.cleared = code, False
            self._lib = self
            self._h = None

        def status(self):
            return [self.code, 3, 7, 6, 123] + [0] * 11

        def b200_heap_status_clear(self, _h):
            self.cleared = True

    with pytest.raises(SymmTimeoutError, match="who=3"):
        bench.emit_result({"value": 1.0}, FakeHeap(1), 0)
    assert capsys.readouterr().out == ""
    bench.emit_result({"value": 1.0}, FakeHeap(0), 0)
    assert json.loads(capsys.readouterr().out) == {"value": 1.0}
    bench.emit_result({"value": 1.0}, FakeHeap(0), 1)   # only rank 0 prints
    assert capsys.readouterr().out == ""


def test_gemm_rs_in_switch_reduction_is_opt_in():
    from types import SimpleNamespace

    from triton_distributed_b200.kernels.nvidia.gemm_reduce_scatter import GEMMReduceScatterTensorParallelContext

    def ctx(world, multicast, nvls=None):
        return GEMMReduceScatterTensorParallelContext(
            rank=0, world_size=world, local_world_size=world, max_M=16384, N=8192, output_dtype=None,
            heap=SimpleNamespace(has_multicast=multicast), slots=[], rs_cnt=None, rs_base=None, sync=None, rs_blocks=4, nvls=nvls)

    assert not ctx(2, True).use_nvls(8192) and not ctx(8, True).use_nvls(8192)   # default: per-source slots
    assert ctx(8, True, nvls=True).use_nvls(128) and not ctx(2, True, nvls=False).use_nvls(8192)
    assert not ctx(8, False, nvls=True).use_nvls(128)                            # no multicast mapping, no in-switch sum


def test_ag_moe_tile_reordering_only_when_it_pays():
    """Arrival-ordered tiles re-stream every expert's weights once per arrival stage; the wrapper reorders only when
    those bytes cost clearly less HBM time than the gather takes on the links."""
    from types import SimpleNamespace

    from triton_distributed_b200.kernels.nvidia.allgather_group_gemm import _reorder_pays

    ctx8 = SimpleNamespace(num_ranks=8, topk=8)
    assert not _reorder_pays(SimpleNamespace(num_ranks=1, topk=8), 8192, 128, 384, 4096, 2)   # one rank: nothing to overlap
    assert not _reorder_pays(ctx8, 8192, 128, 384, 4096, 2)     # 403 MB of weights x 3 extra passes >> 58 MB gather
    assert _reorder_pays(ctx8, 65536, 8, 128, 8192, 2)          # few small experts, many tokens: the gather dominates
