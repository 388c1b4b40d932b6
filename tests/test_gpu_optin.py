"""Runs the existing kernel tests once more with each opt-in variant switched on (the variants are chosen by
environment variables that the native library reads once per process, hence one pytest subprocess per setting).

Off unless B200DIST_TEST_UNVERIFIED=1: these variants are built and desk-checked but have not been run on a GPU yet,
so they are kept out of the default test run until they have been.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))

VARIANTS = [
    ({"B200DIST_ATTN_V2": "3"}, ["tests/test_gpu_ops.py", "-k", "decode_attention"]),
    ({"B200DIST_ATTN_V2": "6"}, ["tests/test_gpu_ops.py", "-k", "decode_attention"]),
    ({"B200DIST_ATTN_FUSED_COMBINE": "1"}, ["tests/test_gpu_ops.py", "-k", "decode_attention"]),
    ({"B200DIST_ATTN_V2": "6", "B200DIST_ATTN_FUSED_COMBINE": "1"}, ["tests/test_gpu_ops.py", "tests/test_gpu_model.py", "-k", "decode or engine or model"]),
    ({"B200DIST_MOE_SORT_SMALL": "1"}, ["tests/test_gpu_moe.py"]),
    ({"B200DIST_AG_GROUP_PUSH": "1"}, ["tests/test_gpu_moe.py", "-k", "ag_group_gemm"]),
    ({"B200DIST_PREFILL_NATIVE": "1"}, ["tests/test_gpu_model.py"]),
    ({"B200DIST_AR_LL": "1"}, ["tests/test_gpu_dist_world1.py", "tests/test_gpu_model.py", "-k", "allreduce or model or engine"]),
]


@pytest.mark.skipif(os.environ.get("B200DIST_TEST_UNVERIFIED", "0") != "1", reason="opt-in variants: set B200DIST_TEST_UNVERIFIED=1")
@pytest.mark.parametrize("env_extra,pytest_args", VARIANTS, ids=[",".join(f"{k}={v}" for k, v in e.items()) for e, _ in VARIANTS])
def test_existing_tests_pass_with_variant(env_extra, pytest_args):
    env = dict(os.environ)
    env.update(env_extra)
    env.pop("B200DIST_TEST_UNVERIFIED", None)  # the child must not recurse into this file's cases
    res = subprocess.run([sys.executable, "-m", "pytest", "-q", "-m", "gpu", "-p", "no:cacheprovider", *pytest_args],
                         cwd=os.path.dirname(HERE), env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(res.stdout[-4000:])
    sys.stderr.write(res.stderr[-2000:])
    assert res.returncode == 0, f"tests failed with {env_extra}"


@pytest.mark.skipif(os.environ.get("B200DIST_TEST_UNVERIFIED", "0") != "1", reason="opt-in variants: set B200DIST_TEST_UNVERIFIED=1")
@pytest.mark.parametrize("lens_q,lens_k,Hq,Hkv,causal", [
    ([128], [128], 2, 1, True), ([300, 77], [300, 77], 8, 2, True), ([64, 200], [256, 333], 4, 4, True),
    ([130], [513], 4, 1, False), ([1024, 1], [1024, 700], 8, 8, True)])
def test_prefill_attention_matches_reference(lens_q, lens_k, Hq, Hkv, causal):
    """The tcgen05 prefill attention against an fp32 masked softmax, packed variable-length sequences, GQA, and the
    bottom-right alignment of the causal mask when a sequence has more keys than queries."""
    import math

    import torch

    from triton_distributed_b200 import ops
    torch.manual_seed(5)
    D = 128
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(lens_q), Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(sum(lens_k), Hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(sum(lens_k), Hkv, D, device="cuda", dtype=torch.bfloat16)
    scale = 1 / math.sqrt(D)
    out = ops.prefill_attention(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), scale, causal)
    torch.cuda.synchronize()
    G = Hq // Hkv
    for b, (lq, lk) in enumerate(zip(lens_q, lens_k)):
        qs, ks = int(cu_q[b]), int(cu_k[b])
        qq = q[qs:qs + lq].float()
        kk = k[ks:ks + lk].float().repeat_interleave(G, dim=1)
        vv = v[ks:ks + lk].float().repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        if causal:
            qi = torch.arange(lq, device="cuda")[:, None] + (lk - lq)
            ki = torch.arange(lk, device="cuda")[None, :]
            s = s.masked_fill(ki > qi, float("-inf"))
        want = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1).nan_to_num(0.0), vv)
        torch.testing.assert_close(out[qs:qs + lq].float(), want, rtol=3e-2, atol=3e-2)
