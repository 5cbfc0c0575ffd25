"""CPU-only checks that pin the oracle: against the reference's own attn_cpu compiled from its
tester.h (oracle/_ref, present where a reference checkout was available at build time), against
golden vectors made by the reference test-suite's torch_attn, and against its own invariants."""
import glob
import os

import numpy as np
import pytest
import torch

from decoding_attention_b200 import synth
from helpers import merge_reference

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def _load(path):
    z = np.load(path)
    batch, seq_k, head_q, head_k, dim, dim_v, is_bf16 = [int(x) for x in z["meta"]]
    dt = torch.bfloat16 if is_bf16 else torch.float16
    q = torch.from_numpy(z["q"]).view(dt)
    k = torch.from_numpy(z["k"]).view(dt)
    v = torch.from_numpy(z["v"]).view(dt) if "v" in z.files else None
    cu = torch.from_numpy(z["cu_seq_k"])
    return q, k, v, cu, dim_v, torch.from_numpy(z["o_native"]).view(dt), torch.from_numpy(z["o_f32"])


def test_golden_fixtures_exist():
    assert len(GOLDEN) >= 8


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_matches_reference_torch_attn(oracle, path):
    q, k, v, cu, dim_v, o_native, o_f32 = _load(path)
    o, o32 = oracle.attn_cpu(q, k, v, cu, dim_v=dim_v, return_f32=True)
    # fp32 evaluation of the reference's torch_attn: only the summation order differs
    assert (o32 - o_f32).abs().max().item() <= 2e-5 + 1e-5 * o_f32.abs().max().item()
    # the reference's own pass criterion, against its native-dtype result
    assert (o.float() - o_native.float()).abs().mean().item() <= 5e-3


CASES = [  # dtype, batch, seq_k, head_q, head_k, dim, dim_v, alibi
    (torch.float16, 2, 128, 32, 32, 128, 128, False),
    (torch.bfloat16, 3, 77, 32, 8, 128, 128, True),
    (torch.float16, 2, 50, 16, 1, 576, 512, False),
    (torch.bfloat16, 2, 33, 32, 8, 64, 64, True),
    (torch.float16, 1, 1, 32, 8, 96, 96, False),
    (torch.bfloat16, 2, 40, 32, 1, 256, 256, True),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(x).replace("torch.", "") for x in c))
def test_oracle_bit_identical_to_reference_attn_cpu(oracle, case):
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (needs a checkout of the reference at build time)")
    dt, b, s, hq, hk, d, dv, alibi = case
    w = synth.Workload("t", dt, hq, hk, d, dv, [s] * b, is_alibi=alibi, dist="uniform", mla=(d != dv), seed=7)
    q, k, v, cu = w.make("cpu")
    o = oracle.attn_cpu(q, k, v, cu, dim_v=dv, is_alibi=alibi)
    r = oracle.ref_attn_cpu(q, k, v, s, dim_v=dv, is_alibi=alibi, threads=2)
    assert torch.equal(o.view(torch.int16), r.view(torch.int16))


def test_oracle_threads_do_not_change_bits(oracle):
    w = synth.Workload("t", torch.bfloat16, 8, 2, 128, 128, [5, 0, 130, 64], dist="normal", seed=3)
    q, k, v, cu = w.make("cpu")
    a = oracle.attn_cpu(q, k, v, cu, threads=1)
    b = oracle.attn_cpu(q, k, v, cu, threads=4)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert (a[1] == 0).all()  # zero-length sequence -> zero row


def test_oracle_varlen_equals_per_sequence(oracle):
    w = synth.Workload("t", torch.float16, 8, 4, 64, 64, [17, 1, 90], is_alibi=True, dist="normal", seed=5)
    q, k, v, cu = w.make("cpu")
    full = oracle.attn_cpu(q, k, v, cu, is_alibi=True)
    for b in range(3):
        lo, hi = w.cu[b], w.cu[b + 1]
        one = oracle.attn_cpu(q[b:b + 1].contiguous(), k[lo:hi].contiguous(), v[lo:hi].contiguous(),
                              torch.tensor([0, hi - lo], dtype=torch.int32), is_alibi=True)
        assert torch.equal(one[0].view(torch.int16), full[b].view(torch.int16))


@pytest.mark.parametrize("alibi", [False, True])
def test_oracle_key_range_shards_merge_to_whole(oracle, alibi):
    """softmax over a partition of the keys merges exactly through (o, lse) -- the identity the
    split-KV kernels and the multi-GPU key-range sharding rely on."""
    w = synth.Workload("t", torch.bfloat16, 8, 2, 128, 128, [300], is_alibi=alibi, dist="normal", scale=0.5, seed=9)
    q, k, v, cu = w.make("cpu")
    _, lse_full, o_full = oracle.attn_cpu(q, k, v, cu, is_alibi=alibi, return_lse=True, return_f32=True)
    parts_o, parts_lse = [], []
    for lo, hi in [(0, 100), (100, 260), (260, 300)]:
        cu_s = torch.tensor([0, hi - lo], dtype=torch.int32)
        _, lse, o32 = oracle.attn_cpu(q, k[lo:hi].contiguous(), v[lo:hi].contiguous(), cu_s, is_alibi=alibi,
                                      kv_pos_offset=torch.tensor([lo], dtype=torch.int32),
                                      kv_total_len=torch.tensor([300], dtype=torch.int32),
                                      return_lse=True, return_f32=True)
        parts_o.append(o32.reshape(-1, 128))
        parts_lse.append(lse.reshape(-1))
    o, lse = merge_reference(torch.stack(parts_o), torch.stack(parts_lse))
    assert (o.float() - o_full.reshape(-1, 128)).abs().max().item() < 1e-5
    assert (lse.float() - lse_full.reshape(-1)).abs().max().item() < 1e-5


def test_oracle_conversions_match_torch(oracle):
    lib = oracle._lib()
    g = torch.Generator().manual_seed(0)
    xs = torch.cat([torch.randn(2000, generator=g) * 10 ** torch.randint(-8, 5, (2000,), generator=g).float(),
                    torch.tensor([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, float("inf"), -float("inf")])])
    for x in xs.tolist():
        h = torch.tensor(x, dtype=torch.float32).to(torch.float16).view(torch.int16).item() & 0xFFFF
        b = torch.tensor(x, dtype=torch.float32).to(torch.bfloat16).view(torch.int16).item() & 0xFFFF
        assert lib.oracle_float_to_half(x) == h, x
        assert lib.oracle_float_to_bf16(x) == b, x
        assert lib.oracle_half_to_float(h) == torch.tensor(h, dtype=torch.int32).to(torch.int16).view(
            torch.float16).float().item() or x != x
