"""The five benchmark configurations at their stated sizes, through the C ABI, against the CPU oracle
(oracle/attn_cpu.cpp, a restatement of the reference's Tester<T>::attn_cpu, csrc/common/tester.h:133-259).

These are the only tests that reach the code paths the full sizes select: the one-wave split plan of a
131 072-key sequence, the many-wave longest-first launch of 256 ragged sequences, the two-wave grid of the
latent-KV shape at batch 128, gigabyte-sized K/V tensors.  Tolerance: |out - oracle| <= 2e-3 + 1e-2 |oracle|
element-wise, mean |diff| <= 5e-3 (the reference suite's own criterion), LSE to 2e-3.

The oracle is multi-threaded over (sequence, head) rows; the largest case (latent-KV, batch 128: 146 GFLOP
of scalar fp32 work) is checked on a seeded subset of sequences, each against the oracle run on that
sequence alone -- rows of different sequences are independent, so this checks the very rows the
full-batch call wrote."""
import pytest
import torch

from decoding_attention_b200 import synth
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_full(cabi, w):
    q, k, v, cu = w.make(DEV)
    o = torch.full((w.batch, w.head_q, w.dim_v), float("nan"), dtype=w.dtype, device=DEV)
    lse = torch.empty(w.batch, w.head_q, dtype=torch.float32, device=DEV)
    args = cabi.make_args(q, k, v, o, cu, w.max_seq_k, w.dim_v, is_alibi=w.is_alibi, lse=lse,
                          stream=torch.cuda.current_stream().cuda_stream)
    before = cabi.launch_count()
    cabi.decode_fwd(args)
    torch.cuda.synchronize()
    assert cabi.launch_count() > before
    assert cabi.device_status() == cabi.DA_OK
    return o, lse, cabi.num_splits(args)


def check_sequences(oracle, w, o, lse, seqs):
    """Oracle on the sequences `seqs` (generated on the CPU from the same seed), one call per chunk."""
    for b in seqs:
        q, k, v, cu = w.make("cpu", seqs=[b])
        expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=w.is_alibi, return_lse=True)
        assert_close(o[b:b + 1], expect, f"{w.name} sequence {b}")
        assert (lse[b:b + 1].cpu() - lse_e).abs().max().item() <= 2e-3, f"{w.name} sequence {b}: LSE"


def test_config1_mha_small(native_lib, oracle):
    w = synth.config_mha_small()
    o, lse, _ = run_full(native_lib, w)
    check_sequences(oracle, w, o, lse, range(w.batch))


def test_config2_gqa_varlen_256_sequences(native_lib, oracle):
    w = synth.config_gqa_varlen()
    assert w.batch == 256 and min(w.seq_lens) >= 512 and max(w.seq_lens) <= 4096
    o, lse, _ = run_full(native_lib, w)
    q, k, v, cu = w.make("cpu")
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, return_lse=True)
    assert_close(o, expect, w.name)
    assert (lse.cpu() - lse_e).abs().max().item() <= 2e-3


def test_config3_mqa_alibi(native_lib, oracle):
    w = synth.config_mqa_alibi()
    o, lse, _ = run_full(native_lib, w)
    q, k, v, cu = w.make("cpu")
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=True, return_lse=True)
    assert_close(o, expect, w.name)
    assert (lse.cpu() - lse_e).abs().max().item() <= 2e-3


@pytest.mark.parametrize("batch", [1, 8, 32, 128])
def test_config4_mla(native_lib, oracle, batch):
    w = synth.config_mla(batch=batch)
    o, lse, _ = run_full(native_lib, w)
    assert torch.isfinite(o.float()).all()
    if batch <= 8:
        seqs = list(range(batch))
    else:  # a seeded subset that always holds the first and the last sequence (first and last wave of the grid)
        g = torch.Generator().manual_seed(4 + batch)
        seqs = sorted(set([0, batch - 1] + torch.randperm(batch, generator=g)[:14].tolist()))
    check_sequences(oracle, w, o, lse, seqs)
    # every sequence has the same length and statistics: rows nobody checked must at least look like the checked ones
    ref_scale = o[seqs].float().abs().mean().item()
    assert abs(o.float().abs().mean().item() - ref_scale) <= 0.1 * ref_scale


def test_config5_long_mha_131072_keys(native_lib, oracle):
    w = synth.config_long_mha()
    o, lse, splits = run_full(native_lib, w)
    assert splits > 1, "one sequence on a whole GPU must be split over key ranges"
    check_sequences(oracle, w, o, lse, [0])


def test_sequences_longer_than_max_seq_k_are_still_read_completely(native_lib, oracle):
    """max_seq_k sizes the split plan; a sequence that turns out longer is finished by its last split."""
    w = synth.Workload("long_hint", torch.bfloat16, 32, 8, 128, 128, [3000, 700, 1800], dist="normal", scale=0.5, seed=51)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu)
    dq, dk, dv, dcu = q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV)
    for hint, splits in ((1024, 0), (1024, 1), (1024, 3), (64, 0)):
        o = torch.full((3, 32, 128), float("nan"), dtype=w.dtype, device=DEV)
        native_lib.decode_fwd(native_lib.make_args(dq, dk, dv, o, dcu, hint, 128, num_splits=splits))
        torch.cuda.synchronize()
        assert_close(o, expect, f"max_seq_k {hint}, splits {splits}")
    wm = synth.Workload("long_hint_mla", torch.bfloat16, 128, 1, 576, 512, [900, 300], dist="normal", scale=0.3, mla=True, seed=52)
    q, k, v, cu = wm.make("cpu")
    expect = oracle.attn_cpu(q, k, None, cu, dim_v=512)
    o = torch.full((2, 128, 512), float("nan"), dtype=wm.dtype, device=DEV)
    native_lib.decode_fwd(native_lib.make_args(q.to(DEV), k.to(DEV), None, o, cu.to(DEV), 256, 512, num_splits=2))
    torch.cuda.synchronize()
    assert_close(o, expect, "latent-KV, max_seq_k 256")
