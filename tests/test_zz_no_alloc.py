"""The allocation-free entry point, da_decode_fwd_static.

Some hosts of this library cannot allocate device memory when they call it: an inference engine
that has given the whole GPU to its own cache pool, or code that runs where the CUDA allocator must
not be entered.  For them the split partials live in a fixed array inside the library.  This test
calls that entry point through the C ABI twice in a row -- the second call on a different, smaller
problem, so that it runs over whatever the first one left in the array -- and requires each result
to match the ordinary entry point's within the parity tolerance of the other GPU tests (in fact bit
for bit: both run the same kernels on the same split plan) and the CPU oracle's.  After the first
call on the device, further calls must leave the amount of free device memory unchanged.  It sits
in a file that pytest collects last, so a run that stops at the first failure has already run
everything else.
"""
import pytest
import torch

from decoding_attention_b200 import synth
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _both(cabi, w, num_splits):
    q, k, v, cu = [t.to(DEV) if t is not None else None for t in w.make("cpu")]
    outs = []
    for fn in (cabi.decode_fwd, cabi.decode_fwd_static):
        o = torch.full((w.batch, w.head_q, w.dim_v), float("nan"), dtype=w.dtype, device=DEV)
        args = cabi.make_args(q, k, v, o, cu, w.max_seq_k, w.dim_v, is_alibi=w.is_alibi, num_splits=num_splits,
                              stream=torch.cuda.current_stream().cuda_stream)
        assert cabi.workspace_bytes(args) > 0, "the case must need split scratch"
        fn(args)
        torch.cuda.synchronize()
        outs.append(o)
    assert cabi.device_status() == cabi.DA_OK
    return outs


def test_static_scratch_matches_ordinary_entry_point_twice(native_lib, oracle):
    first = synth.Workload("noalloc_a", torch.bfloat16, 32, 8, 128, 128, [3000, 517, 64, 1900], dist="normal",
                           scale=0.5, seed=31)
    second = synth.Workload("noalloc_b", torch.float16, 16, 16, 64, 64, [700, 0, 129], is_alibi=True, dist="uniform",
                            seed=32)
    for w, splits in ((first, 6), (second, 3)):
        ref, got = _both(native_lib, w, splits)
        assert_close(got, ref, w.name)
        assert torch.equal(got, ref), "same kernels, same split plan: the two entry points must agree bit for bit"
        assert_close(got, oracle.attn_cpu(*w.make("cpu"), dim_v=w.dim_v, is_alibi=w.is_alibi), w.name + " vs oracle")


def test_static_scratch_calls_allocate_nothing(native_lib):
    """Once the first call on the device has resolved the array, a call must not change the free device memory."""
    w = synth.Workload("noalloc_mem", torch.bfloat16, 32, 8, 128, 128, [2500, 900], dist="normal", scale=0.5, seed=34)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    o = torch.empty(w.batch, w.head_q, w.dim_v, dtype=w.dtype, device=DEV)
    args = native_lib.make_args(q, k, v, o, cu, w.max_seq_k, w.dim_v, num_splits=5,
                                stream=torch.cuda.current_stream().cuda_stream)
    native_lib.decode_fwd_static(args)  # the warm-up call an allocation-free host makes at start-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        native_lib.decode_fwd_static(args)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes"


def test_static_scratch_rejects_oversized_and_foreign_workspace(native_lib):
    cap = native_lib.lib().da_static_scratch_bytes()
    assert 0 < cap <= 64 << 20
    w = synth.Workload("noalloc_big", torch.float16, 64, 64, 64, 64, [8] * 512, dist="normal", seed=33)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    o = torch.empty(w.batch, w.head_q, w.dim_v, dtype=w.dtype, device=DEV)
    args = native_lib.make_args(q, k, v, o, cu, 4096, w.dim_v, num_splits=16)  # max_seq_k hint drives the split plan
    assert native_lib.workspace_bytes(args) > cap
    with pytest.raises(native_lib.DecodingAttnError) as e:
        native_lib.decode_fwd_static(args)
    assert e.value.status == native_lib.DA_ERR_WORKSPACE
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=DEV)
    args = native_lib.make_args(q, k, v, o, cu, 8, w.dim_v, workspace=ws)
    with pytest.raises(native_lib.DecodingAttnError) as e:
        native_lib.decode_fwd_static(args)
    assert e.value.status == native_lib.DA_ERR_INVALID_ARG
