"""GPU tests of the drop-in boundary itself: the C++ entry point decoding_attn() with the reference's
signature (csrc/ops/decoding_attn.h:29-30) executed through its mangled symbol, its exit()-on-error
contract (csrc/common/common.h:17-23), and the failure paths of the bounded waits."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

from decoding_attention_b200 import synth
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MANGLED = "_Z13decoding_attnPvS_S_S_PimmmmmmbbP11CUstream_st"


def cpp_entry(cabi):
    fn = getattr(cabi.lib(), MANGLED)
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_void_p] + [ctypes.c_size_t] * 6 + [ctypes.c_bool, ctypes.c_bool,
                                                                                     ctypes.c_void_p]
    return fn


@pytest.mark.parametrize("case", ["mha", "gqa_alibi_bf16", "mla"])
def test_cpp_decoding_attn_entry_point(native_lib, oracle, case):
    if case == "mha":
        w = synth.Workload("cpp_mha", torch.float16, 32, 32, 128, 128, [300, 64, 1], dist="normal", seed=61)
    elif case == "gqa_alibi_bf16":
        w = synth.Workload("cpp_gqa", torch.bfloat16, 32, 8, 128, 128, [700, 33], is_alibi=True, dist="normal", scale=0.5, seed=62)
    else:
        w = synth.Workload("cpp_mla", torch.bfloat16, 128, 1, 576, 512, [400, 130], dist="normal", scale=0.3, mla=True, seed=63)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=w.is_alibi)
    dq, dk, dcu = q.to(DEV), k.to(DEV), cu.to(DEV)
    dv = v.to(DEV) if v is not None else None
    o = torch.full((w.batch, w.head_q, w.dim_v), float("nan"), dtype=w.dtype, device=DEV)
    before = native_lib.launch_count()
    cpp_entry(native_lib)(dq.data_ptr(), dk.data_ptr(), dv.data_ptr() if dv is not None else None, o.data_ptr(),
                          dcu.data_ptr(), w.max_seq_k, w.batch, w.head_q, w.head_k, w.dim, w.dim_v, w.is_alibi,
                          w.dtype == torch.bfloat16, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert native_lib.launch_count() > before
    assert_close(o, expect, w.name)


def test_cpp_decoding_attn_exits_on_error(native_lib):
    """Like the reference's DA_CHECK, the C++ entry point logs and terminates the process on a bad call."""
    code = f"""
import ctypes, sys, torch
sys.path.insert(0, {ROOT!r})
from decoding_attention_b200 import cabi
fn = getattr(cabi.lib(), {MANGLED!r})
fn.restype = None
fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_size_t] * 6 + [ctypes.c_bool, ctypes.c_bool, ctypes.c_void_p]
t = torch.zeros(1, 8, 128, dtype=torch.float16, device="cuda:0")
cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda:0")
fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), cu.data_ptr(), 1, 1, 8, 3, 128, 128, False, False, None)
print("SURVIVED")
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode != 0 and "SURVIVED" not in r.stdout
    assert "[decoding_attn]" in r.stderr and "head_q" in r.stderr


def test_a_past_timeout_does_not_silence_later_launches(native_lib, oracle):
    """After a bounded wait has run out (status word set, never read), tensor-core launches must still compute."""
    assert native_lib.device_status() == native_lib.DA_OK
    native_lib.check(native_lib.lib().da_selftest_wait_timeout(None))
    torch.cuda.synchronize()
    for w in (synth.Workload("after_to_mla", torch.bfloat16, 128, 1, 576, 512, [300, 64], dist="normal", scale=0.3, mla=True, seed=64),
              synth.Workload("after_to_mqa", torch.float16, 32, 1, 128, 128, [500], dist="normal", seed=65)):
        q, k, v, cu = w.make("cpu")
        expect = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v)
        o = torch.full((w.batch, w.head_q, w.dim_v), float("nan"), dtype=w.dtype, device=DEV)
        native_lib.decode_fwd(native_lib.make_args(q.to(DEV), k.to(DEV), v.to(DEV) if v is not None else None, o, cu.to(DEV),
                                                   w.max_seq_k, w.dim_v))
        torch.cuda.synchronize()
        assert_close(o, expect, w.name)
    assert native_lib.device_status() == native_lib.DA_ERR_TIMEOUT  # the old report is still there, once
    assert native_lib.device_status() == native_lib.DA_OK


def test_exchange_kernel_gives_up_on_a_peer_that_never_posts(native_lib, oracle):
    """da_exchange_merge with world = 2 on one GPU: both gather buffers are local, nobody plays rank 1, so the
    wait for its flag runs out after the short bound given here.  The kernel must return, report the timeout
    once, leave the context usable, and a later ordinary call must be right."""
    rows, dv = 64, 128
    lib = native_lib.lib()
    nbytes = lib.da_exchange_buffer_bytes(2, rows, dv)
    bufs = [torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV) for _ in range(2)]
    rec = torch.randn(rows * (dv + 1), dtype=torch.float32, device=DEV)
    o = torch.full((rows, dv), 7.0, dtype=torch.float16, device=DEV)
    ptrs = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    assert native_lib.device_status() == native_lib.DA_OK
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    native_lib.check(lib.da_exchange_merge_bounded(rec.data_ptr(), ptrs, 2, 0, rows, dv, 1, o.data_ptr(), None, 0, None,
                                                   2_000_000))  # about a millisecond of SM clocks
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 200.0, "the bounded wait did not end in time"
    assert native_lib.device_status() == native_lib.DA_ERR_TIMEOUT
    assert native_lib.device_status() == native_lib.DA_OK
    assert (o == 7.0).all(), "rows must be left unwritten when the exchange gives up"
    # rank 0's record did reach its slot of "rank 1"'s buffer (the push happens before the wait): slots are laid
    # out [epoch parity][rank], each rows * (dv + 1) floats rounded up to a multiple of 4
    slot = (rows * (dv + 1) + 3) // 4 * 4
    at = (1 * 2 + 0) * slot
    assert torch.equal(bufs[1][at:at + rows * dv], rec[:rows * dv])
    w = synth.Workload("after_xchg", torch.float16, 8, 2, 128, 128, [300], dist="normal", seed=66)
    q, k, v, cu = w.make("cpu")
    o2 = torch.empty(1, 8, 128, dtype=w.dtype, device=DEV)
    native_lib.decode_fwd(native_lib.make_args(q.to(DEV), k.to(DEV), v.to(DEV), o2, cu.to(DEV), 300, 128))
    torch.cuda.synchronize()
    assert_close(o2, oracle.attn_cpu(q, k, v, cu), "after the exchange timeout")
