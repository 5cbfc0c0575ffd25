"""GPU tests of the Python call surface (``decoding_attn.decoding_attn_fwd`` and the torch extension
``decoding_attn_cuda`` under it), written the way the reference tests its own
(tests/test_decoding_attn.py:61-128): random q/k/v of a shape grid, the library against a plain
torch attention in fp32, mean |diff| <= 5e-3 -- plus the CPU oracle with the element-wise tolerance
2e-3 + 1e-2 |x| used everywhere else in this suite.
"""
import math

import pytest
import torch

from decoding_attention_b200 import synth
from helpers import REF_MEAN_ABS, assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def api():
    import decoding_attn  # the reference's import name
    return decoding_attn


def torch_attn(q, k, v, cu, dim_v, softmax_scale=None):
    """Plain fp32 torch attention per sequence (the checker of tests/test_decoding_attn.py:35-57,
    restated for packed variable-length inputs)."""
    out = []
    group = q.shape[1] // k.shape[1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[2])
    for b in range(q.shape[0]):
        kb = k[cu[b]:cu[b + 1]].float().repeat_interleave(group, dim=1)            # [s, hq, d]
        vb = (v if v is not None else k[..., :dim_v])[cu[b]:cu[b + 1]].float().repeat_interleave(group, dim=1)
        s = torch.einsum("hd,shd->hs", q[b].float(), kb) * scale
        out.append(torch.einsum("hs,shd->hd", torch.softmax(s, dim=-1), vb))
    return torch.stack(out)


# The reference grid (tests/test_decoding_attn.py:61-66), thinned to one pass over every axis.
GRID = [(1, 1, 32, 32, 128, torch.float16), (2, 128, 32, 8, 128, torch.bfloat16), (16, 512, 64, 8, 128, torch.float16),
        (2, 512, 32, 32, 64, torch.bfloat16), (2, 128, 32, 8, 96, torch.float16), (2, 512, 32, 8, 256, torch.bfloat16)]


@pytest.mark.parametrize("batch,seq_k,head_q,head_k,dim,dt", GRID)
def test_decoding_attn_fwd_like_the_reference_suite(api, oracle, batch, seq_k, head_q, head_k, dim, dt):
    w = synth.Workload("ref_suite", dt, head_q, head_k, dim, dim, [seq_k] * batch, dist="normal", seed=5)
    q, k, v, cu = w.make("cpu")
    out = api.decoding_attn_fwd(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), seq_k, dim, False)
    assert out.shape == (batch, head_q, dim) and out.dtype == dt and out.device.type == "cuda"
    ref = torch_attn(q, k, v, cu.tolist(), dim)
    assert (out.float().cpu() - ref).abs().mean().item() <= REF_MEAN_ABS
    assert_close(out, oracle.attn_cpu(q, k, v, cu), "decoding_attn_fwd vs oracle")


@pytest.mark.parametrize("batch,seq_k,head_q,dt", [(1, 1, 128, torch.bfloat16), (2, 512, 128, torch.float16), (2, 128, 16, torch.bfloat16)])
def test_decoding_attn_fwd_mla_like_the_reference_suite(api, oracle, batch, seq_k, head_q, dt):
    """tests/test_decoding_attn.py:97-128: v = None, dim 576, dim_v 512, one KV head."""
    w = synth.Workload("ref_suite_mla", dt, head_q, 1, 576, 512, [seq_k] * batch, dist="normal", scale=0.3, mla=True, seed=6)
    q, k, v, cu = w.make("cpu")
    assert v is None
    out = api.decoding_attn_fwd(q.to(DEV), k.to(DEV), None, cu.to(DEV), seq_k, 512, False)
    ref = torch_attn(q, k, None, cu.tolist(), 512)
    assert (out.float().cpu() - ref).abs().mean().item() <= REF_MEAN_ABS
    assert_close(out, oracle.attn_cpu(q, k, None, cu, dim_v=512), "mla decoding_attn_fwd vs oracle")


def test_named_entry_points_scale_out_and_lse(api, oracle):
    w = synth.Workload("named", torch.float16, 32, 8, 128, 128, [300, 77], dist="normal", seed=7)
    q, k, v, cu = w.make("cpu")
    dq, dk, dv, dcu = q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV)
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, softmax_scale=0.2, is_alibi=True, return_lse=True)
    out_buf = torch.empty(2, 32, 128, dtype=torch.float16, device=DEV)
    out, lse = api.dmha_fwd(dq, dk, dv, dcu, 300, is_alibi=True, softmax_scale=0.2, out=out_buf, return_lse=True)
    assert out.data_ptr() == out_buf.data_ptr()
    assert_close(out, expect, "dmha_fwd")
    assert (lse.cpu() - lse_e).abs().max().item() <= 2e-3
    # keyword-only scale on the reference-shaped call
    out2 = api.decoding_attn_fwd(dq, dk, dv, dcu, 300, 128, True, softmax_scale=0.2)
    assert torch.equal(out2, out)

    wm = synth.Workload("named_mla", torch.bfloat16, 128, 1, 576, 512, [200], dist="normal", scale=0.3, mla=True, seed=8)
    q, kv, _, cu = wm.make("cpu")
    expect = oracle.attn_cpu(q, kv, None, cu, dim_v=512, softmax_scale=0.05)
    assert_close(api.dmla_fwd(q.to(DEV), kv.to(DEV), cu.to(DEV), 200, softmax_scale=0.05), expect, "dmla_fwd")


def test_mla_keeps_alibi_with_and_without_scale(api, oracle):
    """The reference's fwd() honours is_alibi when v is None (csrc/torch/decoding_torch.cpp:19-21, :76-77)."""
    wm = synth.Workload("mla_alibi", torch.bfloat16, 128, 1, 576, 512, [333, 70], is_alibi=True, dist="normal", scale=0.3,
                        mla=True, seed=12)
    q, kv, _, cu = wm.make("cpu")
    dq, dkv, dcu = q.to(DEV), kv.to(DEV), cu.to(DEV)
    plain = oracle.attn_cpu(q, kv, None, cu, dim_v=512, is_alibi=False)
    expect = oracle.attn_cpu(q, kv, None, cu, dim_v=512, is_alibi=True)
    assert (plain.float() - expect.float()).abs().max().item() > 1e-2, "the case must be sensitive to the bias"
    assert_close(api.decoding_attn_fwd(dq, dkv, None, dcu, 333, 512, True), expect, "fwd, v None, alibi")
    expect_s = oracle.attn_cpu(q, kv, None, cu, dim_v=512, is_alibi=True, softmax_scale=0.05)
    assert_close(api.decoding_attn_fwd(dq, dkv, None, dcu, 333, 512, True, softmax_scale=0.05), expect_s,
                 "decoding_attn_fwd, v None, alibi, scale")
    assert_close(api.dmla_fwd(dq, dkv, dcu, 333, softmax_scale=0.05, is_alibi=True), expect_s, "dmla_fwd alibi")


def test_two_streams_and_graph_capture_through_the_binding(api, oracle):
    """The binding takes its split scratch from torch's stream-ordered allocator: calls on two streams of one
    device do not share it, and a call can be captured in a CUDA graph and replayed."""
    w = synth.Workload("streams", torch.bfloat16, 32, 8, 128, 128, [4000, 900, 2500], dist="normal", scale=0.5, seed=13)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu)
    dq, dk, dv, dcu = q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for _ in range(4):
        for st in (s1, s2):
            with torch.cuda.stream(st):
                outs.append(api.decoding_attn_fwd(dq, dk, dv, dcu, 4000, 128, False))
    torch.cuda.synchronize()
    for o in outs:
        assert_close(o, expect, "two streams")
    out = torch.zeros(3, 32, 128, dtype=w.dtype, device=DEV)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        api.dmha_fwd(dq, dk, dv, dcu, 4000, out=out)  # warm-up outside the capture
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            api.dmha_fwd(dq, dk, dv, dcu, 4000, out=out)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert_close(out, expect, "graph replay through the binding")


def test_non_contiguous_inputs_are_made_contiguous(api, oracle):
    """decoding_attn_interface.py:20-21, :50: maybe_contiguous on q, k, v."""
    w = synth.Workload("noncontig", torch.float16, 8, 8, 64, 64, [90, 40], dist="normal", seed=9)
    q, k, v, cu = w.make("cpu")
    kt = k.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)  # last stride != 1
    assert kt.stride(-1) != 1
    out = api.decoding_attn_fwd(q.to(DEV), kt, v.to(DEV), cu.to(DEV), 90, 64, False)
    assert_close(out, oracle.attn_cpu(q, k, v, cu), "non-contiguous k")


def test_paged_fwd(oracle):
    from decoding_attention_b200 import paged_fwd
    from test_decode_gpu import to_pages
    w = synth.Workload("paged_api", torch.bfloat16, 32, 8, 128, 128, [513, 64, 700], dist="normal", scale=0.5, seed=10)
    q, k, v, cu = w.make("cpu")
    k_pool, v_pool, table = to_pages(k, v, cu, 64, seed=1)
    lens = torch.tensor(w.seq_lens, dtype=torch.int32, device=DEV)
    out, lse = paged_fwd(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), lens, table.to(DEV), return_lse=True)
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, return_lse=True)
    assert_close(out, expect, "paged_fwd")
    assert (lse.cpu() - lse_e).abs().max().item() <= 2e-3

    wm = synth.Workload("paged_api_mla", torch.bfloat16, 128, 1, 576, 512, [300, 65], dist="normal", scale=0.3, mla=True, seed=11)
    q, kv, _, cu = wm.make("cpu")
    kv_pool, _, table = to_pages(kv, None, cu, 64, seed=2)
    lens = torch.tensor(wm.seq_lens, dtype=torch.int32, device=DEV)
    out = paged_fwd(q.to(DEV), kv_pool.to(DEV), None, lens, table.to(DEV), dim_v=512)
    assert_close(out, oracle.attn_cpu(q, kv, None, cu, dim_v=512), "paged_fwd mla")


def test_binding_checks_raise(api):
    """The binding's TORCH_CHECKs (decoding_torch.cpp:25-70) surface as exceptions, not exits."""
    import decoding_attn_cuda
    q = torch.zeros(2, 8, 128, dtype=torch.float16, device=DEV)
    k = torch.zeros(20, 8, 128, dtype=torch.float16, device=DEV)
    cu = torch.tensor([0, 10, 20], dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):  # dtype
        decoding_attn_cuda.fwd(q.float(), k.float(), k.float(), None, cu, 10, 128, False)
    with pytest.raises(RuntimeError):  # cu_seq_k dtype
        decoding_attn_cuda.fwd(q, k, k, None, cu.long(), 10, 128, False)
    with pytest.raises(RuntimeError):  # head_q % head_k
        decoding_attn_cuda.fwd(q, k[:, :3], k[:, :3], None, cu, 10, 128, False)
    with pytest.raises(RuntimeError):  # one query token per sequence
        decoding_attn_cuda.fwd(q[:1], k, k, None, cu, 10, 128, False)
    with pytest.raises(RuntimeError):  # unsupported head dim: an error here, a silent no-op in the reference
        decoding_attn_cuda.fwd(q[..., :32], k[..., :32], k[..., :32], None, cu, 10, 32, False)
    with pytest.raises(RuntimeError):  # CPU tensors
        decoding_attn_cuda.fwd(q.cpu(), k.cpu(), k.cpu(), None, cu.cpu(), 10, 128, False)
