"""GPU parity tests: the CUDA path, called through the C ABI (ctypes), against the CPU oracle on
identical seeded inputs.  Tolerance: |out - oracle| <= 2e-3 + 1e-2 |oracle| element-wise (fp32
accumulation, fp16/bf16 outputs) and the reference suite's mean |diff| <= 5e-3."""
import pytest
import torch

from decoding_attention_b200 import synth
from helpers import assert_close, merge_reference

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_cabi(cabi, w, q, k, v, cu, num_splits=0, want_lse=False, softmax_scale=None, pos_offset=None, total_len=None,
             workspace=None):
    o = torch.empty(q.shape[0], w.head_q, w.dim_v, dtype=w.dtype, device=q.device)
    lse = torch.empty(q.shape[0], w.head_q, dtype=torch.float32, device=q.device) if want_lse else None
    args = cabi.make_args(q, k, v, o, cu, max(w.max_seq_k, 1), w.dim_v, is_alibi=w.is_alibi, lse=lse,
                          softmax_scale=softmax_scale, num_splits=num_splits, kv_pos_offset=pos_offset,
                          kv_total_len=total_len, workspace=workspace,
                          stream=torch.cuda.current_stream().cuda_stream)
    cabi.decode_fwd(args)
    torch.cuda.synchronize()
    assert cabi.device_status() == cabi.DA_OK
    return (o, lse) if want_lse else o


def check(cabi, oracle, w, num_splits=0, **kw):
    q, k, v, cu = w.make("cpu")
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=w.is_alibi, return_lse=True,
                                    softmax_scale=kw.get("softmax_scale"))
    dq, dk, dv, dcu = q.to(DEV), k.to(DEV), (v.to(DEV) if v is not None else None), cu.to(DEV)
    before = cabi.launch_count()
    o, lse = run_cabi(cabi, w, dq, dk, dv, dcu, num_splits=num_splits, want_lse=True, **kw)
    assert cabi.launch_count() > before, "no kernel of this library was launched"
    assert_close(o, expect, w.name)
    fin = torch.isfinite(lse_e)
    assert (lse.cpu()[fin] - lse_e[fin]).abs().max().item() <= 2e-3 if fin.any() else True
    assert torch.equal(torch.isinf(lse.cpu()), ~fin)
    return o


# The reference suite's whole grid (tests/test_decoding_attn.py:61-66): 2 x 2 x 4 x 3 x 3 x 2 = 288 cases.
@pytest.mark.parametrize("hq", [32, 64])
@pytest.mark.parametrize("hk", [8, 32])
@pytest.mark.parametrize("d", [64, 96, 128, 256])
@pytest.mark.parametrize("b", [1, 2, 16])
@pytest.mark.parametrize("s", [1, 128, 512])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_reference_grid_mha_gqa(native_lib, oracle, hq, hk, d, b, s, dt):
    w = synth.Workload(f"grid_{hq}_{hk}_{d}_{b}_{s}", dt, hq, hk, d, d, [s] * b, dist="normal", seed=11)
    check(native_lib, oracle, w)


# tests/test_decoding_attn.py:97-104: 4 x 3 x 3 x 2 = 72 cases.
@pytest.mark.parametrize("hq", [16, 32, 64, 128])
@pytest.mark.parametrize("b", [1, 2, 16])
@pytest.mark.parametrize("s", [1, 128, 512])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_reference_grid_mla(native_lib, oracle, hq, b, s, dt):
    w = synth.Workload(f"mla_{hq}_{b}_{s}", dt, hq, 1, 576, 512, [s] * b, dist="normal", scale=0.5, mla=True, seed=12)
    check(native_lib, oracle, w)


@pytest.mark.parametrize("lens", [[128], [64], [33], [1], [129, 0, 700], [2100], [257, 256, 255]])
@pytest.mark.parametrize("hq", [128, 96, 64, 16, 8])
def test_mla_pair_kernel_edges(native_lib, oracle, lens, hq):
    """The latent-KV kernel on SM pairs: ragged last tiles (one or both CTAs of the pair past the end), empty
    sequences, head counts that leave the second CTA partly or wholly padding, splits, ALiBi."""
    w = synth.Workload(f"mla2_{hq}_{lens}", torch.bfloat16, hq, 1, 576, 512, lens, is_alibi=(len(lens) > 1), dist="normal",
                       scale=0.3, mla=True, seed=23)
    check(native_lib, oracle, w)
    check(native_lib, oracle, w, num_splits=3)


@pytest.mark.parametrize("lens", [[1], [2], [7], [63], [64], [65], [127, 129], [0, 5], [5, 0, 0, 300], [1000, 3, 64]])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_edges_varlen_and_splits(native_lib, oracle, lens, splits):
    w = synth.Workload(f"edge_{lens}_{splits}", torch.float16, 8, 2, 128, 128, lens, dist="normal", seed=13)
    check(native_lib, oracle, w, num_splits=splits)


@pytest.mark.parametrize("hq,hk,d", [(32, 32, 128), (32, 8, 128), (32, 1, 128), (16, 4, 64), (12, 4, 96), (8, 2, 256)])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_alibi(native_lib, oracle, hq, hk, d, dt):
    w = synth.Workload(f"alibi_{hq}_{hk}_{d}", dt, hq, hk, d, d, [700, 33, 1], is_alibi=True, dist="uniform", seed=14)
    check(native_lib, oracle, w)
    check(native_lib, oracle, w, num_splits=4)


@pytest.mark.parametrize("group", [1, 2, 3, 4, 6, 8, 16, 32])
def test_head_ratios(native_lib, oracle, group):
    w = synth.Workload(f"ratio_{group}", torch.bfloat16, 2 * group, 2, 128, 128, [200, 77], dist="normal", seed=15)
    check(native_lib, oracle, w)


def test_softmax_scale_argument(native_lib, oracle):
    w = synth.Workload("scale", torch.float16, 8, 2, 128, 128, [150], dist="normal", seed=16)
    check(native_lib, oracle, w, softmax_scale=0.2)


def test_split_count_does_not_change_result_much_and_is_deterministic(native_lib, oracle):
    w = synth.Workload("det", torch.bfloat16, 32, 8, 128, 128, [3000, 800], dist="normal", scale=0.5, seed=17)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    a = run_cabi(native_lib, w, q, k, v, cu, num_splits=5)
    b = run_cabi(native_lib, w, q, k, v, cu, num_splits=5)
    assert torch.equal(a, b), "same split count must be bit-reproducible"
    c = run_cabi(native_lib, w, q, k, v, cu, num_splits=1)
    assert_close(a, c, "splits 5 vs 1")


def test_caller_workspace_with_canaries(native_lib, oracle):
    w = synth.Workload("ws", torch.float16, 16, 4, 128, 128, [900, 100], dist="normal", seed=18)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    o = torch.empty(2, 16, 128, dtype=w.dtype, device=DEV)
    args = native_lib.make_args(q, k, v, o, cu, w.max_seq_k, 128, num_splits=4)
    need = native_lib.workspace_bytes(args)
    assert need > 0
    pad = 1024
    buf = torch.full((need + 2 * pad,), 0x5A, dtype=torch.uint8, device=DEV)
    ws = buf[pad:pad + need]
    out = run_cabi(native_lib, w, q, k, v, cu, num_splits=4, workspace=ws)
    assert (buf[:pad] == 0x5A).all() and (buf[pad + need:] == 0x5A).all(), "wrote outside the workspace"
    expect = oracle.attn_cpu(*w.make("cpu"))
    assert_close(out, expect, "workspace")
    small = buf[pad:pad + need // 2]
    with pytest.raises(native_lib.DecodingAttnError) as e:
        run_cabi(native_lib, w, q, k, v, cu, num_splits=4, workspace=small)
    assert e.value.status == native_lib.DA_ERR_WORKSPACE


def test_padded_row_strides(native_lib, oracle):
    w = synth.Workload("stride", torch.float16, 8, 2, 128, 128, [130, 40], dist="normal", seed=19)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu)
    kp = torch.zeros(k.shape[0], 3, 128, dtype=w.dtype, device=DEV)
    vp = torch.zeros(v.shape[0], 4, 128, dtype=w.dtype, device=DEV)
    kp[:, :2] = k.to(DEV)
    vp[:, :2] = v.to(DEV)
    out = run_cabi(native_lib, w, q.to(DEV), kp[:, :2], vp[:, :2], cu.to(DEV))
    assert_close(out, expect, "strided rows")


def test_key_range_shards_merge(native_lib, oracle):
    """Key-range sharding as used across GPUs, emulated on one: per-shard (o fp32, lse) with the
    ALiBi position offset, merged by da_merge_partials, equals the unsharded result."""
    w = synth.Workload("shard", torch.bfloat16, 32, 32, 128, 128, [5000], is_alibi=True, dist="normal", scale=0.5,
                       seed=20)
    q, k, v, cu = w.make("cpu")
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, is_alibi=True, return_lse=True)
    dq = q.to(DEV)
    parts_o, parts_lse = [], []
    bounds = [0, 1250, 2500, 3750, 5000]
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        ks, vs = k[lo:hi].to(DEV), v[lo:hi].to(DEV)
        cus = torch.tensor([0, hi - lo], dtype=torch.int32, device=DEV)
        o32 = torch.empty(1, 32, 128, dtype=torch.float32, device=DEV)
        lse = torch.empty(1, 32, dtype=torch.float32, device=DEV)
        args = native_lib.make_args(dq, ks, vs, None, cus, hi - lo, 128, is_alibi=True, lse=lse, o_f32=o32,
                                    kv_pos_offset=torch.tensor([lo], dtype=torch.int32, device=DEV),
                                    kv_total_len=torch.tensor([5000], dtype=torch.int32, device=DEV))
        native_lib.decode_fwd(args)
        parts_o.append(o32.view(32, 128))
        parts_lse.append(lse.view(32))
    po, pl = torch.stack(parts_o).contiguous(), torch.stack(parts_lse).contiguous()
    o = torch.empty(32, 128, dtype=w.dtype, device=DEV)
    lse = torch.empty(32, dtype=torch.float32, device=DEV)
    native_lib.check(native_lib.lib().da_merge_partials(po.data_ptr(), pl.data_ptr(), 4, 32, 128, 32 * 128, 128, 32, 1,
                                                        o.data_ptr(), None, lse.data_ptr(), 1, None))
    torch.cuda.synchronize()
    assert_close(o.view(1, 32, 128), expect, "sharded + merged")
    assert (lse.cpu() - lse_e.view(-1)).abs().max().item() < 2e-3
    o_chk, _ = merge_reference(po.cpu(), pl.cpu())
    assert (o.float().cpu() - o_chk.float()).abs().max().item() < 2e-2


def test_host_buffer_entry_point(native_lib, oracle):
    w = synth.Workload("host", torch.float16, 32, 8, 128, 128, [513, 100, 2000], dist="normal", seed=21)
    q, k, v, cu = [t.pin_memory() for t in w.make("cpu")]
    o = torch.empty(3, 32, 128, dtype=w.dtype).pin_memory()
    args = native_lib.make_args(q, k, v, o, cu, w.max_seq_k, 128, packed=True)
    native_lib.decode_fwd_host(args)
    assert_close(o, oracle.attn_cpu(q, k, v, cu), "host entry point")


def test_argument_errors(native_lib):
    w = synth.Workload("err", torch.float16, 8, 2, 128, 128, [16], dist="normal", seed=22)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    o = torch.empty(1, 8, 128, dtype=w.dtype, device=DEV)
    bad = native_lib.make_args(q, k, v, o, cu, 16, 64)  # (128, 64) is not a supported pair
    with pytest.raises(native_lib.DecodingAttnError) as e:
        native_lib.decode_fwd(bad)
    assert e.value.status == native_lib.DA_ERR_UNSUPPORTED
    bad = native_lib.make_args(q, k, v, o, cu, 16, 128)
    bad.head_k = 3
    with pytest.raises(native_lib.DecodingAttnError) as e:
        native_lib.decode_fwd(bad)
    assert e.value.status == native_lib.DA_ERR_INVALID_ARG
    bad = native_lib.make_args(q, k, v, o, cu, 16, 128)
    bad.q = None
    with pytest.raises(native_lib.DecodingAttnError):
        native_lib.decode_fwd(bad)


def test_bounded_wait_gives_up_and_reports(native_lib, oracle):
    """Failure path without a fault: a wait that nothing satisfies runs out after ~1 ms, the status word
    reports it once, and the context keeps working."""
    assert native_lib.device_status() == native_lib.DA_OK
    native_lib.check(native_lib.lib().da_selftest_wait_timeout(None))
    assert native_lib.device_status() == native_lib.DA_ERR_TIMEOUT
    assert b"bounded wait" in native_lib.lib().da_last_error()
    assert native_lib.device_status() == native_lib.DA_OK  # cleared by the read
    w = synth.Workload("after_timeout", torch.float16, 8, 2, 128, 128, [300], dist="normal", seed=41)
    check(native_lib, oracle, w)


def test_cuda_graph_replay(native_lib, oracle):
    """The call is stream-ordered with no host synchronisation: after a warm-up call (attribute set-up,
    tensor maps) it can be captured in a CUDA graph with a caller workspace and replayed."""
    w = synth.Workload("graph", torch.bfloat16, 32, 8, 128, 128, [1500, 64, 700], dist="normal", scale=0.5, seed=42)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    expect = oracle.attn_cpu(*w.make("cpu"))
    o = torch.zeros(3, 32, 128, dtype=w.dtype, device=DEV)
    probe = native_lib.make_args(q, k, v, o, cu, w.max_seq_k, 128, num_splits=3)
    ws = torch.empty(native_lib.workspace_bytes(probe), dtype=torch.uint8, device=DEV)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        args = native_lib.make_args(q, k, v, o, cu, w.max_seq_k, 128, num_splits=3, workspace=ws,
                                    stream=side.cuda_stream)
        native_lib.decode_fwd(args)  # warm-up outside the capture
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            native_lib.decode_fwd(args)
    o.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert_close(o, expect, "graph replay")
    q.copy_(torch.roll(q, 1, dims=1))  # new query, same graph
    g.replay()
    torch.cuda.synchronize()
    expect2 = oracle.attn_cpu(q.cpu(), *w.make("cpu")[1:])
    assert_close(o, expect2, "graph replay with new q")


def to_pages(k, v, cu, page_size, seed):
    """Scatter a packed cache into a shuffled page pool whose unused rows are NaN (a kernel that reads
    a row it should not turns the output NaN).  Returns (k_pool, v_pool, block_table)."""
    g = torch.Generator().manual_seed(seed)
    lens = (cu[1:] - cu[:-1]).tolist()
    blocks = [(n + page_size - 1) // page_size for n in lens]
    n_pages = sum(blocks) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    fill = 0x7F if k.dtype == torch.uint8 else float("nan")  # 0x7f is NaN in FP8 e4m3 (pools passed as raw bytes)
    k_pool = torch.full((n_pages, page_size) + tuple(k.shape[1:]), fill, dtype=k.dtype)
    v_pool = torch.full((n_pages, page_size) + tuple(v.shape[1:]), fill, dtype=v.dtype) if v is not None else None
    table = torch.zeros(len(lens), max(max(blocks), 1) + 1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(lens):
        for i in range(blocks[b]):
            page = order[nxt]
            nxt += 1
            table[b, i] = page
            lo = int(cu[b]) + i * page_size
            hi = min(lo + page_size, int(cu[b]) + n)
            k_pool[page, :hi - lo] = k[lo:hi]
            if v is not None:
                v_pool[page, :hi - lo] = v[lo:hi]
    return k_pool, v_pool, table


PAGED = [
    # dtype, head_q, head_k, dim, dim_v, lens, page_size, alibi, splits
    (torch.bfloat16, 32, 8, 128, 128, [700, 64, 1, 129, 0], 64, False, 0),     # CUDA-core kernel, 4 heads per CTA
    (torch.float16, 32, 8, 128, 128, [700, 64, 1, 129], 128, True, 3),
    (torch.float16, 16, 16, 64, 64, [333, 1000], 128, False, 0),
    (torch.bfloat16, 8, 4, 96, 96, [257, 31], 256, False, 2),
    (torch.float16, 8, 2, 256, 256, [100, 400], 64, False, 0),                # 32-key tiles
    (torch.float16, 32, 1, 128, 128, [300, 2048, 65], 64, True, 0),            # tensor-core GQA kernel
    (torch.bfloat16, 128, 1, 576, 512, [500, 64, 1000, 1], 64, False, 0),      # tensor-core MLA kernel
    (torch.bfloat16, 128, 1, 576, 512, [900, 130], 128, False, 2),
    (torch.float16, 16, 1, 576, 512, [200, 70], 64, False, 0),                 # tensor-core MLA kernel, 16 heads
    (torch.float16, 4, 1, 576, 512, [200, 70], 32, False, 0),                  # CUDA-core MLA kernel, short pages
    # pages shorter than a key tile (vLLM's default is 16): a tile is fetched page by page
    (torch.bfloat16, 32, 8, 128, 128, [700, 64, 1, 129, 17], 16, False, 0),
    (torch.float16, 32, 8, 128, 128, [333, 50], 32, True, 3),
    (torch.float16, 8, 2, 256, 256, [100, 400], 16, False, 0),
    (torch.bfloat16, 16, 16, 64, 64, [333, 1000], 16, False, 2),
    (torch.float16, 32, 1, 128, 128, [300, 2048, 65], 16, True, 0),            # tensor-core GQA kernel
    (torch.bfloat16, 64, 8, 256, 256, [300, 90], 32, False, 0),
    (torch.bfloat16, 128, 1, 576, 512, [500, 64, 1000, 1], 16, False, 0),      # tensor-core MLA kernel
    (torch.float16, 128, 1, 576, 512, [900, 130], 32, True, 2),
]


@pytest.mark.parametrize("dt,hq,hk,d,dv,lens,page,alibi,splits", PAGED)
def test_paged_cache(native_lib, oracle, dt, hq, hk, d, dv, lens, page, alibi, splits):
    """Paged input (block table + page pool) gives what the packed cache gives: the oracle runs on the
    packed tensors, the library on a shuffled pool with NaN in every row no sequence owns."""
    mla = d == 576
    w = synth.Workload(f"paged_{d}_{page}", dt, hq, hk, d, dv, lens, is_alibi=alibi, dist="normal", scale=0.4, mla=mla, seed=77)
    q, k, v, cu = w.make("cpu")
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=dv, is_alibi=alibi, return_lse=True)
    k_pool, v_pool, table = to_pages(k, v, cu, page, seed=page + d)
    o = torch.full((len(lens), hq, dv), float("nan"), dtype=dt, device=DEV)
    lse = torch.empty(len(lens), hq, dtype=torch.float32, device=DEV)
    args = native_lib.make_args(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV) if v_pool is not None else None, o, cu.to(DEV),
                                max(w.max_seq_k, 1), dv, is_alibi=alibi, lse=lse, num_splits=splits,
                                block_table=table.to(DEV), page_size=page)
    native_lib.decode_fwd(args)
    torch.cuda.synchronize()
    assert native_lib.device_status() == native_lib.DA_OK
    assert_close(o, expect, w.name)
    fin = torch.isfinite(lse_e)
    assert (lse.cpu()[fin] - lse_e[fin]).abs().max().item() <= 2e-3
    assert torch.equal(torch.isinf(lse.cpu()), ~fin)


def test_paged_cache_argument_errors(native_lib):
    w = synth.Workload("paged_err", torch.float16, 8, 8, 128, 128, [100], seed=3)
    q, k, v, cu = [t.to(DEV) for t in w.make("cpu")]
    o = torch.empty(1, 8, 128, dtype=torch.float16, device=DEV)
    table = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    for page in (8, 96):  # too small; not a power of two
        with pytest.raises(native_lib.DecodingAttnError):
            native_lib.decode_fwd(native_lib.make_args(q, k, v, o, cu, 100, 128, block_table=table, page_size=page))
    with pytest.raises(native_lib.DecodingAttnError):  # table rows too short for max_seq_k
        native_lib.decode_fwd(native_lib.make_args(q, k, v, o, cu, 1000, 128, block_table=table, page_size=64))


@pytest.mark.parametrize("splits", [1, 0])
def test_longest_first_launch_order(native_lib, oracle, splits):
    """A grid of more than one wave of long CTAs takes its sequences longest first (a device-side sort of
    the batch by length): every sequence must still land in its own output row."""
    g = torch.Generator().manual_seed(99)
    lens = torch.randint(16, 3000, (64,), generator=g).tolist()
    lens[5], lens[40] = 0, 2999
    w = synth.Workload("order", torch.bfloat16, 32, 8, 128, 128, lens, dist="normal", scale=0.5, seed=98)
    q, k, v, cu = w.make("cpu")
    dq, dk, dv, dcu = q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV)
    o = torch.full((64, 32, 128), float("nan"), dtype=w.dtype, device=DEV)
    args = native_lib.make_args(dq, dk, dv, o, dcu, w.max_seq_k, 128, num_splits=splits)
    if splits == 1:  # partials are not needed, so any scratch is the launch-order array
        assert native_lib.workspace_bytes(args) >= 64 * 4
    native_lib.decode_fwd(args)
    torch.cuda.synchronize()
    assert native_lib.device_status() == native_lib.DA_OK
    assert_close(o, oracle.attn_cpu(q, k, v, cu), "longest-first order")


def test_cuda_graph_replay_with_launch_order_and_overlapped_launches(native_lib, oracle):
    """The longest-first order kernel, the attention kernel and the merge kernel are chained with
    programmatic dependent launches; the chain must survive stream capture and replay."""
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(900, 2600, (48,), generator=g).tolist()
    w = synth.Workload("graph_order", torch.float16, 32, 8, 128, 128, lens, dist="normal", scale=0.5, seed=8)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu)
    dq, dk, dv, dcu = q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV)
    o = torch.zeros(48, 32, 128, dtype=w.dtype, device=DEV)
    probe = native_lib.make_args(dq, dk, dv, o, dcu, w.max_seq_k, 128, num_splits=2)
    need = native_lib.workspace_bytes(probe)
    assert need > 48 * 32 * 2 * 129 * 4, "the plan must include the launch-order array"
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        args = native_lib.make_args(dq, dk, dv, o, dcu, w.max_seq_k, 128, num_splits=2, workspace=ws,
                                    stream=side.cuda_stream)
        native_lib.decode_fwd(args)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            native_lib.decode_fwd(args)
    for _ in range(3):
        o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert native_lib.device_status() == native_lib.DA_OK
        assert_close(o, expect, "graph replay with launch order")


def quantise_e4m3(x, scale):
    """(FP8 bytes, dequantised tensor in x's dtype): x / scale rounded to e4m3.  Every e4m3 value is exact in fp16 and
    bf16 and the scales used here are powers of two, so the dequantised cache the oracle sees is exactly what the
    kernel reconstructs."""
    x8 = (x.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return x8, (x8.float() * scale).to(x.dtype)


FP8_CASES = [
    # dtype, head_q, head_k, dim, lens, alibi, splits, k_scale, v_scale
    (torch.bfloat16, 32, 8, 128, [700, 64, 1, 129, 0], False, 0, 1.0, 1.0),
    (torch.float16, 32, 8, 128, [2100, 333], True, 3, 0.5, 0.25),
    (torch.float16, 32, 32, 128, [513], False, 0, 0.125, 2.0),
    (torch.bfloat16, 16, 4, 64, [333, 1000], False, 2, 0.5, 0.5),
    (torch.float16, 12, 4, 96, [257, 31], True, 0, 0.25, 1.0),
    (torch.bfloat16, 8, 2, 256, [100, 400], False, 0, 0.5, 0.5),
    (torch.float16, 32, 1, 128, [300, 65], True, 0, 0.25, 0.25),   # a group of 32: eight 4-head chunks on the CUDA-core kernel
]


@pytest.mark.parametrize("dt,hq,hk,d,lens,alibi,splits,ks,vs", FP8_CASES)
def test_fp8_kv_cache(native_lib, oracle, dt, hq, hk, d, lens, alibi, splits, ks, vs):
    """FP8 e4m3 K / V with per-tensor scales: the oracle runs on the dequantised cache (quantisation error is the
    caller's business, not the kernel's), so the usual tolerance applies."""
    w = synth.Workload(f"fp8_{d}_{hq}_{hk}", dt, hq, hk, d, d, lens, is_alibi=alibi, dist="normal", scale=0.5, seed=81)
    q, k, v, cu = w.make("cpu")
    k8, k_deq = quantise_e4m3(k, ks)
    v8, v_deq = quantise_e4m3(v, vs)
    expect, lse_e = oracle.attn_cpu(q, k_deq, v_deq, cu, dim_v=d, is_alibi=alibi, return_lse=True)
    o = torch.full((len(lens), hq, d), float("nan"), dtype=dt, device=DEV)
    lse = torch.empty(len(lens), hq, dtype=torch.float32, device=DEV)
    args = native_lib.make_args(q.to(DEV), k8.to(DEV), v8.to(DEV), o, cu.to(DEV), max(w.max_seq_k, 1), d, is_alibi=alibi,
                                lse=lse, num_splits=splits, k_scale=ks, v_scale=vs)
    before = native_lib.launch_count()
    native_lib.decode_fwd(args)
    torch.cuda.synchronize()
    assert native_lib.launch_count() > before and native_lib.device_status() == native_lib.DA_OK
    assert_close(o, expect, w.name)
    fin = torch.isfinite(lse_e)
    assert (lse.cpu()[fin] - lse_e[fin]).abs().max().item() <= 2e-3


def test_fp8_kv_cache_paged_and_errors(native_lib, oracle):
    w = synth.Workload("fp8_paged", torch.bfloat16, 32, 8, 128, 128, [700, 64, 130], dist="normal", scale=0.5, seed=82)
    q, k, v, cu = w.make("cpu")
    k8, k_deq = quantise_e4m3(k, 0.5)
    v8, v_deq = quantise_e4m3(v, 0.5)
    expect = oracle.attn_cpu(q, k_deq, v_deq, cu)
    for page in (64, 16):
        kp, vp, table = to_pages(k8.view(torch.uint8), v8.view(torch.uint8), cu, page, seed=5)
        kp, vp = kp.view(torch.float8_e4m3fn), vp.view(torch.float8_e4m3fn)  # rows no sequence owns hold NaN bytes
        o = torch.full((3, 32, 128), float("nan"), dtype=w.dtype, device=DEV)
        args = native_lib.make_args(q.to(DEV), kp.to(DEV), vp.to(DEV), o, cu.to(DEV), w.max_seq_k, 128, block_table=table.to(DEV),
                                    page_size=page, k_scale=0.5, v_scale=0.5)
        native_lib.decode_fwd(args)
        torch.cuda.synchronize()
        assert_close(o, expect, f"fp8 paged {page}")
    # the latent-KV shape has no FP8 path
    wm = synth.Workload("fp8_mla", torch.bfloat16, 128, 1, 576, 512, [64], dist="normal", scale=0.3, mla=True, seed=83)
    q, kv, _, cu = wm.make("cpu")
    kv8 = kv.float().to(torch.float8_e4m3fn)
    o = torch.empty(1, 128, 512, dtype=wm.dtype, device=DEV)
    with pytest.raises(native_lib.DecodingAttnError) as e:
        native_lib.decode_fwd(native_lib.make_args(q.to(DEV), kv8.to(DEV), None, o, cu.to(DEV), 64, 512))
    assert e.value.status == native_lib.DA_ERR_UNSUPPORTED


@pytest.mark.parametrize("hq,hk", [(64, 8), (40, 8), (32, 1), (24, 4)])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_head_dim_96_large_groups(native_lib, oracle, hq, hk, dt):
    """Head dim 96 with more than four query heads per KV head runs on the tensor-core kernel's 128-column
    instantiation (tensor maps zero-fill columns 96-127): ragged tiles, ALiBi, splits, paged caches."""
    w = synth.Workload(f"d96_{hq}_{hk}", dt, hq, hk, 96, 96, [700, 64, 1, 129, 0, 2100], is_alibi=True, dist="normal",
                       scale=0.5, seed=91)
    check(native_lib, oracle, w)
    check(native_lib, oracle, w, num_splits=3)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu, dim_v=96, is_alibi=True)
    for page in (64, 16):
        k_pool, v_pool, table = to_pages(k, v, cu, page, seed=page)
        o = torch.full((w.batch, hq, 96), float("nan"), dtype=dt, device=DEV)
        native_lib.decode_fwd(native_lib.make_args(q.to(DEV), k_pool.to(DEV), v_pool.to(DEV), o, cu.to(DEV), w.max_seq_k, 96,
                                                   is_alibi=True, block_table=table.to(DEV), page_size=page))
        torch.cuda.synchronize()
        assert_close(o, expect, f"{w.name} paged {page}")


def quantise_int(x, scale, bits):
    """(stored tensor, dequantised tensor in x's dtype) for signed `bits`-bit integers with one scale per tensor.
    8 bits: torch.int8.  4 bits: torch.uint8 of half the last dimension, the even element in the low nibble.
    Integers up to 127 times a power-of-two scale are exact in fp16 and bf16."""
    lim = (1 << (bits - 1)) - 1
    qi = torch.round(x.float() / scale).clamp(-lim - 1, lim).to(torch.int32)
    deq = (qi.float() * scale).to(x.dtype)
    if bits == 8:
        return qi.to(torch.int8), deq
    lo, hi = qi[..., 0::2] & 0xF, qi[..., 1::2] & 0xF
    return (lo | (hi << 4)).to(torch.uint8), deq


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("dt,hq,hk,d,lens,alibi,splits", [
    (torch.bfloat16, 32, 8, 128, [700, 64, 1, 129, 0], False, 0),
    (torch.float16, 32, 8, 128, [2100, 333], True, 3),
    (torch.bfloat16, 16, 4, 64, [333, 1000], False, 2),
    (torch.float16, 12, 4, 96, [257, 31], True, 0),
    (torch.bfloat16, 8, 2, 256, [100, 400], False, 0),
    (torch.float16, 32, 1, 128, [300, 65], False, 0),
])
def test_integer_kv_cache(native_lib, oracle, bits, dt, hq, hk, d, lens, alibi, splits):
    """Signed 8-bit and 4-bit K / V with per-tensor scales, against the oracle on the dequantised cache."""
    w = synth.Workload(f"int{bits}_{d}_{hq}_{hk}", dt, hq, hk, d, d, lens, is_alibi=alibi, dist="normal", scale=0.5, seed=85)
    q, k, v, cu = w.make("cpu")
    ks, vs = (2.0 ** -6, 2.0 ** -5) if bits == 8 else (0.25, 0.5)
    kq, k_deq = quantise_int(k, ks, bits)
    vq, v_deq = quantise_int(v, vs, bits)
    expect, lse_e = oracle.attn_cpu(q, k_deq, v_deq, cu, dim_v=d, is_alibi=alibi, return_lse=True)
    o = torch.full((len(lens), hq, d), float("nan"), dtype=dt, device=DEV)
    lse = torch.empty(len(lens), hq, dtype=torch.float32, device=DEV)
    args = native_lib.make_args(q.to(DEV), kq.to(DEV), vq.to(DEV), o, cu.to(DEV), max(w.max_seq_k, 1), d, is_alibi=alibi,
                                lse=lse, num_splits=splits, k_scale=ks, v_scale=vs, int4=(bits == 4))
    assert args.kv_dtype == (2 if bits == 8 else 3)
    native_lib.decode_fwd(args)
    torch.cuda.synchronize()
    assert native_lib.device_status() == native_lib.DA_OK
    assert_close(o, expect, w.name)
    fin = torch.isfinite(lse_e)
    assert (lse.cpu()[fin] - lse_e[fin]).abs().max().item() <= 2e-3


# Scores whose row maximum keeps rising along the sequence: the tensor-core kernels then have to raise their
# lazy reference maximum (and rescale the accumulator rows in tensor memory) many times, which seeded N(0,1)
# inputs hardly ever ask for.  Covers the four-stream kernel (groups of at most 32), the kernel for larger
# groups and head dim 256, and the latent-KV pair kernel; with ALiBi the same kernels walk the keys back to front.
@pytest.mark.parametrize("hq,hk,d,dv", [(32, 1, 128, 128), (64, 8, 128, 128), (16, 2, 64, 64), (64, 1, 128, 128),
                                        (16, 2, 256, 256), (128, 1, 576, 512)])
@pytest.mark.parametrize("alibi", [False, True])
@pytest.mark.parametrize("splits", [0, 1])
def test_rising_scores_take_the_rescale_path(native_lib, oracle, hq, hk, d, dv, alibi, splits):
    if alibi and d == 576:
        pytest.skip("covered by the interface tests")
    lens = [2048 + 37, 700]
    w = synth.Workload(f"rising_{hq}_{hk}_{d}", torch.bfloat16, hq, hk, d, dv, lens, dist="normal", scale=0.5, seed=29,
                       is_alibi=alibi, mla=(d == 576))
    q, k, v, cu = w.make("cpu")
    # key j of a sequence is scaled by 0.25 + 4 j / len: score magnitudes, and with them the running maximum, grow
    # (latent-KV rows: only the 64 columns that are not also V, three times as steeply, so that V keeps its range)
    for b, n in enumerate(lens):
        pos = torch.arange(n, dtype=torch.float32) / n
        if d == 576:
            k[cu[b]:cu[b] + n, :, 512:] = (k[cu[b]:cu[b] + n, :, 512:].float() * (0.25 + 12.0 * pos).view(n, 1, 1)).to(k.dtype)
        else:
            k[cu[b]:cu[b] + n] = (k[cu[b]:cu[b] + n].float() * (0.25 + 4.0 * pos).view(n, 1, 1)).to(k.dtype)
    scale = 0.5  # (1/sqrt(dim) would be 0.04 .. 0.125): the row maxima climb by some twenty units of log2, threshold 8
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v, is_alibi=alibi, return_lse=True, softmax_scale=scale)
    o, lse = run_cabi(native_lib, w, q.to(DEV), k.to(DEV), v.to(DEV) if v is not None else None, cu.to(DEV),
                      num_splits=splits, want_lse=True, softmax_scale=scale)
    assert_close(o, expect, w.name)
    assert (lse.cpu() - lse_e).abs().max().item() <= 5e-3


def test_total_k_hint_changes_the_plan_not_the_result(native_lib, oracle):
    """A ragged batch of fewer latent-KV sequences than CTA slots: with the optional total_k hint the planner
    splits the long sequences, without it every sequence runs unsplit; both agree with the oracle."""
    lens = [2048, 2000] + [64 + 7 * i for i in range(58)]  # 60 sequences on 74 pair slots, two of them long
    w = synth.Workload("ragged_mla", torch.bfloat16, 128, 1, 576, 512, lens, dist="normal", scale=0.5, seed=41, mla=True)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu, dim_v=w.dim_v)
    dq, dk, dcu = q.to(DEV), k.to(DEV), cu.to(DEV)
    plans = []
    for hint in (True, False):
        o = torch.empty(len(lens), w.head_q, w.dim_v, dtype=w.dtype, device=DEV)
        args = native_lib.make_args(dq, dk, None, o, dcu, max(lens), w.dim_v, stream=torch.cuda.current_stream().cuda_stream)
        assert args.total_k == sum(lens)
        if not hint:
            args.total_k = 0
        plans.append(native_lib.num_splits(args))
        native_lib.decode_fwd(args)
        torch.cuda.synchronize()
        assert native_lib.device_status() == native_lib.DA_OK
        assert_close(o, expect, f"{w.name}_hint{hint}")
    assert plans[0] > plans[1] == 1
