"""Seeded random sweep over the argument space of da_decode_fwd (through the C ABI) against the CPU
oracle: head counts and ratios, every supported (dim, dim_v), ragged lengths including 0 and 1,
ALiBi, explicit scale, forced split counts, packed and paged caches, padded row strides.
The cases are fixed by their seeds, so a failure names a reproducible case.  Same tolerance as the
other parity tests: |out - oracle| <= 2e-3 + 1e-2 |oracle|, mean |diff| <= 5e-3.
"""
import os
import random

import pytest
import torch

from decoding_attention_b200 import synth
from helpers import assert_close
from test_decode_gpu import to_pages

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

DIMS = [(64, 64), (96, 96), (128, 128), (256, 256), (576, 512)]


def make_case(seed):
    r = random.Random(seed)
    dim, dim_v = r.choice(DIMS)
    mla = dim == 576
    if mla:
        head_k, head_q = 1, r.choice([1, 8, 16, 64, 128, 128])
    else:
        head_k = r.choice([1, 2, 4, 8])
        head_q = head_k * r.choice([1, 1, 2, 4, 5, 8, 16, 32])
    batch = r.choice([1, 2, 3, 5, 9, 20])
    top = r.choice([1, 40, 130, 700, 1500])
    lens = [r.choice([0, 1, top, r.randint(1, top)]) for _ in range(batch)]
    if sum(lens) == 0:
        lens[0] = top
    return dict(seed=seed, dt=r.choice([torch.float16, torch.bfloat16]), head_q=head_q, head_k=head_k, dim=dim,
                dim_v=dim_v, mla=mla, lens=lens, alibi=r.random() < 0.3, scale=r.choice([None, None, 0.07]),
                splits=r.choice([0, 0, 1, 2, 5]), page=r.choice([0, 0, 16, 32, 64, 128]), pad=r.choice([0, 0, 8, 64]))


@pytest.mark.parametrize("seed", range(int(os.environ.get("DA_FUZZ_SEEDS", "150"))))  # more seeds: DA_FUZZ_SEEDS=1000
def test_random_case(native_lib, oracle, seed):
    c = make_case(seed)
    w = synth.Workload(f"fuzz{seed}", c["dt"], c["head_q"], c["head_k"], c["dim"], c["dim_v"], c["lens"], is_alibi=c["alibi"],
                       dist="normal", scale=0.4, mla=c["mla"], seed=1000 + seed)
    q, k, v, cu = w.make("cpu")
    expect, lse_e = oracle.attn_cpu(q, k, v, cu, dim_v=c["dim_v"], is_alibi=c["alibi"], softmax_scale=c["scale"], return_lse=True)
    batch = len(c["lens"])
    table = None
    if c["page"]:
        k, v, table = to_pages(k, v, cu, c["page"], seed=seed)
        table = table.to(DEV)
    dq, dk, dv = q.to(DEV), k.to(DEV), (v.to(DEV) if v is not None else None)
    if c["pad"] and not c["page"]:  # rows with padding between them: views into wider buffers
        def padded(t):
            if t is None:
                return None
            wide = torch.full((t.shape[0], t.shape[1] * t.shape[2] + c["pad"]), float("nan"), dtype=t.dtype, device=DEV)
            wide[:, :t.shape[1] * t.shape[2]] = t.reshape(t.shape[0], -1)
            return wide[:, :t.shape[1] * t.shape[2]].unflatten(1, (t.shape[1], t.shape[2]))
        dq, dk, dv = padded(dq), padded(dk), padded(dv)
    o = torch.full((batch, c["head_q"], c["dim_v"]), float("nan"), dtype=c["dt"], device=DEV)
    lse = torch.empty(batch, c["head_q"], dtype=torch.float32, device=DEV)
    args = native_lib.make_args(dq, dk, dv, o, cu.to(DEV), max(w.max_seq_k, 1), c["dim_v"], is_alibi=c["alibi"],
                                softmax_scale=c["scale"], lse=lse, num_splits=c["splits"], block_table=table,
                                page_size=c["page"])
    native_lib.decode_fwd(args)
    torch.cuda.synchronize()
    assert native_lib.device_status() == native_lib.DA_OK, c
    assert_close(o, expect, str(c))
    fin = torch.isfinite(lse_e)
    if fin.any():
        assert (lse.cpu()[fin] - lse_e[fin]).abs().max().item() <= 2e-3, c
    assert torch.equal(torch.isinf(lse.cpu()), ~fin), c
