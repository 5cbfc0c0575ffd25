"""Host-side logic of the multi-GPU modes, run as two gloo ranks on the CPU: sequence partitioning,
key ranges, record packing and the all-gather.  The per-rank attention is done by the CPU oracle
and the merge by the fp64 checker; on GPUs the same plumbing carries the CUDA kernels' records."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from decoding_attention_b200 import sharded, synth


def test_partition_batch_balances_and_covers():
    lens = synth.seq_lens_uniform(1234, 256, 512, 4096)
    for world in (1, 2, 4, 8):
        parts = sharded.partition_batch(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(256))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.02 * sum(lens) / world + 1


def test_key_ranges_tile_the_sequence():
    for n in (131072, 1000, 63, 1):
        for world in (1, 2, 4, 8):
            rs = [sharded.key_range(n, r, world) for r in range(world)]
            assert rs[0][0] == 0 and rs[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(rs[:-1], rs[1:]))
            assert all(lo % 64 == 0 for lo, hi in rs if hi > lo)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    from helpers import merge_reference
    from oracle import attn_oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # --- key-range sharding of one long sequence, with ALiBi
        w = synth.Workload("long", torch.bfloat16, 8, 8, 128, 128, [1000], is_alibi=True, dist="normal", scale=0.5)
        lo, hi = sharded.key_range(1000, rank, world)
        q, k, v, cu = w.make("cpu", key_range=(lo, hi))
        _, lse, o32 = attn_oracle.attn_cpu(q, k, v, cu, is_alibi=True,
                                           kv_pos_offset=torch.tensor([lo], dtype=torch.int32),
                                           kv_total_len=torch.tensor([1000], dtype=torch.int32),
                                           return_lse=True, return_f32=True)
        rows, dv = 8, 128
        rec = torch.zeros(sharded.record_floats(rows, dv))
        ro, rl = sharded.record_views(rec, rows, dv)
        ro.copy_(o32.view(rows, dv))
        rl.copy_(lse.view(rows))
        got = sharded.gather_records(rec)
        go, gl = sharded.record_views(got, rows, dv)
        o, _ = merge_reference(go, gl)
        qf, kf, vf, cuf = w.make("cpu")
        full = attn_oracle.attn_cpu(qf, kf, vf, cuf, is_alibi=True, return_f32=True)[1]
        err_seq = (o.float() - full.view(rows, dv)).abs().max().item()
        # --- batch sharding: every rank computes its own sequences, results match the whole batch
        w2 = synth.Workload("b", torch.float16, 8, 2, 64, 64, [70, 5, 300, 41, 128], dist="normal")
        mine = sharded.partition_batch(w2.seq_lens, world)[rank]
        q2, k2, v2, cu2 = w2.make("cpu", seqs=mine)
        o2 = attn_oracle.attn_cpu(q2, k2, v2, cu2)
        whole = attn_oracle.attn_cpu(*w2.make("cpu"))
        same = all(torch.equal(o2[j].view(torch.int16), whole[b].view(torch.int16)) for j, b in enumerate(mine))
        ret[rank] = (err_seq, same, len(mine))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding():
    world = 2
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        err_seq, same, n = ret[r]
        assert err_seq < 1e-5, err_seq
        assert same and n >= 1
