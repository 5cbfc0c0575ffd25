"""Key-range sharding on GPUs: the decoder object on one GPU (world 1), and -- where the box has two
GPUs -- two NCCL ranks each holding half of a long sequence, checked against the CPU oracle."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from decoding_attention_b200 import sharded, synth
from helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True])
def test_key_range_decoder_single_rank(native_lib, oracle, fused):
    dev = "cuda:0"
    w = synth.Workload("long1", torch.bfloat16, 32, 32, 128, 128, [9000], is_alibi=True, dist="normal", scale=0.5)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu, is_alibi=True)
    dec = sharded.KeyRangeShardedDecoder(1, 32, 128, w.dtype, dev, fused=fused)
    for _ in range(3):  # several steps: the exchange buffers are double-buffered by step parity
        out = dec.step(q.to(dev), k.to(dev), v.to(dev), cu.to(dev), 9000, is_alibi=True)
    torch.cuda.synchronize()
    assert native_lib.device_status() == native_lib.DA_OK
    assert_close(out, expect, "world-1 key-range decoder")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret, fused=False):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        w = synth.Workload("long2", torch.bfloat16, 32, 32, 128, 128, [20000], is_alibi=True, dist="normal", scale=0.5)
        lo, hi = sharded.key_range(20000, rank, world)
        q, k, v, cu = w.make(dev, key_range=(lo, hi))
        dec = sharded.KeyRangeShardedDecoder(1, 32, 128, w.dtype, dev, fused=fused)
        off = torch.tensor([lo], dtype=torch.int32, device=dev)
        tot = torch.tensor([20000], dtype=torch.int32, device=dev)
        for _ in range(4):
            out = dec.step(q, k, v, cu, hi - lo, is_alibi=True, kv_pos_offset=off, kv_total_len=tot)
        torch.cuda.synchronize()
        from decoding_attention_b200 import cabi
        assert cabi.device_status() == cabi.DA_OK
        ret[rank] = out.cpu()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fused", [False, True])
def test_key_range_decoder_two_ranks(oracle, fused):
    world = 2
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret, fused), nprocs=world, join=True)
    w = synth.Workload("long2", torch.bfloat16, 32, 32, 128, 128, [20000], is_alibi=True, dist="normal", scale=0.5)
    q, k, v, cu = w.make("cpu")
    expect = oracle.attn_cpu(q, k, v, cu, is_alibi=True)
    for r in range(world):
        assert_close(ret[r], expect, f"rank {r}")
    assert torch.equal(ret[0], ret[1])
