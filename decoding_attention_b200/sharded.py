"""Multi-GPU use of the decode-attention library: one process per GPU, torch.distributed for the
plumbing.  The reference is single-GPU (its only device handling is cudaSetDevice(gpu_rank),
benchmarks/cpp/benchmark_decoding_attn.cpp:27, :43), so both modes below are additions:

* batch sharding -- sequences are independent, so a batch is cut into per-rank groups of
  sequences with balanced key counts and every rank runs the ordinary kernel on its own packed
  K/V.  No collective on the data path.
* key-range sharding -- one long sequence's KV cache lives in contiguous key ranges, one per rank.
  Every rank computes a partial (o fp32, lse) over its range, the fixed-size records are
  all-gathered (NCCL over NVLink; tiny, latency-bound) and every rank merges them on its device
  with da_merge_partials -- or, with ``fused=True``, one kernel per rank pushes its record to the
  peers' symmetric buffers with peer stores, waits (bounded) for theirs and merges
  (da_exchange_merge): no collective call, one launch instead of three.
"""
import ctypes
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_batch(seq_lens: Sequence[int], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of sequences to ``world`` ranks balancing total keys.
    Deterministic; every rank's list is sorted by sequence index."""
    order = sorted(range(len(seq_lens)), key=lambda i: (-seq_lens[i], i))
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        out[r].append(i)
        loads[r] += seq_lens[i]
    return [sorted(x) for x in out]


def key_range(seq_len: int, rank: int, world: int, align: int = 64) -> Tuple[int, int]:
    """Contiguous key range of ``rank``: equal shares rounded up to ``align`` keys (the kernels'
    tile), the last ranks possibly shorter or empty."""
    share = -(-seq_len // world)
    share = -(-share // align) * align
    lo = min(rank * share, seq_len)
    return lo, min(lo + share, seq_len)


def record_floats(rows: int, dim_v: int) -> int:
    """Length of one rank's record: rows*dim_v floats of o, then rows floats of lse, padded to 4."""
    return -(-(rows * (dim_v + 1)) // 4) * 4


def record_views(rec: torch.Tensor, rows: int, dim_v: int):
    """(o view [rows, dim_v], lse view [rows]) into a record buffer (or into each of a stack)."""
    o = rec[..., :rows * dim_v].unflatten(-1, (rows, dim_v))
    lse = rec[..., rows * dim_v:rows * dim_v + rows]
    return o, lse


def gather_records(rec: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather equal-size records: [n] -> [world, n].  Works on CUDA (NCCL) and CPU (gloo)."""
    world = dist.get_world_size(group)
    out = torch.empty(world, rec.numel(), dtype=rec.dtype, device=rec.device)
    if rec.is_cuda:
        dist.all_gather_into_tensor(out, rec, group=group)
    else:
        dist.all_gather(list(out.unbind(0)), rec, group=group)
    return out


class KeyRangeShardedDecoder:
    """Decode attention for sequences whose KV cache is sharded by key range over the ranks of a
    process group.  Construct once per (batch, head_q, dim_v); ``step`` is then allocation-free."""

    def __init__(self, batch, head_q, dim_v, out_dtype, device, group=None, fused=False):
        from . import cabi
        self.cabi = cabi
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.fused = fused
        self.epoch = 0
        self._args = {}
        self.rows, self.dim_v, self.head_q, self.batch = batch * head_q, dim_v, head_q, batch
        n = record_floats(self.rows, dim_v)
        self.rec = torch.zeros(n, dtype=torch.float32, device=device)
        self.gathered = torch.zeros(self.world, n, dtype=torch.float32, device=device)
        self.out = torch.empty(batch, head_q, dim_v, dtype=out_dtype, device=device)
        self.lse = torch.empty(batch, head_q, dtype=torch.float32, device=device)
        self.rec_o, self.rec_lse = record_views(self.rec, self.rows, dim_v)
        if fused:
            self._setup_exchange(device)

    def _setup_exchange(self, device):
        """Symmetric gather buffer (one per rank, each mapped into every peer) for da_exchange_merge."""
        nbytes = self.cabi.lib().da_exchange_buffer_bytes(self.world, self.rows, self.dim_v)
        if self.world == 1:
            self.xbuf = torch.zeros(nbytes // 4, dtype=torch.float32, device=device)
            ptrs = [self.xbuf.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm_mem
            pg = self.group if self.group is not None else dist.group.WORLD
            try:
                symm_mem.enable_symm_mem_for_group(pg.group_name)
            except Exception:
                pass  # newer torch enables groups on demand
            self.xbuf = symm_mem.empty(nbytes // 4, dtype=torch.float32, device=device)
            self.xbuf.zero_()
            self._hdl = symm_mem.rendezvous(self.xbuf, pg.group_name)
            ptrs = [int(x) for x in self._hdl.buffer_ptrs]
            torch.cuda.synchronize()
            dist.barrier(group=self.group)  # every rank's flags are zero before anybody pushes
        self.peer_ptrs = (ctypes.c_void_p * self.world)(*ptrs)

    def local_partial(self, q, k, v, cu_seq_k, max_seq_k, is_alibi, kv_pos_offset, kv_total_len, softmax_scale=None):
        stream = torch.cuda.current_stream().cuda_stream
        key = (q.data_ptr(), k.data_ptr(), v.data_ptr() if v is not None else 0, cu_seq_k.data_ptr(), max_seq_k, is_alibi,
               kv_pos_offset.data_ptr() if kv_pos_offset is not None else 0,
               kv_total_len.data_ptr() if kv_total_len is not None else 0, softmax_scale, stream,
               tuple(q.shape), tuple(k.shape), q.stride(0), k.stride(0))
        a = self._args.get(key)
        if a is None:  # a decode loop calls with the same buffers every step: fill the argument block once
            a = self.cabi.make_args(q, k, v, None, cu_seq_k, max_seq_k, self.dim_v, is_alibi=is_alibi,
                                    softmax_scale=softmax_scale, lse=self.rec_lse, o_f32=self.rec_o,
                                    kv_pos_offset=kv_pos_offset, kv_total_len=kv_total_len, stream=stream)
            if len(self._args) > 64:
                self._args.clear()
            self._args[key] = a
        self.cabi.decode_fwd(a)

    def exchange(self):
        if self.world == 1:
            self.gathered[0].copy_(self.rec)
        else:
            dist.all_gather_into_tensor(self.gathered, self.rec, group=self.group)

    def merge(self):
        n = self.rec.numel()
        lse_base = self.gathered.data_ptr() + self.rows * self.dim_v * 4
        self.cabi.check(self.cabi.lib().da_merge_partials(
            self.gathered.data_ptr(), lse_base, self.world, self.rows, self.dim_v, n, self.dim_v, n, 1,
            self.out.data_ptr(), None, self.lse.data_ptr(), int(self.out.dtype == torch.bfloat16),
            torch.cuda.current_stream().cuda_stream))
        return self.out

    def step(self, q, k, v, cu_seq_k, max_seq_k, is_alibi=False, kv_pos_offset=None, kv_total_len=None,
             softmax_scale=None):
        """q replicated; k, v this rank's key range; returns the full result on every rank."""
        self.local_partial(q, k, v, cu_seq_k, max_seq_k, is_alibi, kv_pos_offset, kv_total_len, softmax_scale)
        if self.fused:
            return self.exchange_merge()
        self.exchange()
        return self.merge()

    def exchange_merge(self):
        # 1, 2, ..., 2^32 - 2, 1, ...: never 0 (the flags' initial value) and alternating parity across the wrap
        self.epoch = self.epoch % 0xFFFFFFFE + 1
        self.cabi.check(self.cabi.lib().da_exchange_merge(
            self.rec.data_ptr(), self.peer_ptrs, self.world, self.rank, self.rows, self.dim_v, self.epoch,
            self.out.data_ptr(), self.lse.data_ptr(), int(self.out.dtype == torch.bfloat16),
            torch.cuda.current_stream().cuda_stream))
        return self.out
