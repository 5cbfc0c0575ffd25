"""Seeded synthetic decode-attention workloads.

The reference draws its test and benchmark inputs from unseeded generators
(csrc/common/tensor.h:31-36, tests/test_decoding_attn.py:73-78), so there are no fixed inputs to
reuse.  Here every element is a pure function of (seed, tensor id, element index) -- a splitmix64
style hash evaluated with torch integer ops -- so the same values can be produced on the CPU (for
the oracle), on one GPU, or shard by shard on several GPUs, without moving data between them.
"""
import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

_M64 = (1 << 64) - 1


def _s64(x):
    """Two's-complement int64 value of an unsigned 64-bit constant."""
    x &= _M64
    return x - (1 << 64) if x >= (1 << 63) else x


_GOLDEN = _s64(0x9E3779B97F4A7C15)
_MUL1 = _s64(0xBF58476D1CE4E5B9)
_MUL2 = _s64(0x94D049BB133111EB)


def _lsr(z, n):
    return (z >> n) & ((1 << (64 - n)) - 1)


def _hash64(idx, key):
    """splitmix64 finaliser of (idx + key * golden), int64 tensors with wrap-around arithmetic."""
    z = idx + key
    z = (z ^ _lsr(z, 30)) * _MUL1
    z = (z ^ _lsr(z, 27)) * _MUL2
    return z ^ _lsr(z, 31)


def _key(seed, tensor_id):
    k = (seed * 0x9E3779B97F4A7C15 + tensor_id * 0xD1B54A32D192ED03 + 0x2545F4914F6CDD1D) & _M64
    return _s64(k)


def fill(kind: str, seed: int, tensor_id: int, idx: torch.Tensor, dtype, scale: float = 1.0) -> torch.Tensor:
    """Values for element indices ``idx`` (int64 tensor): ``uniform`` in [-1, 1) * scale or
    ``normal`` N(0, 1) * scale (Box-Muller), rounded once to ``dtype``."""
    z = _hash64(idx, _key(seed, tensor_id))
    a = _lsr(z, 40).to(torch.float32)  # 24 bits
    if kind == "uniform":
        x = a * (2.0 ** -23) - 1.0
    elif kind == "normal":
        b = (_lsr(z, 16) & 0xFFFFFF).to(torch.float32)
        u1 = (a + 1.0) * (2.0 ** -24)
        x = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi * 2.0 ** -24) * b)
    else:
        raise ValueError(kind)
    if scale != 1.0:
        x = x * scale
    return x.to(dtype)


def fill_range(kind, seed, tensor_id, start, count, dtype, device, scale=1.0, chunk=1 << 25):
    """Elements [start, start + count) of a tensor, generated chunk by chunk to bound temporaries."""
    out = torch.empty(count, dtype=dtype, device=device)
    for c0 in range(0, count, chunk):
        n = min(chunk, count - c0)
        idx = torch.arange(start + c0, start + c0 + n, dtype=torch.int64, device=device)
        out[c0:c0 + n] = fill(kind, seed, tensor_id, idx, dtype, scale)
    return out


def seq_lens_uniform(seed: int, batch: int, lo: int, hi: int) -> List[int]:
    """``batch`` lengths uniform in [lo, hi] from the seed (host side, exact integer arithmetic)."""
    idx = torch.arange(batch, dtype=torch.int64)
    z = _lsr(_hash64(idx, _key(seed, 99)), 11)  # 53 bits
    return [int(lo + (int(v) % (hi - lo + 1))) for v in z.tolist()]


@dataclass
class Workload:
    """One decode-attention problem: shapes, lengths and value distributions."""
    name: str
    dtype: torch.dtype
    head_q: int
    head_k: int
    dim: int
    dim_v: int
    seq_lens: List[int]
    is_alibi: bool = False
    dist: str = "uniform"
    scale: float = 1.0
    mla: bool = False  # no V tensor: V = first dim_v elements of each K row
    seed: int = 1234
    softmax_scale: Optional[float] = None
    _cu: Optional[List[int]] = field(default=None, repr=False)

    @property
    def batch(self):
        return len(self.seq_lens)

    @property
    def cu(self):
        if self._cu is None:
            cu = [0]
            for n in self.seq_lens:
                cu.append(cu[-1] + n)
            self._cu = cu
        return self._cu

    @property
    def total_k(self):
        return self.cu[-1]

    @property
    def max_seq_k(self):
        return max(self.seq_lens) if self.seq_lens else 0

    def kv_bytes(self, seq_lens=None):
        """Algorithmic KV bytes of one call: every K and V element read once (MLA: one latent row)."""
        n = sum(self.seq_lens if seq_lens is None else seq_lens)
        per_tok = self.head_k * (self.dim if self.mla else self.dim + self.dim_v) * 2
        return n * per_tok

    def ref_flops(self):
        """The reference's flop count (csrc/common/tester.h:270)."""
        return sum(self.seq_lens) * self.head_q * (self.dim + self.dim_v) * 2

    def ref_bytes(self):
        """The reference's byte count, Q + K + O without V (csrc/common/tester.h:273-276)."""
        return (self.batch * self.head_q * self.dim + self.total_k * self.head_k * self.dim +
                self.batch * self.head_q * self.dim_v) * 2

    # ---- tensors -------------------------------------------------------------------------
    def make_q(self, device, seqs=None):
        row = self.head_q * self.dim
        if seqs is None:
            q = fill_range(self.dist, self.seed, 0, 0, self.batch * row, self.dtype, device, self.scale)
        else:
            q = torch.cat([fill_range(self.dist, self.seed, 0, b * row, row, self.dtype, device, self.scale)
                           for b in seqs])
        return q.view(-1, self.head_q, self.dim)

    def _make_kv(self, tensor_id, width, device, token_ranges):
        row = self.head_k * width
        parts = [fill_range(self.dist, self.seed, tensor_id, t0 * row, (t1 - t0) * row, self.dtype, device,
                            self.scale) for (t0, t1) in token_ranges]
        out = parts[0] if len(parts) == 1 else torch.cat(parts)
        return out.view(-1, self.head_k, width)

    def make(self, device, seqs=None, key_range=None):
        """(q, k, v, cu_seq_k) on ``device``.

        ``seqs``: subset of sequence indices (batch sharding) -- K/V rows of those sequences only,
        packed in that order, with a rebased cu_seq_k.  ``key_range`` = (lo, hi): keys [lo, hi) of
        every sequence (key-range sharding of long sequences).  v is None for the MLA shape.
        """
        seq_ids = list(range(self.batch)) if seqs is None else list(seqs)
        cu = self.cu
        ranges, lens = [], []
        for b in seq_ids:
            lo, hi = cu[b], cu[b + 1]
            if key_range is not None:
                lo, hi = min(cu[b] + key_range[0], cu[b + 1]), min(cu[b] + key_range[1], cu[b + 1])
            ranges.append((lo, hi))
            lens.append(hi - lo)
        merged = []
        for r in ranges:  # coalesce adjacent token ranges so that generation stays in big chunks
            if merged and merged[-1][1] == r[0]:
                merged[-1] = (merged[-1][0], r[1])
            else:
                merged.append(r)
        q = self.make_q(device, None if seqs is None else seq_ids)
        k = self._make_kv(1, self.dim, device, merged)
        v = None if self.mla else self._make_kv(2, self.dim_v, device, merged)
        cu_local = [0]
        for n in lens:
            cu_local.append(cu_local[-1] + n)
        cu_seq_k = torch.tensor(cu_local, dtype=torch.int32, device=device)
        return q, k, v, cu_seq_k


# ---- the benchmark configurations ----------------------------------------------------------

def config_mha_small(seed=1234):
    """MHA fp16, batch 4, 32/32 heads, dim 128, seq_k 1024 each, uniform[-1, 1]."""
    return Workload("mha_fp16_b4_sk1024", torch.float16, 32, 32, 128, 128, [1024] * 4, dist="uniform", seed=seed)


def config_gqa_varlen(seed=1234, batch=256, lo=512, hi=4096):
    """GQA bf16, batch 256, 32/8 heads, dim 128, seq_k uniform in [512, 4096], N(0, 1) * 0.5."""
    return Workload(f"gqa_bf16_b{batch}_sk{lo}-{hi}", torch.bfloat16, 32, 8, 128, 128,
                    seq_lens_uniform(seed, batch, lo, hi), dist="normal", scale=0.5, seed=seed)


def config_mqa_alibi(seed=1234, batch=128, seq_k=2048):
    """MQA fp16 with ALiBi, batch 128, 32/1 heads, dim 128, seq_k 2048, uniform[-1, 1]."""
    return Workload(f"mqa_alibi_fp16_b{batch}_sk{seq_k}", torch.float16, 32, 1, 128, 128, [seq_k] * batch,
                    is_alibi=True, dist="uniform", seed=seed)


def config_mla(seed=1234, batch=128, seq_k=4096, head_q=128):
    """MLA bf16: 128 query heads over one 576-dim latent KV head (V = first 512 dims), N(0, 1) * 0.3."""
    return Workload(f"mla_bf16_b{batch}_sk{seq_k}", torch.bfloat16, head_q, 1, 576, 512, [seq_k] * batch,
                    dist="normal", scale=0.3, mla=True, seed=seed)


def config_long_mha(seed=1234, seq_k=131072):
    """MHA bf16, batch 1, 32/32 heads, dim 128, one sequence of 131072 keys, N(0, 1) * 0.5."""
    return Workload(f"mha_bf16_b1_sk{seq_k}", torch.bfloat16, 32, 32, 128, 128, [seq_k], dist="normal", scale=0.5,
                    seed=seed)


CONFIGS = {
    "mha_small": config_mha_small,
    "gqa_varlen": config_gqa_varlen,
    "mqa_alibi": config_mqa_alibi,
    "mla": config_mla,
    "long_mha": config_long_mha,
}
