"""Python call surface: the reference's ``decoding_attn_fwd``
(decoding_attn/decoding_attn_interface.py:24-53) plus the two named entry points ``dmha_fwd`` /
``dmla_fwd`` with an explicit softmax scale.  Everything goes through the torch extension
``decoding_attn_cuda`` (csrc/torch_binding.cpp), i.e. the C++ binding over the C ABI.
"""
import os
import sys

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
if _PKG not in sys.path:
    sys.path.insert(0, _PKG)
try:
    import decoding_attn_cuda  # noqa: E402  (built in-tree by decoding_attention_b200.build)
except ImportError as e:  # no fallback: fail loudly
    raise ImportError("the decoding_attn_cuda extension is not built: run "
                      "`python -m decoding_attention_b200.build`") from e


def maybe_contiguous(x):
    return x.contiguous() if x is not None and x.stride(-1) != 1 else x


def decoding_attn_fwd(q, k, v, cu_seq_k, max_seq_k, dim_v, is_alibi, *, softmax_scale=None):
    """Same arguments and result as the reference's ``decoding_attn_fwd``.

    q [total_q, head_q, dim]; k [total_k, head_k, dim] (MLA: the latent KV cache); v [total_k, head_k,
    dim_v] or None for MLA; cu_seq_k int32 [batch + 1]; returns o [total_q, head_q, dim_v].
    ``softmax_scale`` (keyword-only, an extension) defaults to the reference's 1/sqrt(dim).
    """
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    if softmax_scale is None:
        return decoding_attn_cuda.fwd(q, k, v, None, cu_seq_k, max_seq_k, dim_v, is_alibi)
    if v is None:
        return decoding_attn_cuda.dmla_fwd(q, k, cu_seq_k, max_seq_k, dim_v, is_alibi, softmax_scale)
    return decoding_attn_cuda.dmha_fwd(q, k, v, cu_seq_k, max_seq_k, is_alibi, softmax_scale)


def dmha_fwd(q, k, v, cu_seq_k, max_seq_k, is_alibi=False, softmax_scale=None, out=None, return_lse=False,
             k_scale=1.0, v_scale=1.0):
    """MHA / GQA / MQA decode attention; ``return_lse`` adds the fp32 natural-log LSE [batch, head_q].
    ``k`` / ``v`` may be an FP8 cache (torch.float8_e4m3fn) standing for ``k * k_scale`` / ``v * v_scale``."""
    q, k, v = [maybe_contiguous(x) for x in (q, k, v)]
    return decoding_attn_cuda.dmha_fwd(q, k, v, cu_seq_k, max_seq_k, is_alibi, softmax_scale, out, return_lse,
                                       k_scale, v_scale)


def dmla_fwd(q, kv, cu_seq_k, max_seq_k, dim_v=512, softmax_scale=None, out=None, return_lse=False, is_alibi=False):
    """MLA decode attention over the latent KV cache ``kv`` [total_k, 1, 576]; V = kv[..., :dim_v]."""
    q, kv = [maybe_contiguous(x) for x in (q, kv)]
    return decoding_attn_cuda.dmla_fwd(q, kv, cu_seq_k, max_seq_k, dim_v, is_alibi, softmax_scale, out, return_lse)


def paged_fwd(q, k_cache, v_cache, seq_lens, block_table, max_seq_k=None, dim_v=None, is_alibi=False, softmax_scale=None,
              out=None, return_lse=False):
    """Decode attention over a paged KV cache (the layout serving engines keep).

    q [batch, head_q, dim]; k_cache [num_pages, page_size, head_k, dim]; v_cache the same with dim_v, or
    None for the latent-KV (MLA) shape; seq_lens int32 [batch]; block_table int32 [batch, blocks]: key j
    of sequence b is row ``j % page_size`` of page ``block_table[b, j // page_size]``.  page_size must be a
    power of two >= 16.  The reference has no paged entry point; its Python benchmark builds such
    layouts for the libraries it compares against (benchmarks/python/benchmark_decoding_attn.py:182-190).
    """
    cu_seq_k = torch.zeros(seq_lens.numel() + 1, dtype=torch.int32, device=seq_lens.device)
    cu_seq_k[1:] = torch.cumsum(seq_lens, 0)
    if max_seq_k is None:
        max_seq_k = block_table.shape[1] * k_cache.shape[1]
    if dim_v is None:
        dim_v = v_cache.shape[-1] if v_cache is not None else 512
    return decoding_attn_cuda.paged_fwd(q, k_cache, v_cache, cu_seq_k, block_table, max_seq_k, dim_v, is_alibi,
                                        softmax_scale, out, return_lse)


def merge_partials(part_o, part_lse, out_dtype):
    """LSE merge of partial results over disjoint key ranges: part_o fp32 [parts, ..., dim_v]."""
    return decoding_attn_cuda.merge_partials(part_o.contiguous(), part_lse.contiguous(), out_dtype)
