// C++ entry point with the signature of the reference's host API
// (Bruce-Lee-LY/decoding_attention, csrc/ops/decoding_attn.h:29-30), implemented on top of the C ABI
// in decoding_attn_b200.h.  A call site of the reference compiles against this header unchanged.
#pragma once

#include <cstddef>

#include "cuda_runtime_api.h"

/**
 * Decode attention (one query token per sequence) for MHA / MQA / GQA / MLA.
 *
 * q        device [total_q = batch, head_q, dim]
 * k        device [total_k, head_k, dim]; the latent-KV cache for MLA
 * v        device [total_k, head_k, dim_v]; nullptr for MLA (V = first dim_v elements of each K row)
 * o        device [total_q, head_q, dim_v]
 * cu_seq_k device int32 [batch + 1]
 * max_seq_k upper bound of the sequence lengths (a scheduling hint here, not a shared-memory size)
 * softmax scale is 1/sqrt(dim) as in the reference (csrc/ops/decoding_attn.cpp:54)
 *
 * Errors: like the reference (csrc/common/common.h:17-23) a failed check logs to stderr and calls
 * exit(EXIT_FAILURE); unlike it, an unsupported (dim, dim_v) pair is such an error instead of a
 * silent no-op (csrc/common/common.h:73-96).
 */
void decoding_attn(void *q, void *k, void *v, void *o, int *cu_seq_k, size_t max_seq_k, size_t batch, size_t head_q,
                   size_t head_k, size_t dim, size_t dim_v, bool is_alibi, bool is_bf16, cudaStream_t stream);
