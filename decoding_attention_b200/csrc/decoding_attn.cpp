// decoding_attn(): the reference's C++ host entry point (csrc/ops/decoding_attn.cpp:70-76) as a
// thin shim over the C ABI.  The reference builds DecodingParams and dispatches on dtype and head
// dim here; both now happen behind da_decode_fwd().
#include "../../include/decoding_attn.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../include/decoding_attn_b200.h"

void decoding_attn(void *q, void *k, void *v, void *o, int *cu_seq_k, size_t max_seq_k, size_t batch, size_t head_q,
                   size_t head_k, size_t dim, size_t dim_v, bool is_alibi, bool is_bf16, cudaStream_t stream) {
    da_decode_args_t a;
    std::memset(&a, 0, sizeof(a));
    a.struct_size = sizeof(a);
    a.is_bf16 = is_bf16;
    a.is_alibi = is_alibi;
    a.q = q;
    a.k = k;
    a.v = v;
    a.o = o;
    a.cu_seq_k = cu_seq_k;
    a.max_seq_k = (int64_t)max_seq_k;
    a.batch = (int64_t)batch;
    a.head_q = (int64_t)head_q;
    a.head_k = (int64_t)head_k;
    a.dim = (int64_t)dim;
    a.dim_v = (int64_t)dim_v;
    a.stream = stream;
    const int rc = da_decode_fwd(&a);
    if (rc != DA_OK) {
        // Same contract as DA_CHECK (csrc/common/common.h:17-23): log and terminate.
        std::fprintf(stderr, "[decoding_attn] %s: %s\n", da_status_string(rc), da_last_error());
        std::exit(EXIT_FAILURE);
    }
}
