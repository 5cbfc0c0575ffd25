// Host-side declarations shared by the translation units of libdecoding_attn_b200.so.
#pragma once
#include <utility>

#include <cuda_runtime.h>

#include <cstdint>

#include "da_common.cuh"

namespace da {

// Tiling of one kernel variant, reported to the dispatcher for the split heuristic.
struct SplitVariantInfo {
    int tile_keys;    // keys per pipeline stage
    int heads;        // query heads per CTA (G)
    int ctas_per_sm;  // resident CTAs per SM the variant is tuned for
};

// Per-shape launchers (da_split_d*.cu).  `heads` must be one of the values the shape instantiates;
// returns cudaErrorInvalidValue otherwise.  `kvq`: how the cache is stored (0 as q, 1 FP8 e4m3, 2 int8, 3 int4; q and o keep the 16-bit type).
struct KvMaps {
    CUtensorMap k, v;
};
cudaError_t launch_split_d64(bool bf16, int kvq, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s);
cudaError_t launch_split_d96(bool bf16, int kvq, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s);
cudaError_t launch_split_d128(bool bf16, int kvq, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s);
cudaError_t launch_split_d256(bool bf16, int kvq, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s);
cudaError_t launch_split_mla_simt(bool bf16, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s);
SplitVariantInfo split_info_d64(int heads);
SplitVariantInfo split_info_d96(int heads);
SplitVariantInfo split_info_d128(int heads);
SplitVariantInfo split_info_d256(int heads);
SplitVariantInfo split_info_mla_simt(int heads);

// Tensor-core (tcgen05 / TMEM) kernel for up to 128 query heads over one latent KV head, on SM pairs
// (da_mla_2sm_sm100.cu): clusters of two CTAs issue cta_group::2 MMAs, each CTA
// holding 64 of the 128 head rows.  tm_q: box {64, min(64, head_q), 1}; tm_k: box {64, 64 keys or a shorter page};
// both with the 128-byte swizzle.
cudaError_t launch_mla_2sm(bool bf16, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                           cudaStream_t s);
SplitVariantInfo split_info_mla_2sm();
// Tensor-core kernel for head dims 64 / 128 / 256 and groups of up to 128 query heads per KV head (da_gqa_tc_sm100.cu).
cudaError_t launch_gqa_tc(bool bf16, int dim, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                          const CUtensorMap &tm_v, cudaStream_t s);
SplitVariantInfo split_info_gqa_tc();
// Tensor-core kernel for head dims 64 / 128 and groups of at most 32 query heads per KV head: four key streams,
// one per TMEM lane quadrant (da_gqa_quad_sm100.cu).  tm_q: box {64, min(32, head_q), 1}.
cudaError_t launch_gqa_quad(bool bf16, int dim, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                            cudaStream_t s);
SplitVariantInfo split_info_gqa_quad();

// Merge of split / shard partials (da_merge.cu).  cu_seq_k and chunk_keys (both optional) limit a
// row to the splits that cover keys; without them every part is read.
struct MergeParams {
    const float *part_o;
    const float *part_lse;
    void *o;
    float *o_f32;
    float *lse;
    const int *cu_seq_k;
    long long part_stride_o, row_stride_o, part_stride_lse, row_stride_lse;
    long long o_row_stride;  // elements between sequences in o
    long long rows;
    int num_parts, dim_v, head_q, chunk_keys, is_bf16;
};
cudaError_t launch_merge(const MergeParams &p, cudaStream_t s, bool overlap = false);

// Batch indices sorted by descending sequence length into order[batch] (da_order.cu).
cudaError_t launch_order(const int *cu_seq_k, int batch, long long max_len, int *order, cudaStream_t s);

void count_launch(int n = 1);

// Launches `kernel`.  With `overlap` the launch may begin while the preceding kernel of the stream is
// still running (programmatic dependent launch); the kernel then calls pdl_wait() before it reads
// anything that kernel wrote.
template <typename... P, typename... A>
inline cudaError_t launch_kernel(void (*kernel)(P...), dim3 grid, unsigned threads, size_t smem_bytes, cudaStream_t s,
                                 bool overlap, A &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = overlap ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
    return e != cudaSuccess ? e : cudaGetLastError();
}

// Records `msg` as the calling thread's last error (da_last_error) and returns `code`.
int report_error(int code, const char *msg);

}  // namespace da
