// LSE merge of partial attention results (sm_100a).
//
// Partials are normalised fp32 rows o_r with their natural-log LSE lse_r over disjoint key ranges.
// The merged row is sum_r w_r o_r / sum_r w_r with w_r = exp(lse_r - max lse).  Used (a) after the
// split-KV kernels of one GPU and (b) after the per-GPU records of a key-range-sharded sequence
// have been gathered.  The reference never splits a row, so it has no such step; the identity
// is the one its softmax (csrc/common/tester.h:206-219) satisfies over a partition of the keys.
#include "da_internal.h"

namespace da {

template <typename T>
__global__ void __launch_bounds__(128) da_merge_kernel(const MergeParams p) {
    pdl_launch_dependents();  // a successor launched for overlap (the exchange kernel) may be scheduled early
    const int tpr = p.dim_v / 4;  // threads per row, one float4 each
    const int rpb = 128 / tpr;    // rows per block
    const int r_in_blk = threadIdx.x / tpr;
    const int t = threadIdx.x % tpr;
    if (r_in_blk >= rpb) return;
    const long long row = (long long)blockIdx.x * rpb + r_in_blk;
    if (row >= p.rows) return;
    const int b = (int)(row / p.head_q), h = (int)(row % p.head_q);

    int n = p.num_parts;
    if (p.cu_seq_k) {
        const int len = p.cu_seq_k[b + 1] - p.cu_seq_k[b];
        n = min(n, (len + p.chunk_keys - 1) / p.chunk_keys);
    }
    pdl_wait();  // the partials come from the kernel launched just before this one
    const float *lse_row = p.part_lse + row * p.row_stride_lse;
    const float *o_row = p.part_o + row * p.row_stride_o + t * 4;

    float mx = -INFINITY;
    for (int r = 0; r < n; ++r) mx = fmaxf(mx, lse_row[r * p.part_stride_lse]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    if (mx > -INFINITY) {
        for (int r = 0; r < n; ++r) {
            const float w = exp2f((lse_row[r * p.part_stride_lse] - mx) * kLog2e);
            const float4 x = *reinterpret_cast<const float4 *>(o_row + r * p.part_stride_o);
            acc.x = fmaf(w, x.x, acc.x);
            acc.y = fmaf(w, x.y, acc.y);
            acc.z = fmaf(w, x.z, acc.z);
            acc.w = fmaf(w, x.w, acc.w);
            wsum += w;
        }
        const float inv = 1.0f / wsum;
        acc.x *= inv, acc.y *= inv, acc.z *= inv, acc.w *= inv;
    }
    if (p.o) {
        T *dst = reinterpret_cast<T *>(p.o) + (size_t)b * p.o_row_stride + (size_t)h * p.dim_v + t * 4;
        dst[0] = from_float<T>(acc.x);
        dst[1] = from_float<T>(acc.y);
        dst[2] = from_float<T>(acc.z);
        dst[3] = from_float<T>(acc.w);
    }
    if (p.o_f32) *reinterpret_cast<float4 *>(p.o_f32 + row * p.dim_v + t * 4) = acc;
    if (p.lse && t == 0) p.lse[row] = (mx > -INFINITY) ? mx + log2f(wsum) * kLn2 : -INFINITY;
}

// `overlap`: the launch may begin while the preceding kernel of the stream is still running (programmatic
// dependent launch); the kernel waits for that kernel's results itself.
cudaError_t launch_merge(const MergeParams &p, cudaStream_t s, bool overlap) {
    if (p.dim_v % 4 != 0 || p.dim_v > 512 || p.dim_v <= 0) return cudaErrorInvalidValue;
    if (p.rows <= 0) return cudaSuccess;
    const int rpb = 128 / (p.dim_v / 4);
    const long long blocks = (p.rows + rpb - 1) / rpb;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(128);
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = overlap ? 1 : 0;
    cudaError_t e = p.is_bf16 ? cudaLaunchKernelEx(&cfg, da_merge_kernel<__nv_bfloat16>, p)
                              : cudaLaunchKernelEx(&cfg, da_merge_kernel<__half>, p);
    count_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace da
