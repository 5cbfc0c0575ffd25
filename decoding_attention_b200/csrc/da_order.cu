// Longest-first launch order for batches whose sequences differ in length.
//
// The grid of the attention kernels is (key-range splits, KV heads, batch) and CTAs are handed out
// in that order, so the last CTAs to start belong to the last sequences of the batch.  When those
// happen to be long, the GPU drains with a few SMs busy: on 256 sequences of 512..4096 keys that
// tail costs ~8 % of the call.  Only the device knows the lengths (cu_seq_k), so a one-block kernel
// sorts the batch indices by descending length (counting sort over 1024 length buckets) and the
// attention kernels take sequence order[blockIdx.z] instead of blockIdx.z.  The order inside a bucket
// is arbitrary; results do not depend on it.  The reference launches one CTA per (sequence, head) in
// batch order and has no such step (decoding_fwd_launch_template.h:20-27).
#include "da_internal.h"

namespace da {
namespace {

constexpr int kBuckets = 1024;

__global__ void __launch_bounds__(kBuckets) da_order_kernel(const int *__restrict__ cu_seq_k, int batch, long long max_len,
                                                            int *__restrict__ order) {
    __shared__ int count[kBuckets];  // count[k]: sequences in bucket k; bucket 0 holds the longest
    __shared__ int start[kBuckets];
    pdl_launch_dependents();  // the attention kernel may be scheduled now; it waits for this grid before reading `order`
    const int tid = threadIdx.x;
    count[tid] = 0;
    __syncthreads();
    auto bucket = [&](int i) {
        const long long len = cu_seq_k[i + 1] - cu_seq_k[i];
        long long k = len * kBuckets / (max_len + 1);
        k = k < 0 ? 0 : (k > kBuckets - 1 ? kBuckets - 1 : k);
        return kBuckets - 1 - (int)k;
    };
    for (int i = tid; i < batch; i += kBuckets) atomicAdd(&count[bucket(i)], 1);
    __syncthreads();
    // exclusive prefix sum over the buckets: warp scans, then a scan of the 32 warp totals
    __shared__ int warp_total[32];
    const int lane = tid & 31, warp = tid >> 5;
    const int own = count[tid];
    int v = own;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
    }
    if (lane == 31) warp_total[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = warp_total[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, t, d);
            if (lane >= d) t += n;
        }
        warp_total[lane] = t;
    }
    __syncthreads();
    start[tid] = v - own + (warp > 0 ? warp_total[warp - 1] : 0);
    __syncthreads();
    for (int i = tid; i < batch; i += kBuckets) order[atomicAdd(&start[bucket(i)], 1)] = i;
}

}  // namespace

cudaError_t launch_order(const int *cu_seq_k, int batch, long long max_len, int *order, cudaStream_t s) {
    da_order_kernel<<<1, kBuckets, 0, s>>>(cu_seq_k, batch, max_len < 1 ? 1 : max_len, order);
    count_launch();
    return cudaGetLastError();
}

}  // namespace da
