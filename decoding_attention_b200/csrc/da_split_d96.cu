// Instantiations of the CUDA-core split-KV kernel for head dims (96, 96).  These replace the
// reference's per-shape tiling choices (csrc/kernel/decoding_attn/decoding_fwd_hd*.cu).
#include "da_internal.h"
#include "da_split_kernel.cuh"

namespace da {
namespace {
// lanes per key row, keys per lane-group and tile, consumer warps, pipeline stages
template <typename T, int G, int KPT, int KVQ = 0>
using Cfg = SplitCfg<T, 96, 96, 4, G, KPT, 4, 3, false, 1, KVQ>;

template <typename T, int KVQ>
cudaError_t launch_t(int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s) {
    switch (heads) {
        case 1: return launch_split<Cfg<T, 1, 2, KVQ>>(p, m.k, m.v, s);
        case 2: return launch_split<Cfg<T, 2, 2, KVQ>>(p, m.k, m.v, s);
        case 4: return launch_split<Cfg<T, 4, 2, KVQ>>(p, m.k, m.v, s);
        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

// kvq: how K and V are stored (0 as q, 1 FP8 e4m3, 2 int8, 3 int4); q and o stay 16-bit
cudaError_t launch_split_d96(bool bf16, int kvq, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s) {
    switch (kvq) {
        case 1: return bf16 ? launch_t<__nv_bfloat16, 1>(heads, p, m, s) : launch_t<__half, 1>(heads, p, m, s);
        case 2: return bf16 ? launch_t<__nv_bfloat16, 2>(heads, p, m, s) : launch_t<__half, 2>(heads, p, m, s);
        case 3: return bf16 ? launch_t<__nv_bfloat16, 3>(heads, p, m, s) : launch_t<__half, 3>(heads, p, m, s);
        default: return bf16 ? launch_t<__nv_bfloat16, 0>(heads, p, m, s) : launch_t<__half, 0>(heads, p, m, s);
    }
}

SplitVariantInfo split_info_d96(int heads) {
    switch (heads) {
        case 1: return {Cfg<__half, 1, 2>::TILE, 1, (227 * 1024) / (Cfg<__half, 1, 2>::SMEM_BYTES + 1024)};
        case 2: return {Cfg<__half, 2, 2>::TILE, 2, (227 * 1024) / (Cfg<__half, 2, 2>::SMEM_BYTES + 1024)};
        case 4: return {Cfg<__half, 4, 2>::TILE, 4, (227 * 1024) / (Cfg<__half, 4, 2>::SMEM_BYTES + 1024)};
        default: return {0, 0, 0};
    }
}
}  // namespace da
