// Instantiations of the CUDA-core split-KV kernel for head dims (576, 512).  These replace the
// reference's per-shape tiling choices (csrc/kernel/decoding_attn/decoding_fwd_hd*.cu).
#include "da_internal.h"
#include "da_split_kernel.cuh"

namespace da {
namespace {
// lanes per key row, keys per lane-group and tile, consumer warps, pipeline stages
template <typename T, int G, int KPT>
using Cfg = SplitCfg<T, 576, 512, 8, G, KPT, 4, 3, true>;

template <typename T>
cudaError_t launch_t(int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s) {
    switch (heads) {
        case 1: return launch_split<Cfg<T, 1, 2>>(p, m.k, m.v, s);
        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

cudaError_t launch_split_mla_simt(bool bf16, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s) {
    return bf16 ? launch_t<__nv_bfloat16>(heads, p, m, s) : launch_t<__half>(heads, p, m, s);
}

SplitVariantInfo split_info_mla_simt(int heads) {
    switch (heads) {
        case 1: return {Cfg<__half, 1, 2>::TILE, 1, (227 * 1024) / (Cfg<__half, 1, 2>::SMEM_BYTES + 1024)};
        default: return {0, 0, 0};
    }
}
}  // namespace da
