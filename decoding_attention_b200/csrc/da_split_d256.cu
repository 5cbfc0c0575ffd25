// Instantiations of the CUDA-core split-KV kernel for head dims (256, 256).  These replace the
// reference's per-shape tiling choices (csrc/kernel/decoding_attn/decoding_fwd_hd*.cu).
#include "da_internal.h"
#include "da_split_kernel.cuh"

namespace da {
namespace {
// lanes per key row, keys per lane-group and tile, consumer warps, pipeline stages
template <typename T, int G, int KPT, bool FP8 = false>
using Cfg = SplitCfg<T, 256, 256, 16, G, KPT, 4, 2, false, 1, FP8>;

template <typename T, bool FP8>
cudaError_t launch_t(int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s) {
    switch (heads) {
        case 1: return launch_split<Cfg<T, 1, 4, FP8>>(p, m.k, m.v, s);
        case 2: return launch_split<Cfg<T, 2, 4, FP8>>(p, m.k, m.v, s);
        case 4: return launch_split<Cfg<T, 4, 4, FP8>>(p, m.k, m.v, s);
        default: return cudaErrorInvalidValue;
    }
}
}  // namespace

// fp8: K and V are FP8 e4m3 bytes (q and o stay 16-bit)
cudaError_t launch_split_d256(bool bf16, bool fp8, int heads, const SplitParams &p, const KvMaps &m, cudaStream_t s) {
    if (fp8) return bf16 ? launch_t<__nv_bfloat16, true>(heads, p, m, s) : launch_t<__half, true>(heads, p, m, s);
    return bf16 ? launch_t<__nv_bfloat16, false>(heads, p, m, s) : launch_t<__half, false>(heads, p, m, s);
}

SplitVariantInfo split_info_d256(int heads) {
    switch (heads) {
        case 1: return {Cfg<__half, 1, 4>::TILE, 1, (227 * 1024) / (Cfg<__half, 1, 4>::SMEM_BYTES + 1024)};
        case 2: return {Cfg<__half, 2, 4>::TILE, 2, (227 * 1024) / (Cfg<__half, 2, 4>::SMEM_BYTES + 1024)};
        case 4: return {Cfg<__half, 4, 4>::TILE, 4, (227 * 1024) / (Cfg<__half, 4, 4>::SMEM_BYTES + 1024)};
        default: return {0, 0, 0};
    }
}
}  // namespace da
