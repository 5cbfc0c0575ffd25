// Shared device-side building blocks of the sm_100a decode-attention kernels: the kernel parameter
// block, mbarrier / bulk-copy (TMA) PTX wrappers with bounded waits, and 16-bit -> fp32 unpacking.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace da {

// Device status word values (written by a kernel whose bounded wait ran out; read by the host with
// da_device_status()).  0 means no kernel reported a problem.  The status lives in a two-int block per
// device: [0] the status word, [1] the id of the launch that timed out (0 = none), which lets the CTAs
// of that launch that have not started yet retire at once without affecting any later launch.
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1 };

// Arguments of the split-KV kernels.  It plays the role of the reference's DecodingParams
// (csrc/kernel/decoding_attn/decoding.h:11-51) with the split-KV, LSE and ALiBi-shard extensions.
struct SplitParams {
    const void *q;   // [batch, head_q, dim]
    const void *k;   // [total_k, head_k, dim]
    const void *v;   // [total_k, head_k, dim_v]; equals k for the latent-KV (MLA) shape
    void *o;         // [batch, head_q, dim_v] in the input type, or nullptr
    float *o_f32;    // optional fp32 copy of the result
    float *lse;      // optional natural-log LSE [batch, head_q]
    float *part_o;   // split partials [batch, head_q, num_splits, dim_v] (normalised), num_splits > 1
    float *part_lse; // split partials [batch, head_q, num_splits]
    const int *cu_seq_k;       // [batch + 1]
    const int *kv_pos_offset;  // optional [batch]: position of key 0 inside a longer sequence (ALiBi)
    const int *kv_total_len;   // optional [batch]: length of that longer sequence (ALiBi)
    int *status;               // device status block: [0] status word, [1] id of a launch that gave up
    int launch_id;             // this launch's id (never 0), compared with status[1]
    const int *batch_order;    // optional [batch]: sequence handled by grid slice z (longest first), else z itself
    const int *block_table;    // optional [batch, block_table_stride]: page of each page_size-key block (paged cache)
    long long block_table_stride;
    int page_shift;            // log2(page_size); pages hold a whole number of key tiles
    long long q_row_stride, k_row_stride, v_row_stride, o_row_stride;  // in elements
    int head_q, head_k;
    int dim;           // head dim of q / k as the caller gave it (a kernel may run it padded, e.g. 96 as 128)
    int group;         // query heads per KV head
    int head_chunks;   // CTAs that share one KV head (group / heads-per-CTA)
    int batch;
    int num_splits;
    int chunk_keys;    // keys per split (multiple of the tile)
    int is_alibi;
    int use_tmap;      // full tiles are fetched with one tiled TMA copy through the tensor maps
    float scale_log2;  // softmax scale * log2(e) (times the K scale of a quantised cache)
    float out_scale;   // factor on the output: the V scale of a quantised cache, else 1
};

// Has an earlier CTA of this very launch given up a bounded wait?  (Later launches carry another id
// and are not affected; a replayed CUDA graph repeats its id, so after a timeout inside a replay
// the host should read da_device_status(), which clears the block, before replaying again.)
__device__ __forceinline__ bool launch_aborted(const SplitParams &p) {
    return reinterpret_cast<volatile int *>(p.status)[1] == p.launch_id;
}
__device__ __forceinline__ void report_timeout(const SplitParams &p) {
    atomicExch(p.status, kStatusWaitTimeout);
    atomicExch(p.status + 1, p.launch_id);
}
// Last key (exclusive) of key-range split `split`: splits cover chunk_keys keys each; the last one
// runs to the end of the sequence, so a sequence longer than the max_seq_k the plan was sized for
// is still read completely.
__device__ __forceinline__ int split_key_end(const SplitParams &p, int split, int len) {
    const long long e = (long long)(split + 1) * p.chunk_keys;
    return (split == p.num_splits - 1 || e > len) ? len : (int)e;
}

// Row of the cache that holds key `key0` of sequence `b`.  Packed cache: the sequence's rows are
// consecutive from cu_seq_k[b].  Paged cache: the block table names the page.  Rows are consecutive for
// kv_run_keys() keys from a multiple of that number: a whole tile, or a page when pages are shorter.
__device__ __forceinline__ size_t kv_tile_row(const SplitParams &p, int b, int seq_begin, int key0) {
    if (!p.block_table) return (size_t)seq_begin + key0;
    const int page = p.block_table[(size_t)b * p.block_table_stride + (key0 >> p.page_shift)];
    return ((size_t)page << p.page_shift) + (key0 & ((1 << p.page_shift) - 1));
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream is still running; it must not touch the predecessor's
// output before pdl_wait() (which returns once the predecessor has finished and flushed).  The
// predecessor lets the successor's CTAs be scheduled early with pdl_launch_dependents().  Both are
// no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ int kv_run_keys(const SplitParams &p, int tile) {
    return (p.block_table && (1 << p.page_shift) < tile) ? (1 << p.page_shift) : tile;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  A legitimate wait here lasts microseconds; after kMaxWaitCycles SM clocks (about
// a quarter of a second) the waiter gives up, raises the CTA's abort flag so that the other
// waiters of the CTA leave too, and the caller records kStatusWaitTimeout.
constexpr long long kMaxWaitCycles = 500ll * 1000 * 1000;
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kMaxWaitCycles) break;
        }
    }
    *abort_flag = 1;
    return false;
}

// One row of a K/V tile: global -> shared bulk copy (TMA engine, no tensor map), completion
// signalled on an mbarrier as transferred bytes.  Addresses and size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s_hint(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                                   uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Shared -> global bulk copy (TMA engine, no tensor map): addresses and size multiples of 16 bytes.  The
// copies of a thread form a group (commit); wait_read returns once their source bytes have been read,
// which a thread must do before the shared memory is reused or the CTA exits.
__device__ __forceinline__ void bulk_store_s2g(void *dst_gmem, const void *src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// 16-byte asynchronous copy global -> shared through the load/store unit (not the TMA engine).  With
// src_bytes = 0 nothing is read and the 16 bytes are zero-filled.
__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src_gmem, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(src_bytes)
                 : "memory");
}
// The same asking L2 to fetch the whole 256-byte block around a missing sector (what the tensor maps of this
// library ask for too): a stream that is the first to touch its rows then reads DRAM in 256-byte pieces.
__device__ __forceinline__ void cp_async16_l2_256(void *dst_smem, const void *src_gmem, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem),
                 "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A whole K/V tile: tiled TMA copy of the box {dim, 1 head, tile rows} at (0, head, row) of the
// rank-3 tensor map [rows][heads][dim].  One instruction per tile; the engine walks the rows.
__device__ __forceinline__ void tma_load_tile_3d(void *dst_smem, const CUtensorMap *tmap, int c0, int c1, int c2,
                                                 uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(smem_u32(dst_smem)),
        "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Unpack eight 16-bit values (one 16-byte chunk) to fp32.
template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &raw, float (&f)[8]);

template <>
__device__ __forceinline__ void unpack8<__half>(const uint4 &raw, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4 &raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Eight FP8 e4m3 values (8 bytes) to fp32.
__device__ __forceinline__ void unpack8_e4m3(const uint2 &raw, float (&f)[8]) {
    const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_fp8x2_storage_t pair = (__nv_fp8x2_storage_t)((w[i >> 1] >> ((i & 1) * 16)) & 0xffffu);
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3);
        const float2 t = __half22float2(*reinterpret_cast<const __half2 *>(&h));
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
// One lane's chunk of a K or V row in shared memory, eight elements, to fp32.  KVQ: 0 = the 16-bit type T (16 bytes),
// 1 = FP8 e4m3 (8 bytes), 2 = signed 8-bit integers (8 bytes), 3 = signed 4-bit integers, low nibble first (4 bytes).
template <typename T, int KVQ>
__device__ __forceinline__ void load_chunk8(const uint8_t *ptr, float (&f)[8]) {
    if (KVQ == 1) {
        unpack8_e4m3(*reinterpret_cast<const uint2 *>(ptr), f);
    } else if (KVQ == 2) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(ptr);
        const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (float)(int)(int8_t)((w[i >> 2] >> ((i & 3) * 8)) & 0xffu);
    } else if (KVQ == 3) {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(ptr);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (float)(((int)(w << (28 - 4 * i))) >> 28);  // sign-extended nibble i
    } else {
        unpack8<T>(*reinterpret_cast<const uint4 *>(ptr), f);
    }
}

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ __half from_float<__half>(float x) {
    return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace da
