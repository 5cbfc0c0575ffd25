// C ABI of libdecoding_attn_b200.so: argument checks, split heuristic, scratch management and
// kernel dispatch.  It does the work of the reference's set_dmha_fwd_params / run_dmha_fwd
// (csrc/ops/decoding_attn.cpp:13-68) and of its DA_FP16_SWITCH / DA_HEADDIM_SWITCH macros
// (csrc/common/common.h:62-96), but returns status codes instead of calling exit().
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/decoding_attn_b200.h"
#include "da_internal.h"

namespace da {

namespace {

thread_local char g_err[512] = "";
thread_local cudaEvent_t g_prof_start = nullptr, g_prof_stop = nullptr;
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// Kernel status block: one per device (a __device__ variable lives in every device's copy of the
// module).  [0]: kernels that give up a bounded wait write kStatusWaitTimeout here; [1]: the id of
// the launch that did, so that only the remaining CTAs of that launch retire early.
__device__ int g_status_word[2];
std::atomic<uint32_t> g_launch_id{0};

// Ids of launches: 1, 2, ... (never 0, the "no launch gave up" value of the status block).
int next_launch_id() {
    const uint32_t n = g_launch_id.fetch_add(1, std::memory_order_relaxed);
    return (int)(n % 0x7ffffffeu) + 1;
}

constexpr int kMaxDevices = 64;
struct DeviceState {
    std::mutex mu;
    int *status_ptr = nullptr;
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    std::vector<void *> retired;  // outgrown scratch buffers, kept until the process ends
    std::mutex staging_mu;    // held for the whole of a da_decode_fwd_host call
    void *staging = nullptr;  // device copies of host tensors for da_decode_fwd_host
    size_t staging_bytes = 0;
    int sm_count = 0;
};
DeviceState g_dev[kMaxDevices];

int device_state(DeviceState **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(DA_ERR_CUDA, "device ordinal %d out of range", dev);
    DeviceState &st = g_dev[dev];
    std::lock_guard<std::mutex> lock(st.mu);
    if (!st.status_ptr) {
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&st.status_ptr), g_status_word);
        if (e != cudaSuccess) return fail(DA_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        e = cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return fail(DA_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    }
    *out = &st;
    return DA_OK;
}

enum class Shape { kD64, kD96, kD128, kD256, kMla, kMla2Sm, kGqaTc, kGqaQuad, kNone };

Shape shape_of(int64_t dim, int64_t dim_v, bool has_v) {
    if (has_v) {
        if (dim == 64 && dim_v == 64) return Shape::kD64;
        if (dim == 96 && dim_v == 96) return Shape::kD96;
        if (dim == 128 && dim_v == 128) return Shape::kD128;
        if (dim == 256 && dim_v == 256) return Shape::kD256;
        return Shape::kNone;
    }
    if (dim == 576 && dim_v == 512) return Shape::kMla;
    return Shape::kNone;
}

// Environment overrides, read once per process (the reference has none; these exist for benchmarks):
//   DA_NUM_SPLITS=<n>   key-range splits per sequence when the caller leaves num_splits at 0
//   DA_KERNEL=simt      keep every shape on the CUDA-core kernel (no tensor-core path)
//   DA_KERNEL=gqa1      groups of at most 32 query heads stay on da_gqa_tc_kernel (for comparisons with the four-stream kernel)
struct EnvOverrides {
    int num_splits = 0;
    bool force_simt = false;
    bool no_quad = false;
};
const EnvOverrides &env_overrides() {
    static const EnvOverrides env = [] {
        EnvOverrides e;
        if (const char *s = getenv("DA_NUM_SPLITS")) e.num_splits = atoi(s) > 0 ? atoi(s) : 0;
        if (const char *k = getenv("DA_KERNEL")) e.force_simt = strcmp(k, "simt") == 0;
        if (const char *k = getenv("DA_KERNEL")) e.no_quad = strcmp(k, "gqa1") == 0;
        return e;
    }();
    return env;
}

// The tensor-core kernel covers the shape the latent-KV layout exists for: up to 128 query heads over
// one KV head (128 in the full model, 16..64 per GPU under tensor parallelism; the reference's suite
// runs 16, 32, 64 and 128, tests/test_decoding_attn.py:97).  Fewer than 8 heads, or several KV heads,
// run on the CUDA-core kernel.
bool mla_on_tensor_cores(const da_decode_args_t &a) {
    if (a.v != nullptr || a.dim != 576 || a.dim_v != 512 || a.head_k != 1 || env_overrides().force_simt) return false;
    return a.head_q >= 8 && a.head_q <= 128;
}

// Head dims 64, 128 and 256 run on the tensor cores unless the group of query heads per KV head is one
// the CUDA-core kernel serves well: 1, 2 or 4 heads, which it handles in one CTA per KV head at the HBM
// rate (and 3 heads at dims 64 and 256, where its two chunks still win).  Any other group would cost it
// one pass over K and V per 1-, 2- or 4-head chunk (dim 128, 7 heads: 344 us against 121 us on the
// tensor cores for 64 x 4096 keys), and from 8 heads up it is bound by instruction issue anyway (dim
// 256, 32 heads: 979 against 141 us).
bool gqa_on_tensor_cores(const da_decode_args_t &a) {
    if (!a.v || a.dim != a.dim_v || (a.dim != 64 && a.dim != 96 && a.dim != 128 && a.dim != 256)) return false;
    const int64_t group = a.head_q / a.head_k;
    if (env_overrides().force_simt || group > 128) return false;
    // (head dim 96 runs on the tensor-core kernel's 128-column instantiation, the tensor maps zero-filling columns 96-127)
    return a.dim == 128 ? (group >= 3 && group != 4) : group >= 5;
}

int heads_per_cta(Shape s, int group) {
    if (s == Shape::kMla) return 1;
    if (s == Shape::kGqaTc || s == Shape::kGqaQuad) return group;
    if (s == Shape::kMla2Sm) return group;  // all heads of the KV head in one CTA / CTA pair
    if (group % 4 == 0) return 4;
    if (group % 2 == 0) return 2;
    return 1;
}

SplitVariantInfo variant_info(Shape s, int heads) {
    switch (s) {
        case Shape::kD64: return split_info_d64(heads);
        case Shape::kD96: return split_info_d96(heads);
        case Shape::kD128: return split_info_d128(heads);
        case Shape::kD256: return split_info_d256(heads);
        case Shape::kMla: return split_info_mla_simt(heads);
        case Shape::kGqaTc: return split_info_gqa_tc();
        case Shape::kGqaQuad: return split_info_gqa_quad();
        case Shape::kMla2Sm: return split_info_mla_2sm();
        default: return {0, 0, 0};
    }
}

// ---- tensor maps -----------------------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver-API function; it is looked up at run time so that the library
// links against the CUDA runtime only.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess) {
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// Rank-3 map over a K or V tensor seen as [rows][head_k][dim] with box {dim, 1, tile_keys}.  The
// row extent is not known to the library (only cu_seq_k on the device is), so it is set to the
// largest value a coordinate can take; the kernels use the map only for tiles that lie wholly
// inside a sequence and fetch ragged tails row by row.
constexpr uint64_t kMapRows = 1ull << 31;
struct MapKey {
    const void *base;
    uint64_t dims[3];
    uint64_t strides[2];
    uint32_t box[3];
    int rank, swizzle128, dtype;  // dtype: 0 fp16, 1 bf16, 2 one-byte elements
};
struct MapCacheEntry {
    MapKey key;
    CUtensorMap map;
    bool valid = false;
};
thread_local MapCacheEntry g_map_cache[8];
thread_local int g_map_next = 0;

// Tiled tensor map over 16-bit (or, dtype 2, one-byte) elements; dims/strides/box innermost first, strides in bytes for
// dimensions 1.. (dimension 0 is contiguous).  Recently built maps are kept per thread.
int make_tensor_map(const void *base, int rank, const uint64_t *dims, const uint64_t *strides, const uint32_t *box,
                    bool swizzle128, int dtype, CUtensorMap *out) {
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.base = base;
    key.rank = rank;
    key.swizzle128 = swizzle128;
    key.dtype = dtype;
    for (int i = 0; i < rank; ++i) {
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (i + 1 < rank) key.strides[i] = strides[i];
    }
    for (auto &e : g_map_cache) {
        if (e.valid && memcmp(&e.key, &key, sizeof(key)) == 0) {
            *out = e.map;
            return DA_OK;
        }
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(DA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint32_t estr[3] = {1, 1, 1};
    cuuint64_t d[3], st[2];
    cuuint32_t bx[3];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        bx[i] = box[i];
        if (i + 1 < rank) st[i] = strides[i];
    }
    const CUtensorMapDataType dt = dtype == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                              : (dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    CUresult r = fn(out, dt, (cuuint32_t)rank,
                    const_cast<void *>(base), d, st, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    MapCacheEntry &slot = g_map_cache[g_map_next];
    g_map_next = (g_map_next + 1) % 8;
    slot.key = key;
    slot.map = *out;
    slot.valid = true;
    return DA_OK;
}

int make_kv_tensor_map(const void *base, long long row_stride, int head_k, int dim, int tile, int dtype,
                       CUtensorMap *out) {
    const uint64_t eb = dtype == 2 ? 1 : 2;
    const uint64_t dims[3] = {(uint64_t)dim, (uint64_t)head_k, kMapRows};
    const uint64_t strides[2] = {(uint64_t)dim * eb, (uint64_t)row_stride * eb};
    const uint32_t box[3] = {(uint32_t)dim, 1, (uint32_t)tile};
    return make_tensor_map(base, 3, dims, strides, box, false, dtype, out);
}

struct Plan {
    Shape shape;
    int heads;       // query heads per CTA
    int head_chunks; // CTAs per KV head
    int num_splits;
    int chunk_keys;
    int tile_keys;
    size_t scratch_bytes;
    size_t order_offset;  // byte offset of the launch-order array inside the scratch, or 0 if none
};

// Pick the number of key-range splits.  The host does not know the sequence lengths (cu_seq_k is a
// device array), only max_seq_k, so the grid is (splits, kv heads * head chunks, batch) and CTAs
// whose range lies beyond their sequence's end retire at once.  Aim for several waves of CTAs over
// all SMs, but keep at least kMinTiles tiles per CTA (pipeline fill, partial write-out) and at most
// kMaxTiles when the batch is too small for the longest-first launch order (tail effect when lengths
// vary inside a batch).
int make_plan(const da_decode_args_t &a, int sm_count, Plan *plan) {
    const bool has_v = a.v != nullptr;
    Shape shape = shape_of(a.dim, a.dim_v, has_v);
    if (shape == Shape::kNone) {
        return fail(DA_ERR_UNSUPPORTED,
                    "unsupported (dim=%lld, dim_v=%lld, v %s): supported are (64,64) (96,96) (128,128) (256,256) "
                    "with v and (576,512) without",
                    (long long)a.dim, (long long)a.dim_v, has_v ? "given" : "NULL");
    }
    if (a.kv_dtype != DA_KV_SAME_AS_Q) {
        if (shape == Shape::kMla) {
            return fail(DA_ERR_UNSUPPORTED, "a quantised cache is supported for (dim, dim_v) (64,64) (96,96) (128,128) (256,256) with v given");
        }
    } else if (shape == Shape::kMla && mla_on_tensor_cores(a)) {
        shape = Shape::kMla2Sm;
    }
    if (a.kv_dtype == DA_KV_SAME_AS_Q &&
        (shape == Shape::kD64 || shape == Shape::kD96 || shape == Shape::kD128 || shape == Shape::kD256) &&
        gqa_on_tensor_cores(a)) {
        shape = Shape::kGqaTc;  // (a quantised cache is read by the CUDA-core kernel, whatever the group size)
        // Up to 32 heads per KV head: four key streams, one per TMEM lane quadrant (head dim 256 has no room for it).
        if (a.head_q / a.head_k <= 32 && a.dim != 256 && !env_overrides().no_quad) shape = Shape::kGqaQuad;
    }
    const int group = (int)(a.head_q / a.head_k);
    const int heads = heads_per_cta(shape, group);
    const SplitVariantInfo info = variant_info(shape, heads);
    const int tile = info.tile_keys;
    // The tensor-core MLA kernel runs two CTAs (one per half of the output columns) per key range.
    // The tensor-core MLA kernel runs one pair of CTAs (two SMs) per key range.
    const int64_t units = shape == Shape::kMla2Sm ? a.batch : a.batch * a.head_k * (group / heads);
    const int64_t max_len = a.max_seq_k > 0 ? a.max_seq_k : 1;
    const int64_t tiles_per_unit = (max_len + tile - 1) / tile;

    // A tensor-core MLA CTA first stages 144 KB of Q: give it at least 256 keys to amortise that.
    const int kMinTiles = 4, kWaves = 4, kMaxTiles = 32;
    int64_t splits;
    if (a.num_splits > 0) {
        splits = a.num_splits;
    } else if (env_overrides().num_splits > 0) {
        splits = env_overrides().num_splits;
    } else if (shape == Shape::kMla2Sm || shape == Shape::kGqaTc || shape == Shape::kGqaQuad) {
        // One CTA per SM and long-running CTAs: pick the split count whose CTA total fills whole
        // waves best, weighed against the fixed cost of every extra CTA.
        const int64_t slots = shape == Shape::kMla2Sm ? sm_count / 2 : sm_count;
        double best = -1.0;
        splits = 1;
        for (int64_t s = 1; s <= tiles_per_unit && s <= 64; ++s) {
            const int64_t tpc = (tiles_per_unit + s - 1) / s;
            if (s > 1 && tpc < kMinTiles) break;
            const int64_t s_eff = (tiles_per_unit + tpc - 1) / tpc;
            if (s_eff != s) continue;
            const int64_t total = units * s_eff;
            const int64_t waves = (total + slots - 1) / slots;
            // wave efficiency x the share of a CTA's life spent on tiles (a CTA costs about six tiles'
            // worth of set-up: barrier/TMEM set-up, Q staging, pipeline fill, epilogue)
            const double score = (double)total / (double)(waves * slots) * (double)tpc / (double)(tpc + 6);
            if (score > best) {
                best = score;
                splits = s;
            }
        }
        // The scores above take every sequence for max_seq_k long.  A ragged batch (the caller's total_k hint puts
        // the mean length under three quarters of that) is bound by its longest sequences when they run unsplit:
        // keep a CTA's share near the average load of a CTA slot (64 latent-KV sequences of 1 K-16 K keys: 233 us
        // unsplit, 182 us in four splits, 200 us in the three this rule picks).
        if (a.total_k > 0 && a.batch > 0 && units <= slots) {  // (more units than slots: the launch order balances them)
            const int64_t mean_tiles = ((int64_t)a.total_k / a.batch + tile - 1) / tile;
            if (mean_tiles * 4 <= tiles_per_unit * 3) {
                int64_t per_slot = units * mean_tiles / slots;
                if (per_slot < kMinTiles) per_slot = kMinTiles;
                const int64_t ragged = (tiles_per_unit + per_slot - 1) / per_slot;
                if (ragged > splits) splits = ragged < 64 ? ragged : 64;
            }
        }
    } else {
        const int64_t slots = (int64_t)sm_count * (info.ctas_per_sm > 0 ? info.ctas_per_sm : 1);
        int64_t tiles_per_cta = (units * tiles_per_unit) / (slots * kWaves);
        if (tiles_per_cta < kMinTiles) tiles_per_cta = kMinTiles;
        // (with 16 sequences or more the CTAs are handed out longest sequence first and no cap is needed:
        // config 2, 2 048 units of up to 64 tiles, 396 us with the two splits the cap asks for, 377 us unsplit)
        if (a.batch < 16 && tiles_per_cta > kMaxTiles) tiles_per_cta = kMaxTiles;
        splits = (tiles_per_unit + tiles_per_cta - 1) / tiles_per_cta;
        // A ragged batch (the caller's total_k hint puts the mean length under three quarters of max_seq_k) with
        // half as many units again as CTA slots balances itself once it is launched longest first: unsplit it saves
        // the partials and the CTAs that find their range empty (96 / 128 / 192 sequences of 512-4096 keys, 8 KV
        // heads: 157 -> 142, 199 -> 187, 304 -> 291 us).
        if (a.total_k > 0 && a.batch >= 16 && units * 2 >= slots * 3) {
            const int64_t mean_tiles = ((int64_t)a.total_k / a.batch + tile - 1) / tile;
            if (mean_tiles * 4 <= tiles_per_unit * 3) splits = 1;
        }
        // Fewer units than CTA slots: one full wave of equal chunks beats several waves of short CTAs
        // (measured: 16 K keys x 32 heads 75.7 -> 50.1 us, 64 K keys 190 -> 167 us), as long as a chunk
        // still amortises a CTA's set-up.
        if (units <= slots) {
            const int64_t one_wave = slots / units;
            const bool fills = units * one_wave * 5 >= slots * 4;  // at least 80 % of the slots get a CTA
            if (fills && (tiles_per_unit + one_wave - 1) / one_wave >= kMinTiles) splits = one_wave;
            if (max_len <= 2048) {
                // Short sequences: a CTA's set-up and the merge launch weigh as much as the keys.  Cost of a split
                // count in keys' worth of time: waves x (set-up + chunk) + merge (measured, 32 heads x dim 128:
                // 8 x 1024 keys 35.8 us with 4 splits, 28.7 us unsplit; 4 x 1024 keys 23.6 / 21.5 / 24.6 us with 3 / 2 / 1).
                const int64_t kSetupKeys = 384, kMergeKeys = 512;
                int64_t best_cost = INT64_MAX;
                for (int64_t s = 1; s <= tiles_per_unit && s <= 64; ++s) {
                    const int64_t tpc = (tiles_per_unit + s - 1) / s;
                    if (s > 1 && tpc < kMinTiles) break;
                    if ((tiles_per_unit + tpc - 1) / tpc != s) continue;
                    const int64_t waves = (units * s + slots - 1) / slots;
                    const int64_t cost = waves * (kSetupKeys + tpc * tile) + (s > 1 ? kMergeKeys : 0);
                    if (cost < best_cost) {
                        best_cost = cost;
                        splits = s;
                    }
                }
            }
        }
    }
    if (splits < 1) splits = 1;
    if (splits > tiles_per_unit) splits = tiles_per_unit;
    if (splits > 65535) splits = 65535;
    int64_t chunk_tiles = (tiles_per_unit + splits - 1) / splits;
    splits = (tiles_per_unit + chunk_tiles - 1) / chunk_tiles;  // drop splits that would be empty for every row

    plan->shape = shape;
    plan->heads = heads;
    plan->head_chunks = group / heads;
    plan->num_splits = (int)splits;
    plan->chunk_keys = (int)(chunk_tiles * tile);
    plan->tile_keys = tile;
    plan->scratch_bytes =
        splits > 1 ? (size_t)a.batch * a.head_q * splits * ((size_t)a.dim_v + 1) * sizeof(float) : 0;
    // More CTAs than fit at once and enough sequences for their order to matter: launch longest first.
    const int64_t all_slots = (int64_t)sm_count * (info.ctas_per_sm > 0 ? info.ctas_per_sm : 1);
    plan->order_offset = 0;
    // (the order kernel costs 3-4 us: worth it only when a CTA runs long enough for a ragged tail to cost more)
    if (a.batch >= 16 && units * splits > all_slots && chunk_tiles >= 16) {
        plan->scratch_bytes = (plan->scratch_bytes + 15) / 16 * 16;
        plan->order_offset = plan->scratch_bytes + 16;  // never 0
        plan->scratch_bytes = plan->order_offset + (size_t)a.batch * sizeof(int);
    }
    return DA_OK;
}

int check_args(const da_decode_args_t *a) {
    if (!a) return fail(DA_ERR_INVALID_ARG, "args is NULL");
    if (a->struct_size != sizeof(da_decode_args_t)) {
        return fail(DA_ERR_INVALID_ARG, "struct_size %u != sizeof(da_decode_args_t) %zu", a->struct_size,
                    sizeof(da_decode_args_t));
    }
    // Same conditions as the reference's DA_CHECKs (csrc/ops/decoding_attn.cpp:16-22).
    if (!a->q || !a->k || !a->cu_seq_k) return fail(DA_ERR_INVALID_ARG, "q, k and cu_seq_k must not be NULL");
    if (!a->o && !a->o_f32) return fail(DA_ERR_INVALID_ARG, "one of o / o_f32 must be given");
    if (a->batch <= 0 || a->head_q <= 0 || a->head_k <= 0 || a->dim <= 0 || a->dim_v <= 0) {
        return fail(DA_ERR_INVALID_ARG, "batch, head_q, head_k, dim and dim_v must be positive");
    }
    if (a->head_q % a->head_k != 0) {
        return fail(DA_ERR_INVALID_ARG, "head_q (%lld) must be a multiple of head_k (%lld)", (long long)a->head_q,
                    (long long)a->head_k);
    }
    if (a->dim > 576 || a->dim_v > 512) return fail(DA_ERR_INVALID_ARG, "dim must be <= 576 and dim_v <= 512");
    if (a->batch > 65535) return fail(DA_ERR_INVALID_ARG, "batch must be <= 65535");
    if (a->max_seq_k < 0) return fail(DA_ERR_INVALID_ARG, "max_seq_k must not be negative");
    const uintptr_t align_or = (uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->o |
                               (uintptr_t)a->o_f32 | (uintptr_t)a->workspace;
    if (align_or & 15u) return fail(DA_ERR_INVALID_ARG, "q, k, v, o, o_f32 and workspace must be 16-byte aligned");
    const int64_t strides[4] = {a->q_row_stride, a->k_row_stride, a->v_row_stride, a->o_row_stride};
    const int64_t mins[4] = {a->head_q * a->dim, a->head_k * a->dim, a->head_k * (a->v ? a->dim_v : a->dim),
                             a->head_q * a->dim_v};
    for (int i = 0; i < 4; ++i) {
        if (strides[i] == 0) continue;
        const bool kv_stride = i == 1 || i == 2;  // 16 bytes, whatever the element size
        const int64_t unit = !kv_stride || a->kv_dtype == DA_KV_SAME_AS_Q ? 8 : (a->kv_dtype == DA_KV_INT4 ? 32 : 16);
        if (strides[i] < mins[i] || strides[i] % unit != 0) {
            return fail(DA_ERR_INVALID_ARG, "row stride %d must be a multiple of 16 bytes and cover a row", i);
        }
    }
    if (a->kv_dtype < DA_KV_SAME_AS_Q || a->kv_dtype > DA_KV_INT4) {
        return fail(DA_ERR_INVALID_ARG, "kv_dtype %d: 0 (the type of q), 1 (FP8 e4m3), 2 (int8) or 3 (int4) expected", a->kv_dtype);
    }
    if (a->kv_dtype != DA_KV_SAME_AS_Q && !a->v) return fail(DA_ERR_UNSUPPORTED, "a quantised cache needs a separate v tensor");
    if (a->block_table) {
        // A key tile (32 or 64 keys) is fetched in runs of consecutive rows: whole, or page by page.
        if (a->page_size < 16 || (a->page_size & (a->page_size - 1)) != 0) {
            return fail(DA_ERR_UNSUPPORTED, "page_size %d: paged caches need a power-of-two page size >= 16", a->page_size);
        }
        if (a->block_table_stride <= 0) return fail(DA_ERR_INVALID_ARG, "block_table_stride must be positive");
        if (a->max_seq_k > a->block_table_stride * (int64_t)a->page_size) {
            return fail(DA_ERR_INVALID_ARG, "block table rows (%lld pages of %d keys) cannot hold max_seq_k = %lld",
                        (long long)a->block_table_stride, a->page_size, (long long)a->max_seq_k);
        }
    } else if (a->page_size != 0 || a->block_table_stride != 0) {
        return fail(DA_ERR_INVALID_ARG, "page_size / block_table_stride given without a block_table");
    }
    return DA_OK;
}

}  // namespace

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int report_error(int code, const char *msg) { return fail(code, "%s", msg); }

int xmerge_status_ptr(int **out) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc == DA_OK) *out = st->status_ptr;
    return rc;
}

}  // namespace da

using namespace da;

extern "C" {

size_t da_decode_workspace_bytes(const da_decode_args_t *a) {
    if (check_args(a) != DA_OK) return 0;
    DeviceState *st = nullptr;
    if (device_state(&st) != DA_OK) return 0;
    Plan plan;
    if (make_plan(*a, st->sm_count, &plan) != DA_OK) return 0;
    return plan.scratch_bytes;
}

int da_decode_num_splits(const da_decode_args_t *a) {
    if (check_args(a) != DA_OK) return -1;
    DeviceState *st = nullptr;
    if (device_state(&st) != DA_OK) return -1;
    Plan plan;
    if (make_plan(*a, st->sm_count, &plan) != DA_OK) return -1;
    return plan.num_splits;
}

int da_plan_num_splits(const da_decode_args_t *a, int sm_count) {
    if (check_args(a) != DA_OK || sm_count <= 0) return -1;
    Plan plan;
    if (make_plan(*a, sm_count, &plan) != DA_OK) return -1;
    return plan.num_splits;
}

int da_decode_fwd(const da_decode_args_t *a) {
    int rc = check_args(a);
    if (rc != DA_OK) return rc;
    DeviceState *st = nullptr;
    rc = device_state(&st);
    if (rc != DA_OK) return rc;
    Plan plan;
    rc = make_plan(*a, st->sm_count, &plan);
    if (rc != DA_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(a->stream);

    float *scratch = nullptr;
    if (plan.scratch_bytes) {
        if (a->workspace) {
            if (a->workspace_bytes < plan.scratch_bytes) {
                return fail(DA_ERR_WORKSPACE, "workspace has %zu bytes, %zu needed", a->workspace_bytes,
                            plan.scratch_bytes);
            }
            scratch = static_cast<float *>(a->workspace);
        } else {
            std::lock_guard<std::mutex> lock(st->mu);
            if (st->scratch_bytes < plan.scratch_bytes) {
                // Grow-only, at least doubling.  Kernels already queued may still use the old buffer, so it
                // is parked instead of freed (no device synchronisation inside a decode call); doubling
                // keeps all parked buffers together below the size of the live one.
                size_t want = st->scratch_bytes * 2 > plan.scratch_bytes ? st->scratch_bytes * 2 : plan.scratch_bytes;
                void *fresh = nullptr;
                cudaError_t e = cudaMalloc(&fresh, want);
                if (e != cudaSuccess) {
                    return fail(DA_ERR_WORKSPACE, "cudaMalloc(%zu) for split scratch: %s", want,
                                cudaGetErrorString(e));
                }
                if (st->scratch) st->retired.push_back(st->scratch);
                st->scratch = fresh;
                st->scratch_bytes = want;
            }
            scratch = static_cast<float *>(st->scratch);
        }
    }

    SplitParams p;
    memset(&p, 0, sizeof(p));
    p.q = a->q;
    p.k = a->k;
    p.v = a->v ? a->v : a->k;  // csrc/ops/decoding_attn.cpp:30
    p.o = a->o;
    p.o_f32 = a->o_f32;
    p.lse = a->lse;
    p.cu_seq_k = a->cu_seq_k;
    p.kv_pos_offset = a->kv_pos_offset;
    p.kv_total_len = a->kv_total_len;
    p.status = st->status_ptr;
    p.launch_id = next_launch_id();
    p.block_table = a->block_table;
    p.block_table_stride = a->block_table_stride;
    p.page_shift = 0;
    for (int ps = a->page_size; ps > 1; ps >>= 1) ++p.page_shift;
    p.q_row_stride = a->q_row_stride ? a->q_row_stride : a->head_q * a->dim;
    p.k_row_stride = a->k_row_stride ? a->k_row_stride : a->head_k * a->dim;
    p.v_row_stride = a->v ? (a->v_row_stride ? a->v_row_stride : a->head_k * a->dim_v) : p.k_row_stride;
    p.o_row_stride = a->o_row_stride ? a->o_row_stride : a->head_q * a->dim_v;
    p.head_q = (int)a->head_q;
    p.head_k = (int)a->head_k;
    p.dim = (int)a->dim;
    p.group = (int)(a->head_q / a->head_k);
    p.head_chunks = plan.head_chunks;
    p.batch = (int)a->batch;
    p.num_splits = plan.num_splits;
    p.chunk_keys = plan.chunk_keys;
    p.is_alibi = a->is_alibi ? 1 : 0;
    const float scale = a->softmax_scale > 0.0f ? a->softmax_scale : (float)(1.0 / std::sqrt((double)a->dim));
    p.scale_log2 = scale * kLog2e;
    p.out_scale = 1.0f;
    if (a->kv_dtype != DA_KV_SAME_AS_Q) {  // the cache stands for k * k_scale, v * v_scale: both factors leave the loops
        p.scale_log2 *= a->k_scale > 0.0f ? a->k_scale : 1.0f;
        p.out_scale = a->v_scale > 0.0f ? a->v_scale : 1.0f;
    }
    if (plan.order_offset) {
        int *order = reinterpret_cast<int *>(reinterpret_cast<char *>(scratch) + plan.order_offset);
        cudaError_t oe = launch_order(a->cu_seq_k, (int)a->batch, a->max_seq_k, order, stream);
        if (oe != cudaSuccess) return fail(DA_ERR_CUDA, "order kernel launch: %s", cudaGetErrorString(oe));
        p.batch_order = order;
    }
    if (plan.num_splits > 1) {
        p.part_o = scratch;
        p.part_lse = scratch + (size_t)a->batch * a->head_q * plan.num_splits * a->dim_v;
    }
    if ((int64_t)p.head_k * p.head_chunks > 65535) {
        return fail(DA_ERR_INVALID_ARG, "head_k * head chunks exceeds the grid limit");
    }
    // Rows per TMA box: the tile, or a page when pages are shorter than the tile.
    const int box_keys = (a->block_table && a->page_size < plan.tile_keys) ? a->page_size : plan.tile_keys;

    const bool bf16 = a->is_bf16 != 0;
    const int kvq = a->kv_dtype;  // 0 as q, 1 FP8, 2 int8, 3 int4
    KvMaps maps;
    memset(&maps, 0, sizeof(maps));
    // Tiled TMA needs a global stride that is a multiple of 16 bytes (checked above: 8 elements) and
    // a box of at most 256 elements per dimension; the latent-KV rows (576) keep the row-wise path.
    p.use_tmap = (plan.shape != Shape::kMla) && (plan.shape != Shape::kMla2Sm) && (plan.shape != Shape::kGqaTc) &&
                 (plan.shape != Shape::kGqaQuad);
    CUtensorMap tm_q;
    memset(&tm_q, 0, sizeof(tm_q));
    if (plan.shape == Shape::kGqaTc || plan.shape == Shape::kGqaQuad) {
        // q as [batch][head_q][dim] in boxes {64, min(128, head_q), 1} (32 rows for the four-stream kernel, which
        // stages the group once per row block); K and V as [rows][head_k][dim] in
        // boxes {64, 1, tile}: all 128-byte-swizzled, the layout the UMMA descriptors name.
        const uint64_t dim = (uint64_t)a->dim;  // 64, 96, 128 or 256 (96: boxes at column 64 come back half zero-filled)
        const uint64_t qd[3] = {dim, (uint64_t)a->head_q, (uint64_t)a->batch};
        const uint64_t qs[2] = {dim * 2, (uint64_t)p.q_row_stride * 2};
        const uint32_t q_rows = plan.shape == Shape::kGqaQuad ? 32 : 128;
        const uint32_t qb[3] = {64, (uint32_t)(a->head_q < q_rows ? a->head_q : q_rows), 1};
        rc = make_tensor_map(p.q, 3, qd, qs, qb, true, bf16 ? 1 : 0, &tm_q);
        if (rc != DA_OK) return rc;
        const uint64_t kd[3] = {dim, (uint64_t)a->head_k, kMapRows};
        const uint64_t ks[2] = {dim * 2, (uint64_t)p.k_row_stride * 2};
        const uint64_t vs[2] = {dim * 2, (uint64_t)p.v_row_stride * 2};
        const uint32_t kb[3] = {64, 1, (uint32_t)box_keys};
        rc = make_tensor_map(p.k, 3, kd, ks, kb, true, bf16 ? 1 : 0, &maps.k);
        if (rc != DA_OK) return rc;
        rc = make_tensor_map(p.v, 3, kd, vs, kb, true, bf16 ? 1 : 0, &maps.v);
        if (rc != DA_OK) return rc;
    }
    if (plan.shape == Shape::kMla2Sm) {
        // q as [batch][head_q][576] in boxes {64, min(64, head_q), 1} (one CTA's heads; rows past head_q read as
        // zeros); the latent cache as [rows][576] in boxes {64, half a tile of keys}; both 128-byte-swizzled.
        const uint64_t qd[3] = {576, (uint64_t)a->head_q, (uint64_t)a->batch};
        const uint64_t qs[2] = {576 * 2, (uint64_t)p.q_row_stride * 2};
        const uint32_t qb[3] = {64, (uint32_t)(a->head_q < 64 ? a->head_q : 64), 1};
        rc = make_tensor_map(p.q, 3, qd, qs, qb, true, bf16 ? 1 : 0, &maps.k);
        if (rc != DA_OK) return rc;
        const uint64_t kd[2] = {576, kMapRows};
        const uint64_t ks[1] = {(uint64_t)p.k_row_stride * 2};
        // one CTA's keys of a tile, or a page when pages are shorter
        const uint32_t half = (uint32_t)(plan.tile_keys / 2);
        const uint32_t kb[2] = {64, (a->block_table && (uint32_t)a->page_size < half) ? (uint32_t)a->page_size : half};
        rc = make_tensor_map(p.k, 2, kd, ks, kb, true, bf16 ? 1 : 0, &maps.v);
        if (rc != DA_OK) return rc;
    }
    if (p.use_tmap) {
        // a quantised cache is mapped as bytes: a head's row is dim (8-bit) or dim / 2 (4-bit) of them
        const int kv_dt = kvq ? 2 : (bf16 ? 1 : 0);
        const int per_byte = kvq == DA_KV_INT4 ? 2 : 1;
        rc = make_kv_tensor_map(p.k, p.k_row_stride / per_byte, p.head_k, (int)a->dim / per_byte, box_keys, kv_dt, &maps.k);
        if (rc != DA_OK) return rc;
        rc = make_kv_tensor_map(p.v, p.v_row_stride / per_byte, p.head_k, (int)a->dim_v / per_byte, box_keys, kv_dt, &maps.v);
        if (rc != DA_OK) return rc;
    }
    cudaError_t e;
    if (g_prof_start) cudaEventRecord(g_prof_start, stream);
    switch (plan.shape) {
        case Shape::kD64: e = launch_split_d64(bf16, kvq, plan.heads, p, maps, stream); break;
        case Shape::kD96: e = launch_split_d96(bf16, kvq, plan.heads, p, maps, stream); break;
        case Shape::kD128: e = launch_split_d128(bf16, kvq, plan.heads, p, maps, stream); break;
        case Shape::kD256: e = launch_split_d256(bf16, kvq, plan.heads, p, maps, stream); break;
        case Shape::kMla: e = launch_split_mla_simt(bf16, plan.heads, p, maps, stream); break;
        case Shape::kGqaTc: e = launch_gqa_tc(bf16, a->dim == 96 ? 128 : (int)a->dim, p, tm_q, maps.k, maps.v, stream); break;
        case Shape::kGqaQuad: e = launch_gqa_quad(bf16, a->dim == 96 ? 128 : (int)a->dim, p, tm_q, maps.k, stream); break;
        case Shape::kMla2Sm: e = launch_mla_2sm(bf16, p, maps.k, maps.v, stream); break;
        default: e = cudaErrorInvalidValue; break;
    }
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "split kernel launch: %s", cudaGetErrorString(e));
    count_launch();
    if (g_prof_stop) cudaEventRecord(g_prof_stop, stream);

    if (plan.num_splits > 1) {
        MergeParams m;
        memset(&m, 0, sizeof(m));
        m.part_o = p.part_o;
        m.part_lse = p.part_lse;
        m.o = a->o;
        m.o_f32 = a->o_f32;
        m.lse = a->lse;
        m.cu_seq_k = a->cu_seq_k;
        m.part_stride_o = a->dim_v;
        m.row_stride_o = (long long)plan.num_splits * a->dim_v;
        m.part_stride_lse = 1;
        m.row_stride_lse = plan.num_splits;
        m.o_row_stride = p.o_row_stride;
        m.rows = a->batch * a->head_q;
        m.num_parts = plan.num_splits;
        m.dim_v = (int)a->dim_v;
        m.head_q = (int)a->head_q;
        m.chunk_keys = plan.chunk_keys;
        m.is_bf16 = bf16;
        e = launch_merge(m, stream, /*overlap=*/true);
        if (e != cudaSuccess) return fail(DA_ERR_CUDA, "merge kernel launch: %s", cudaGetErrorString(e));
    }
    return DA_OK;
}

int da_decode_fwd_host(const da_decode_args_t *h) {
    int rc = check_args(h);
    if (rc != DA_OK) return rc;
    if (!h->o) return fail(DA_ERR_INVALID_ARG, "o must be given");
    if (h->o_f32 || h->kv_pos_offset || h->kv_total_len || h->workspace || h->block_table) {
        return fail(DA_ERR_INVALID_ARG, "o_f32, kv_pos_offset, kv_total_len, workspace and block_table are device-only fields");
    }
    if (h->q_row_stride || h->k_row_stride || h->v_row_stride || h->o_row_stride) {
        return fail(DA_ERR_INVALID_ARG, "host tensors must be packed (row strides 0)");
    }
    DeviceState *st = nullptr;
    rc = device_state(&st);
    if (rc != DA_OK) return rc;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(h->stream);
    const int64_t total_k = h->cu_seq_k[h->batch];
    if (total_k < 0) return fail(DA_ERR_INVALID_ARG, "cu_seq_k must not decrease");
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t q_b = up((size_t)h->batch * h->head_q * h->dim * 2);
    const size_t kv_bits = h->kv_dtype == DA_KV_SAME_AS_Q ? 16 : (h->kv_dtype == DA_KV_INT4 ? 4 : 8);  // per cache element
    const size_t k_bytes = (size_t)total_k * h->head_k * h->dim * kv_bits / 8;
    const size_t v_bytes = h->v ? (size_t)total_k * h->head_k * h->dim_v * kv_bits / 8 : 0;
    const size_t k_b = up(k_bytes), v_b = up(v_bytes);
    const size_t o_b = up((size_t)h->batch * h->head_q * h->dim_v * 2);
    const size_t cu_b = up((size_t)(h->batch + 1) * 4);
    const size_t lse_b = h->lse ? up((size_t)h->batch * h->head_q * 4) : 0;
    const size_t need = q_b + k_b + v_b + o_b + cu_b + lse_b;
    // The staging buffer is one per device and may be regrown: the lock is held until this call has
    // drained its stream, so concurrent host-buffer calls on one device take turns.
    std::lock_guard<std::mutex> staging_lock(st->staging_mu);
    if (st->staging_bytes < need) {
        if (st->staging) {
            cudaDeviceSynchronize();
            cudaFree(st->staging);
            st->staging = nullptr;
            st->staging_bytes = 0;
        }
        cudaError_t e = cudaMalloc(&st->staging, need);
        if (e != cudaSuccess) return fail(DA_ERR_WORKSPACE, "cudaMalloc(%zu) staging: %s", need, cudaGetErrorString(e));
        st->staging_bytes = need;
    }
    char *base = static_cast<char *>(st->staging);
    da_decode_args_t d = *h;
    char *dq = base, *dk = dq + q_b, *dv = dk + k_b, *dout = dv + v_b, *dcu = dout + o_b, *dlse = dcu + cu_b;
    d.q = dq;
    d.k = dk;
    d.v = h->v ? dv : nullptr;
    d.o = dout;
    d.cu_seq_k = reinterpret_cast<const int32_t *>(dcu);
    d.lse = h->lse ? reinterpret_cast<float *>(dlse) : nullptr;
    cudaError_t e = cudaMemcpyAsync(dcu, h->cu_seq_k, (size_t)(h->batch + 1) * 4, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(dq, h->q, (size_t)h->batch * h->head_q * h->dim * 2, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(dk, h->k, k_bytes, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess && h->v)
        e = cudaMemcpyAsync(dv, h->v, v_bytes, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "host-to-device copy: %s", cudaGetErrorString(e));
    rc = da_decode_fwd(&d);
    if (rc != DA_OK) return rc;
    e = cudaMemcpyAsync(h->o, dout, (size_t)h->batch * h->head_q * h->dim_v * 2, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess && h->lse)
        e = cudaMemcpyAsync(h->lse, dlse, (size_t)h->batch * h->head_q * 4, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "device-to-host copy: %s", cudaGetErrorString(e));
    return DA_OK;
}

int da_merge_partials(const float *part_o, const float *part_lse, int32_t num_parts, int64_t rows, int32_t dim_v,
                      int64_t part_stride_o, int64_t row_stride_o, int64_t part_stride_lse, int64_t row_stride_lse,
                      void *o, float *o_f32, float *lse, int32_t is_bf16, void *stream) {
    if (!part_o || !part_lse || (!o && !o_f32)) return fail(DA_ERR_INVALID_ARG, "NULL partials or no output");
    if (num_parts <= 0 || rows < 0 || dim_v <= 0 || dim_v % 4 != 0 || dim_v > 512) {
        return fail(DA_ERR_INVALID_ARG, "num_parts > 0, rows >= 0, dim_v in (0, 512] and a multiple of 4 required");
    }
    if (((uintptr_t)part_o | (uintptr_t)o | (uintptr_t)o_f32) & 15u || part_stride_o % 4 || row_stride_o % 4) {
        return fail(DA_ERR_INVALID_ARG, "part_o, o, o_f32 must be 16-byte aligned, strides multiples of 4 floats");
    }
    MergeParams m;
    memset(&m, 0, sizeof(m));
    m.part_o = part_o;
    m.part_lse = part_lse;
    m.o = o;
    m.o_f32 = o_f32;
    m.lse = lse;
    m.part_stride_o = part_stride_o;
    m.row_stride_o = row_stride_o;
    m.part_stride_lse = part_stride_lse;
    m.row_stride_lse = row_stride_lse;
    m.rows = rows;
    m.num_parts = num_parts;
    m.dim_v = dim_v;
    m.head_q = 1;  // rows are addressed flat: o row i at o + i * dim_v
    m.o_row_stride = dim_v;
    m.is_bf16 = is_bf16;
    cudaError_t e = launch_merge(m, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "merge kernel launch: %s", cudaGetErrorString(e));
    return DA_OK;
}

void da_set_profile_events(void *start_event, void *stop_event) {
    g_prof_start = reinterpret_cast<cudaEvent_t>(start_event);
    g_prof_stop = reinterpret_cast<cudaEvent_t>(stop_event);
}

namespace da {
namespace {
// A wait that nothing ever satisfies, with a short bound: exercises the give-up path of the kernels'
// bounded waits (flag -> status word -> da_device_status) without harming the context.
__global__ void da_selftest_wait_kernel(int *status, long long max_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        const long long t0 = clock64();
        bool done = false;
        while (!done && clock64() - t0 < max_cycles) done = mbar_try_wait(&bar, 0);
        if (!done) atomicExch(status, kStatusWaitTimeout);
    }
}
}  // namespace
}  // namespace da

int da_selftest_wait_timeout(void *stream) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc != DA_OK) return rc;
    da_selftest_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(st->status_ptr, 2000000ll);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "selftest launch: %s", cudaGetErrorString(e));
    return DA_OK;
}

int da_device_status(void) {
    DeviceState *st = nullptr;
    int rc = device_state(&st);
    if (rc != DA_OK) return rc;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int word = 0;
    e = cudaMemcpy(&word, st->status_ptr, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(DA_ERR_CUDA, "cudaMemcpy(status): %s", cudaGetErrorString(e));
    if (word != kStatusOk) {
        const int zero[2] = {0, 0};
        cudaMemcpy(st->status_ptr, zero, sizeof(zero), cudaMemcpyHostToDevice);
        return fail(DA_ERR_TIMEOUT, "a kernel gave up a bounded wait (status word %d)", word);
    }
    return DA_OK;
}

const char *da_status_string(int status) {
    switch (status) {
        case DA_OK: return "ok";
        case DA_ERR_INVALID_ARG: return "invalid argument";
        case DA_ERR_UNSUPPORTED: return "unsupported shape";
        case DA_ERR_WORKSPACE: return "workspace too small or not allocatable";
        case DA_ERR_CUDA: return "CUDA runtime error";
        case DA_ERR_TIMEOUT: return "device wait timed out";
        default: return "unknown status";
    }
}

const char *da_last_error(void) { return g_err; }

uint64_t da_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
