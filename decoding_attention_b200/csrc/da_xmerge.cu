// Fused exchange + LSE merge for key-range sharding across GPUs (one process per GPU, NVLink peers).
//
// Each rank holds the partial result of its key range as a record (o fp32 [rows, dim_v], lse fp32
// [rows]).  Instead of an all-gather collective followed by a merge kernel, ONE kernel per rank
//   1. stores its record into slot `rank` of every peer's gather buffer with plain peer stores and
//      then raises a per-CTA flag there (system-scope release),
//   2. waits -- bounded -- until every peer's flag for this step has arrived in its own buffer,
//   3. merges the `world` records (its own straight from local memory) into the final rows.
// The gather buffers are symmetric allocations made by the host (torch symmetric memory); this
// file only sees the peers' base pointers.  Steps are numbered by `epoch`; slots and flags are
// double-buffered by epoch parity, which is enough because no rank can run more than one step ahead
// of another (it needs that rank's record of the step to finish its own merge).
// No multimem, no multicast, no collective library: peer stores and flag polling only.
// The reference is single-GPU and has nothing like it.
#include <cstring>

#include "../../include/decoding_attn_b200.h"
#include "da_internal.h"

namespace da {
namespace {

constexpr int kMaxWorld = 16;
constexpr int kRowsPerCta = 32;
constexpr int kMaxCtas = 256;
constexpr int kThreads = 256;

struct XMergeParams {
    float *bufs[kMaxWorld];  // gather buffer base of every rank (bufs[rank] is local)
    const float *rec;        // this rank's record: o [rows, dim_v] then lse [rows]
    void *o;
    float *lse;
    int *status;
    long long rows;
    long long slot_floats;   // floats per (parity, rank) slot = record size rounded up to 4
    int dim_v, world, rank, is_bf16;
    unsigned epoch;
    long long max_wait_cycles;  // bound of the flag poll, in SM clocks
};

// buffer layout (floats): [2 parities][world][slot_floats] records, then [2][world][kMaxCtas] flags (uint32)
__device__ __forceinline__ float *slot_ptr(float *base, const XMergeParams &p, int parity, int r) {
    return base + ((size_t)parity * p.world + r) * p.slot_floats;
}
__device__ __forceinline__ unsigned *flag_ptr(float *base, const XMergeParams &p, int parity, int r, int cta) {
    unsigned *flags = reinterpret_cast<unsigned *>(base + (size_t)2 * p.world * p.slot_floats);
    return flags + ((size_t)parity * p.world + r) * kMaxCtas + cta;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) da_xmerge_kernel(const XMergeParams p) {
    pdl_wait();  // the record comes from the kernel launched just before this one
    const int cta = blockIdx.x, tid = threadIdx.x;
    const long long r0 = (long long)cta * kRowsPerCta;
    const int nrows = (int)min((long long)kRowsPerCta, p.rows - r0);
    const int parity = (int)(p.epoch & 1u);
    const int dv4 = p.dim_v / 4;
    const float *rec_o = p.rec + r0 * p.dim_v;
    const float *rec_lse = p.rec + p.rows * p.dim_v + r0;
    __shared__ int s_ok;
    if (tid == 0) s_ok = 1;

    // 1. push this CTA's rows of the record to every peer
    for (int pr = 0; pr < p.world; ++pr) {
        if (pr == p.rank) continue;
        float *dst = slot_ptr(p.bufs[pr], p, parity, p.rank);
        float4 *dst_o = reinterpret_cast<float4 *>(dst + r0 * p.dim_v);
        for (int i = tid; i < nrows * dv4; i += kThreads) dst_o[i] = reinterpret_cast<const float4 *>(rec_o)[i];
        float *dst_lse = dst + p.rows * p.dim_v + r0;
        for (int i = tid; i < nrows; i += kThreads) dst_lse[i] = rec_lse[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.world && tid != p.rank) {
        // release: the record stores above are visible to the peer before the flag is
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag_ptr(p.bufs[tid], p, parity, p.rank, cta)), "r"(p.epoch)
                     : "memory");
    }

    // 2. bounded wait for every peer's flag of this step in the local buffer
    if (tid < p.world && tid != p.rank) {
        const unsigned *f = flag_ptr(p.bufs[p.rank], p, parity, tid, cta);
        const long long t0 = clock64();
        bool got = false;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == p.epoch) {
                got = true;
                break;
            }
            if (clock64() - t0 > p.max_wait_cycles) break;
        }
        if (!got) {
            s_ok = 0;
            atomicExch(p.status, kStatusWaitTimeout);
        }
    }
    __syncthreads();
    if (!s_ok) return;

    // 3. merge: o = sum_r w_r o_r / sum_r w_r, w_r = exp(lse_r - max lse)
    float *mine = p.bufs[p.rank];
    for (int i = tid; i < nrows * dv4; i += kThreads) {
        const int row = i / dv4, c = i % dv4;
        float mx = -INFINITY;
        for (int r = 0; r < p.world; ++r) {
            const float x = (r == p.rank) ? rec_lse[row] : __ldcg(slot_ptr(mine, p, parity, r) + p.rows * p.dim_v + r0 + row);
            mx = fmaxf(mx, x);
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float wsum = 0.f;
        if (mx > -INFINITY) {
            for (int r = 0; r < p.world; ++r) {
                const float *src = (r == p.rank) ? p.rec : slot_ptr(mine, p, parity, r);
                const float x = (r == p.rank) ? rec_lse[row] : __ldcg(src + p.rows * p.dim_v + r0 + row);
                const float w = exp2f((x - mx) * kLog2e);
                const float4 v = (r == p.rank) ? reinterpret_cast<const float4 *>(rec_o)[i]
                                               : __ldcg(reinterpret_cast<const float4 *>(src + r0 * p.dim_v) + i);
                acc.x = fmaf(w, v.x, acc.x);
                acc.y = fmaf(w, v.y, acc.y);
                acc.z = fmaf(w, v.z, acc.z);
                acc.w = fmaf(w, v.w, acc.w);
                wsum += w;
            }
            const float inv = 1.0f / wsum;
            acc.x *= inv, acc.y *= inv, acc.z *= inv, acc.w *= inv;
        }
        T *dst = reinterpret_cast<T *>(p.o) + (size_t)(r0 + row) * p.dim_v + c * 4;
        dst[0] = from_float<T>(acc.x);
        dst[1] = from_float<T>(acc.y);
        dst[2] = from_float<T>(acc.z);
        dst[3] = from_float<T>(acc.w);
        if (p.lse && c == 0) p.lse[r0 + row] = (mx > -INFINITY) ? mx + log2f(wsum) * kLn2 : -INFINITY;
    }
}

}  // namespace

int xmerge_status_ptr(int **out);  // da_api.cu

}  // namespace da

extern "C" size_t da_exchange_buffer_bytes(int32_t world, int64_t rows, int32_t dim_v) {
    if (world <= 0 || rows <= 0 || dim_v <= 0) return 0;
    const size_t slot = ((size_t)rows * ((size_t)dim_v + 1) + 3) / 4 * 4;
    return (2 * (size_t)world * slot + 2 * (size_t)world * da::kMaxCtas) * sizeof(float);
}

extern "C" int da_exchange_merge(const float *rec, void *const *peer_bufs, int32_t world, int32_t rank, int64_t rows,
                                 int32_t dim_v, uint32_t epoch, void *o, float *lse, int32_t is_bf16, void *stream) {
    return da_exchange_merge_bounded(rec, peer_bufs, world, rank, rows, dim_v, epoch, o, lse, is_bf16, stream, 0);
}

extern "C" int da_exchange_merge_bounded(const float *rec, void *const *peer_bufs, int32_t world, int32_t rank,
                                         int64_t rows, int32_t dim_v, uint32_t epoch, void *o, float *lse,
                                         int32_t is_bf16, void *stream, int64_t max_wait_cycles) {
    using namespace da;
    if (max_wait_cycles < 0) return report_error(DA_ERR_INVALID_ARG, "max_wait_cycles must not be negative");
    if (!rec || !peer_bufs || !o) return report_error(DA_ERR_INVALID_ARG, "rec, peer_bufs and o must not be NULL");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) {
        return report_error(DA_ERR_INVALID_ARG, "world must be 1..16 and rank inside it");
    }
    if (rows <= 0 || rows > (int64_t)kMaxCtas * kRowsPerCta || dim_v <= 0 || dim_v % 4 != 0 || dim_v > 512) {
        return report_error(DA_ERR_INVALID_ARG, "rows must be 1..8192, dim_v a multiple of 4 up to 512");
    }
    if (epoch == 0) return report_error(DA_ERR_INVALID_ARG, "epoch starts at 1 (flags are zero-initialised)");
    XMergeParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || ((uintptr_t)peer_bufs[r] & 15u)) {
            return report_error(DA_ERR_INVALID_ARG, "every peer buffer must be a 16-byte aligned device pointer");
        }
        p.bufs[r] = static_cast<float *>(peer_bufs[r]);
    }
    p.rec = rec;
    p.o = o;
    p.lse = lse;
    int rc = xmerge_status_ptr(&p.status);
    if (rc != DA_OK) return rc;
    p.rows = rows;
    p.slot_floats = (rows * ((long long)dim_v + 1) + 3) / 4 * 4;
    p.dim_v = dim_v;
    p.world = world;
    p.rank = rank;
    p.is_bf16 = is_bf16;
    p.epoch = epoch;
    p.max_wait_cycles = max_wait_cycles > 0 ? max_wait_cycles : kMaxWaitCycles;
    const unsigned ctas = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // Launched for overlap with the preceding kernel of the stream (it waits for that kernel's results itself).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = is_bf16 ? cudaLaunchKernelEx(&cfg, da_xmerge_kernel<__nv_bfloat16>, p)
                            : cudaLaunchKernelEx(&cfg, da_xmerge_kernel<__half>, p);
    count_launch();
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return report_error(DA_ERR_CUDA, cudaGetErrorString(e));
    return DA_OK;
}
