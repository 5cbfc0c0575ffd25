// Latent-KV (MLA) decode attention on the sm_100a tensor cores, two CTAs per key range working as a
// thread-block cluster: tcgen05.mma with accumulators in tensor memory (TMEM), operands staged by
// TMA, partial scores exchanged through distributed shared memory.
//
// Shape: 128 query heads share one KV head whose rows hold 576 values; V is the first 512 of them
// (the reference runs this shape through its generic kernel, one CTA per query head:
// csrc/kernel/decoding_attn/decoding_fwd_hd576_hdv512.cu:9-17, so every K row is fetched 128
// times).  The 128 heads are the M dimension of two dense contractions per 64-key tile:
//     S[128 x 64]   = Q[128 x 576] . K_tile[64 x 576]^T
//     O[128 x 512] += P[128 x 64]  . V_tile[64 x 512]          (V = columns 0..511 of the K tile)
// One SM cannot hold this: the fp32 output alone fills the 512 TMEM columns, and Q (144 KB) plus
// enough K tiles in flight overflow shared memory.  So the pair splits BOTH contractions:
//   * CTA c owns output columns [256c, 256c+256)  -> needs V columns of 64-wide blocks 4c..4c+3;
//   * CTA 0 contracts S over dims [0, 320) (blocks 0..4), CTA 1 over [320, 576) (blocks 5..8).
// Each CTA therefore streams five 64-wide column blocks of every K row (CTA 0: blocks 0..4, CTA 1:
// blocks 4..8 -- block 4 is fetched twice, 1.11x in total, the second fetch hits L2), keeps its
// share of Q entirely in TMEM (A operand from TMEM), and computes a partial S.  The two partial
// S tiles are swapped row by row through the peer's shared memory and added, after which both CTAs
// hold the same full S and run identical online softmax on it.  No multicast, no cta_group::2.
//
// Warp roles (192 threads): warps 0-3 = exchange/softmax/epilogue, thread r owns TMEM lane r =
// head r (row maxima, sums, rescale of O and the exchange are all row-local); warp 4 = TMA
// producer; warp 5 = TMEM allocation and MMA issue (whole warp walks the unrolled issue sequence,
// one elected lane issues).  Online softmax with a lazy reference max (raised only when exceeded
// by 2^8).  Every wait is bounded; on expiry the CTA records kStatusWaitTimeout, still meets its
// peer at the final cluster barrier and frees its TMEM.
#include <type_traits>

#include "da_internal.h"
#include "da_tcgen05.cuh"

namespace da {
namespace {

constexpr int kHeads = 128;
constexpr int kDim = 576;
constexpr int kDimV = 512;
constexpr int kHalfV = 256;                           // output columns per CTA
constexpr int kTile = 64;                             // keys per tile
constexpr int kStages = 3;                            // K tiles in flight per CTA
constexpr int kLocalBlocks = 5;                       // 64-wide column blocks a CTA streams per key
constexpr int kKBlockBytes = kTile * 128;             // [64 keys x 64 dims], 128-byte swizzle
constexpr int kKStageBytes = kLocalBlocks * kKBlockBytes;
constexpr int kPBytes = kHeads * kTile * 2;           // P tile, core-matrix (no swizzle) K-major
constexpr int kXRowBytes = kTile * 4;                 // one row of a partial S tile (fp32)
constexpr int kXBytes = kHeads * kXRowBytes;          // receive buffer (written by the peer's bulk copy) and send staging
constexpr int kOffK = 0;
constexpr int kOffP = kOffK + kStages * kKStageBytes;
constexpr int kOffX = kOffP + 2 * kPBytes;            // peer's partial S lands here; the full S is formed in place
constexpr int kOffY = kOffX + kXBytes;                // this CTA's partial S, source of the copy to the peer
constexpr int kOffBar = kOffY + kXBytes;
// q_tmem, k_full/k_empty[kStages], s_full, s_empty, p_full[2], pv_done[2], x_full, x_free, s_ready
constexpr int kNumBars = 1 + 2 * kStages + 2 + 2 + 2 + 3;
constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;  // + tmem slot/abort flag + alignment slack
constexpr int kThreads = 320;   // warps 0-3 softmax, 4-7 exchange, 8 TMA producer, 9 MMA issuer
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kTmemCols = 512;
constexpr int kColS = 0;      // 64 columns
constexpr int kColO = 64;     // 256 columns
constexpr int kColQ = 320;    // up to 5 blocks x 32 columns: this CTA's share of Q, packed 16-bit pairs
static_assert(kColQ + kLocalBlocks * 32 <= kTmemCols, "TMEM budget");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
constexpr float kRescaleThreshold = 8.0f;

#ifdef DA_MLA_PROFILE
// Development aid (not compiled into the shipped library): cycles CTA (0,0,0) spends in each step.
__device__ long long g_mla_prof[64];
#define PROF_DECL long long prof_t0 = 0, prof_acc[16] = {}; (void)prof_t0
#define PROF_BEGIN() prof_t0 = clock64()
#define PROF_END(slot) do { long long now_ = clock64(); prof_acc[(slot) & 15] += now_ - prof_t0; prof_t0 = now_; } while (0)
#define PROF_FLUSH(base) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0) { for (int i_ = 0; i_ < 16; ++i_) g_mla_prof[(base) + i_] += prof_acc[i_]; } } while (0)
#else
#define PROF_DECL
#define PROF_BEGIN()
#define PROF_END(slot)
#define PROF_FLUSH(base)
#endif

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
da_mla_pair_kernel(const SplitParams p, const __grid_constant__ CUtensorMap tm_k) {
    extern __shared__ uint8_t smem_raw[];
    // The offset of every buffer inside the CTA's shared window is the same in both CTAs of the pair
    // (remote addresses are formed from local ones): both round the same base up alike.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const uint32_t rank = cluster_ctarank();  // 0 or 1: which half of the output columns / of the contraction
    const int split = blockIdx.y;
    const int b = p.batch_order ? p.batch_order[blockIdx.z] : (int)blockIdx.z;
    pdl_launch_dependents();  // the merge kernel may be scheduled behind this grid's last CTAs
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq_begin = p.cu_seq_k[b];
    const int len = p.cu_seq_k[b + 1] - seq_begin;
    const int k_begin = split * p.chunk_keys;
    const int k_end = min(len, k_begin + p.chunk_keys);
    T *o_out = reinterpret_cast<T *>(p.o);
    // Both CTAs of a pair see the same key range, so they leave together here.
    if (k_begin >= k_end) {
        if (p.num_splits == 1) {  // empty sequence: zero row, LSE = -inf
            for (int idx = tid; idx < kHeads * kHalfV; idx += kThreads) {
                const int h = idx / kHalfV, d = (int)rank * kHalfV + idx % kHalfV;
                if (o_out) o_out[(size_t)b * p.o_row_stride + (size_t)h * kDimV + d] = from_float<T>(0.0f);
                if (p.o_f32) p.o_f32[((size_t)b * p.head_q + h) * kDimV + d] = 0.0f;
            }
            if (p.lse && rank == 0 && tid < kHeads) p.lse[(size_t)b * p.head_q + tid] = -INFINITY;
        }
        return;
    }
    const int n_tiles = (k_end - k_begin + kTile - 1) / kTile;

    uint8_t *k_s = smem + kOffK;
    uint8_t *p_s = smem + kOffP;
    uint8_t *x_s = smem + kOffX;
    uint8_t *y_s = smem + kOffY;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    uint64_t *q_tmem = bars;
    uint64_t *k_full = bars + 1;
    uint64_t *k_empty = k_full + kStages;
    uint64_t *s_full = k_empty + kStages;
    uint64_t *s_empty = s_full + 1;
    uint64_t *p_full = s_empty + 1;
    uint64_t *pv_done = p_full + 2;
    uint64_t *x_full = pv_done + 2;   // the peer has written its partial S of a tile into x_s
    uint64_t *x_free = x_full + 1;    // the peer has read what this CTA wrote into the peer's x_s
    uint64_t *s_ready = x_free + 1;   // the full S of a tile is in x_s
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (tid == 0) {
        mbar_init(q_tmem, kHeads);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_empty, kHeads);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&p_full[s], kHeads);
            mbar_init(&pv_done[s], 1);
        }
        mbar_init(x_full, 1);       // one arrive.expect_tx from the peer per tile, then the copy's bytes
        mbar_init(x_free, 1);       // one remote arrival per tile (remote arrivals are expensive: keep them few)
        mbar_init(s_ready, kHeads);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kMmaWarp) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anybody arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr uint32_t kIdescQK = instr_desc(kFmt, 0, kHeads, kTile);
    constexpr uint32_t kIdescPV = instr_desc(kFmt, 1, kHeads, kHalfV);
    const int first_block = (int)rank * 4;   // global index of local block 0 (CTA 0: 0, CTA 1: 4)
    const int qk_begin = (int)rank;          // local blocks [qk_begin, 5) enter S (CTA 1 skips block 4)
    bool ok = true;

    if (warp == kProducerWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) tma_prefetch_desc(&tm_k);
        const T *k_g = reinterpret_cast<const T *>(p.k) + first_block * 64;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int st = t % kStages;
            const uint32_t ph = (uint32_t)(t / kStages) & 1u;
            const int key0 = k_begin + t * kTile;
            const int rows = min(kTile, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            if (t >= kStages) ok = mbar_wait(&k_empty[st], ph ^ 1u, abort_flag);
            if (!ok) break;
            uint8_t *dst = k_s + st * kKStageBytes;
            if (rows == kTile) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(&k_full[st], kKStageBytes);
                    for (int j = 0; j < kLocalBlocks; ++j) {
                        tma_load_2d(dst + j * kKBlockBytes, &tm_k, (first_block + j) * 64, (int)tok0, &k_full[st]);
                    }
                }
            } else {
                // Ragged tail: plain loads into the 128-byte-swizzled layout, rows past the end zeroed
                // (the tensor map must not be asked for rows beyond the sequence).
                constexpr int kChunks = kLocalBlocks * 8;  // 16-byte chunks per row
                for (int i = lane; i < kTile * kChunks; i += 32) {
                    const int r = i / kChunks, c = i % kChunks;
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (r < rows) v = *reinterpret_cast<const uint4 *>(k_g + (tok0 + r) * p.k_row_stride + c * 8);
                    const int j = c >> 3, cc = c & 7;
                    *reinterpret_cast<uint4 *>(dst + j * kKBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&k_full[st]);
            }
            __syncwarp();
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        const uint32_t leader = elect_one();
        const uint32_t k_addr = smem_u32(k_s), p_addr = smem_u32(p_s);
        // Descriptors differ between tiles only in the start-address field (low 14 bits, 16-byte units).
        const uint64_t k_desc0 = smem_desc(k_addr, 16, 1024, 2);            // K-major, 8-row groups 1 KB apart
        const uint64_t v_desc0 = smem_desc(k_addr, kKBlockBytes, 1024, 2);  // MN-major: 64-col blocks LBO apart
        const uint64_t p_desc0 = smem_desc(p_addr, kHeads * 16, 128, 0);    // core matrices, 8-key chunks 2 KB apart
        const uint32_t q_tmem_addr = tmem_base + kColQ;
        auto issue_qk = [&](int t) {
            const uint64_t kd = k_desc0 + (uint64_t)(((t % kStages) * kKStageBytes) >> 4);
            const uint32_t d = tmem_base + kColS;
#pragma unroll
            for (int j = 0; j < kLocalBlocks; ++j) {
                if (j >= qk_begin) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // Q block (j - qk_begin) of this CTA sits in TMEM columns [32 (j - qk_begin), +32).
                        umma_ts(d, q_tmem_addr + (j - qk_begin) * 32 + ks * 8,
                                kd + (uint64_t)((j * kKBlockBytes + ks * 32) >> 4), kIdescQK,
                                (j > qk_begin || ks > 0) ? 1u : 0u, leader);
                    }
                }
            }
            umma_commit(s_full, leader);
        };
        ok = mbar_wait(q_tmem, 0, abort_flag);
        if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
        if (ok) {
            tc_fence_after();
            issue_qk(0);
        }
        PROF_DECL;
        for (int t = 0; t < n_tiles && ok; ++t) {
            PROF_BEGIN();
            if (t + 1 < n_tiles) {
                const int t1 = t + 1;
                ok = mbar_wait(&k_full[t1 % kStages], (uint32_t)(t1 / kStages) & 1u, abort_flag);
                PROF_END(10);
                if (ok) ok = mbar_wait(s_empty, (uint32_t)t & 1u, abort_flag);  // S of tile t has been read out
                PROF_END(11);
                if (!ok) break;
                tc_fence_after();
                issue_qk(t1);
                PROF_END(12);
            }
            ok = mbar_wait(&p_full[t & 1], (uint32_t)(t / 2) & 1u, abort_flag);
            PROF_END(13);
            if (!ok) break;
            tc_fence_after();
            const int st = t % kStages;
            const uint64_t pd = p_desc0 + (uint64_t)(((t & 1) * kPBytes) >> 4);
            const uint64_t vd = v_desc0 + (uint64_t)((st * kKStageBytes) >> 4);
#pragma unroll
            for (int ks = 0; ks < kTile / 16; ++ks) {
                umma_ss(tmem_base + kColO, pd + (uint64_t)((ks * 2 * (kHeads * 16)) >> 4),
                        vd + (uint64_t)((ks * 16 * 128) >> 4), kIdescPV, (t | ks) ? 1u : 0u, leader);
            }
            umma_commit(&k_empty[st], leader);
            umma_commit(&pv_done[t & 1], leader);
            PROF_END(14);
        }
        PROF_FLUSH(0);
        __syncwarp();
    } else if (warp >= 4) {
        // ------- exchange warps: thread (tid - 128) <-> TMEM lane r <-> head r -------
        // Per tile: read this CTA's partial S row from TMEM, stage it, one bulk copy ships the whole
        // 32 KB tile into the peer's receive buffer; when the peer's tile has landed here, add the own
        // row in place: x_s then holds the full S for the softmax warps.
        const int r = tid - 128;
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp - 4) * 32) << 16);
        const uint32_t peer = rank ^ 1u;
        const uint32_t x_remote = map_to_cta(smem_u32(x_s), peer);
        const uint32_t x_full_remote = map_to_cta(smem_u32(x_full), peer);
        // 16-byte chunk c of row r sits at c * (128 * 16) + r * 16 in both buffers: warp-wide accesses
        // are contiguous and conflict-free.
        uint8_t *y_row = y_s + r * 16;
        uint8_t *x_row = x_s + r * 16;
        uint32_t buf[32];
        {
            // This CTA's share of head r's query (CTA 0: dims 0..319, CTA 1: dims 320..575) goes to TMEM
            // as packed 16-bit pairs: the A operand of S = Q K^T.
            const int nq = kLocalBlocks - (int)rank;
            const T *q_row = reinterpret_cast<const T *>(p.q) + (size_t)b * p.q_row_stride + (size_t)r * kDim + rank * 320;
#pragma unroll 1
            for (int kb = 0; kb < nq; ++kb) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(q_row + kb * 64 + j * 8);
                    buf[4 * j] = v.x, buf[4 * j + 1] = v.y, buf[4 * j + 2] = v.z, buf[4 * j + 3] = v.w;
                }
                tmem_st32(lane_base + kColQ + kb * 32, buf);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(q_tmem);
        }
        PROF_DECL;
        for (int t = 0; t < n_tiles; ++t) {
            PROF_BEGIN();
            ok = __all_sync(0xffffffffu, mbar_wait(s_full, (uint32_t)t & 1u, abort_flag));
            PROF_END(0);
            float s[kTile];
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < kTile; c0 += 32) {
                    tmem_ld32(lane_base + kColS + c0, buf);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) s[c0 + j] = __uint_as_float(buf[j]);
                }
                tc_fence_before();
                mbar_arrive(s_empty);
            }
            PROF_END(1);
            // The peer has read tile t-1 out of its receive buffer, so the copy that fed it is over
            // and the staging buffer may be rewritten.
            if (ok && t >= 1) ok = mbar_wait_cluster(x_free, (uint32_t)(t - 1) & 1u, abort_flag);
            PROF_END(2);
            if (ok) {
#pragma unroll
                for (int c = 0; c < kTile / 4; ++c) {
                    *reinterpret_cast<float4 *>(y_row + c * (kHeads * 16)) =
                        make_float4(s[4 * c], s[4 * c + 1], s[4 * c + 2], s[4 * c + 3]);
                }
                fence_proxy_async();
            }
            // Every exchange thread reaches this barrier, also after a wait has run out somewhere
            // (the abort flag then ends the loop for all of them just behind it).
            named_bar_sync(2, 128);
            if (*abort_flag) {
                ok = false;
                break;
            }
            if (r == 0) {
                mbar_arrive_expect_tx_remote(x_full_remote, kXBytes);
                bulk_copy_s2peer(x_remote, y_s, kXBytes, x_full_remote);
            }
            PROF_END(3);
            ok = mbar_wait_cluster(x_full, (uint32_t)t & 1u, abort_flag);
            PROF_END(4);
            if (!ok) break;
#pragma unroll
            for (int c = 0; c < kTile / 4; ++c) {
                float4 *px = reinterpret_cast<float4 *>(x_row + c * (kHeads * 16));
                float4 o4 = *px;
                o4.x += s[4 * c], o4.y += s[4 * c + 1], o4.z += s[4 * c + 2], o4.w += s[4 * c + 3];
                *px = o4;
            }
            mbar_arrive(s_ready);
            PROF_END(5);
        }
        PROF_FLUSH(32);
    } else {
        // ------- softmax / epilogue warps: thread r <-> TMEM lane r <-> head r -------
        const int r = tid;
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        const uint32_t x_free_remote = map_to_cta(smem_u32(x_free), rank ^ 1u);
        const uint8_t *x_row = x_s + r * 16;
        const float slope2 = p.is_alibi ? exp2f(-8.0f * (float)(r + 1) / (float)p.head_q) * kLog2e : 0.0f;
        const int pos_shift = (p.kv_pos_offset ? p.kv_pos_offset[b] : 0) - ((p.kv_total_len ? p.kv_total_len[b] : len) - 1);
        float m_ref = -INFINITY, l = 0.0f;
        uint32_t buf[32];
        PROF_DECL;
        for (int t = 0; t < n_tiles; ++t) {
            const int key0 = k_begin + t * kTile;
            const int rows = min(kTile, k_end - key0);
            PROF_BEGIN();
            ok = mbar_wait(s_ready, (uint32_t)t & 1u, abort_flag);
            PROF_END(16);
            if (!ok) break;
            float s[kTile];
#pragma unroll
            for (int c = 0; c < kTile / 4; ++c) {
                const float4 o4 = *reinterpret_cast<const float4 *>(x_row + c * (kHeads * 16));
                s[4 * c] = o4.x, s[4 * c + 1] = o4.y, s[4 * c + 2] = o4.z, s[4 * c + 3] = o4.w;
            }
            named_bar_sync(3, 128);             // all 128 rows have been read ...
            if (r == 0) mbar_arrive_remote(x_free_remote);  // ... the peer may send its next tile
            PROF_END(21);
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < kTile; ++j) {
                const float x = s[j] * p.scale_log2 + slope2 * (float)(key0 + j + pos_shift);
                s[j] = (j < rows) ? x : -INFINITY;
                mx = fmaxf(mx, s[j]);
            }
            const bool raise = mx > m_ref + kRescaleThreshold;
            float alpha = 1.0f;
            if (raise) {
                alpha = exp2f(m_ref - mx);  // 0 on the first tile
                m_ref = mx;
                l *= alpha;
            }
            PROF_END(22);
            if (t >= 2) {
                // The P buffer of this tile was last read by the P.V of tile t-2.
                ok = mbar_wait(&pv_done[t & 1], ((uint32_t)(t / 2) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
            }
            PROF_END(23);
            if (t >= 1 && __any_sync(0xffffffffu, raise)) {
                // Rare: the reference max of some row in this warp moved.  O must be idle (P.V of tile
                // t-1 complete) while its rows are rescaled in place.
                ok = mbar_wait(&pv_done[(t - 1) & 1], (uint32_t)((t - 1) / 2) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < kHalfV / 32; ++c) {
                    tmem_ld32(lane_base + kColO + c * 32, buf);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) buf[j] = __float_as_uint(__uint_as_float(buf[j]) * alpha);
                    tmem_st32(lane_base + kColO + c * 32, buf);
                }
                tmem_wait_st();
            }
            // P = exp2(S - m_ref), rounded to the input type, into the A-operand layout.
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < kTile / 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = exp2f(s[c * 8 + 2 * j] - m_ref), p1 = exp2f(s[c * 8 + 2 * j + 1] - m_ref);
                    sum += p0 + p1;
                    if (std::is_same<T, __nv_bfloat16>::value) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                        w[j] = *reinterpret_cast<uint32_t *>(&h);
                    } else {
                        __half2 h = __floats2half2_rn(p0, p1);
                        w[j] = *reinterpret_cast<uint32_t *>(&h);
                    }
                }
                *reinterpret_cast<uint4 *>(p_s + (t & 1) * kPBytes + c * (kHeads * 16) + r * 16) =
                    make_uint4(w[0], w[1], w[2], w[3]);
            }
            l += sum;
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&p_full[t & 1]);
            PROF_END(24);
#ifdef DA_MLA_PROFILE
            if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0) g_mla_prof[63] += 1;
#endif
        }
        if (warp == 0) PROF_FLUSH(16);
        if (ok) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], (uint32_t)((n_tiles - 1) / 2) & 1u, abort_flag);
        if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l;
            const float lse = (m_ref + log2f(l)) * kLn2;
            const size_t row = ((size_t)b * p.head_q + r) * p.num_splits + split;
#pragma unroll 1
            for (int c = 0; c < kHalfV / 32; ++c) {
                tmem_ld32(lane_base + kColO + c * 32, buf);
                tmem_wait_ld();
                const int d0 = (int)rank * kHalfV + c * 32;
                if (p.num_splits > 1) {
                    float4 *dst = reinterpret_cast<float4 *>(p.part_o + row * kDimV + d0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        dst[j] = make_float4(__uint_as_float(buf[4 * j]) * inv, __uint_as_float(buf[4 * j + 1]) * inv,
                                             __uint_as_float(buf[4 * j + 2]) * inv, __uint_as_float(buf[4 * j + 3]) * inv);
                    }
                } else {
                    if (o_out) {
                        uint4 *dst = reinterpret_cast<uint4 *>(o_out + (size_t)b * p.o_row_stride + (size_t)r * kDimV + d0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            alignas(16) T tmp[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) tmp[e] = from_float<T>(__uint_as_float(buf[8 * j + e]) * inv);
                            dst[j] = *reinterpret_cast<uint4 *>(tmp);
                        }
                    }
                    if (p.o_f32) {
                        float *dst = p.o_f32 + ((size_t)b * p.head_q + r) * kDimV + d0;
#pragma unroll
                        for (int j = 0; j < 32; ++j) dst[j] = __uint_as_float(buf[j]) * inv;
                    }
                }
            }
            if (rank == 0) {
                if (p.num_splits > 1) {
                    p.part_lse[row] = lse;
                } else if (p.lse) {
                    p.lse[(size_t)b * p.head_q + r] = lse;
                }
            }
            tc_fence_before();
        }
    }

    if (!ok && lane == 0) atomicExch(p.status, kStatusWaitTimeout);
    __syncthreads();
    // The peer may still be writing into this CTA's exchange buffer or arriving on its barriers:
    // nobody leaves (and no shared memory is released) before both CTAs are here.
    cluster_sync_all();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace

#ifdef DA_MLA_PROFILE
extern "C" void da_debug_mla_prof(long long *out, int reset) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, g_mla_prof, sizeof(long long) * 64);
    if (reset) {
        long long z[64] = {};
        cudaMemcpyToSymbol(g_mla_prof, z, sizeof(z));
    }
}
#endif

SplitVariantInfo split_info_mla_pair() { return {kTile, kHeads, 1}; }

// tm_k: rank-2 map over the latent cache [rows][576], box {64, 64 keys}, 128-byte swizzle.
// Grid (2, splits, batch) in clusters of two along x: the two CTAs of a key range.
cudaError_t launch_mla_pair(bool bf16, const SplitParams &p, const CUtensorMap &tm_k, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !attr_set[dev]) {
        err = cudaFuncSetAttribute(da_mla_pair_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (err != cudaSuccess) return err;
        err = cudaFuncSetAttribute(da_mla_pair_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kSmemBytes);
        if (err != cudaSuccess) return err;
        attr_set[dev] = true;
    }
    dim3 grid(2, p.num_splits, p.batch);
    if (bf16) {
        da_mla_pair_kernel<__nv_bfloat16><<<grid, kThreads, kSmemBytes, stream>>>(p, tm_k);
    } else {
        da_mla_pair_kernel<__half><<<grid, kThreads, kSmemBytes, stream>>>(p, tm_k);
    }
    return cudaGetLastError();
}

}  // namespace da
