// CUDA-core split-KV decode attention for MHA / GQA / MQA (and a slow all-shapes path for the
// latent-KV shape), sm_100a.
//
// It replaces the reference's single kernel dmha_fwd_kernel
// (csrc/kernel/decoding_attn/decoding_fwd_kernel.h:13-236), which runs one CTA per (batch, query
// head), materialises the whole score row in shared memory and re-reads K/V once per query head.
// Here one CTA owns (sequence, KV head, head chunk, key range):
//   * a producer warp streams K and V tiles of that key range into a ring of shared-memory stages
//     with per-row cp.async.bulk copies (TMA engine) that complete on mbarriers;
//   * NWARPS consumer warps are cut into groups of LANES lanes.  A group owns every NG-th key of a
//     tile; each lane owns NCH 16-byte chunks of the head dimension for all G query heads of the
//     CTA, so a K/V element is unpacked to fp32 once and used G times;
//   * per-lane partial dot products are reduce-scattered inside the group with xor shuffles, the
//     softmax is kept online per group in fp32 (no CTA-wide synchronisation per tile), and the
//     groups are merged once at the end;
//   * the CTA writes either the final row (one split) or a normalised fp32 partial plus its LSE
//     for the merge kernel (da_merge.cu).
// Everything that waits does so with a bound (mbar_wait) and reports through the status word.
#pragma once

#include "da_common.cuh"

namespace da {

// KVQ_: how K and V are stored (q and o keep the 16-bit type T): 0 = as T, 1 = FP8 e4m3 bytes, 2 = signed 8-bit
// integers, 3 = signed 4-bit integers, two per byte (low nibble first).  A lane always owns eight elements at a time.
template <typename T_, int D_, int DV_, int LANES_, int G_, int KPT_, int NWARPS_, int STAGES_, bool MLA_, int MINB_ = 1,
          int KVQ_ = 0>
struct SplitCfg {
    using T = T_;
    static constexpr int KVQ = KVQ_;
    static constexpr int KV_BITS = KVQ_ == 0 ? 16 : (KVQ_ == 3 ? 4 : 8);  // bits per K / V element
    static constexpr int CHUNK_BYTES = KV_BITS;        // eight elements: what one lane reads at a time
    static constexpr int D = D_, DV = DV_, LANES = LANES_, G = G_, KPT = KPT_, NWARPS = NWARPS_, STAGES = STAGES_;
    static constexpr bool MLA = MLA_;
    static constexpr int MINB = MINB_;             // resident CTAs per SM the register budget must allow              // V is the first DV elements of each K row
    static constexpr int NCH = D / (8 * LANES);    // 16-byte chunks of a K row per lane
    static constexpr int NCHV = DV / (8 * LANES);  // 16-byte chunks of a V row per lane
    static constexpr int GPW = 32 / LANES;         // groups per warp
    static constexpr int NG = NWARPS * GPW;        // groups per CTA
    static constexpr int TILE = NG * KPT;          // keys per pipeline stage
    static constexpr int NV = KPT * G;             // scores per group per tile
    static constexpr int RV = NV >= LANES ? NV / LANES : 1;   // scores a lane holds after the reduce-scatter
    static constexpr int REP = NV >= LANES ? 1 : LANES / NV;  // lanes holding the same score
    static constexpr int K_ROW_BYTES = D * KV_BITS / 8, V_ROW_BYTES = DV * KV_BITS / 8;
    static constexpr int K_TILE_BYTES = TILE * K_ROW_BYTES;
    static constexpr int V_TILE_BYTES = MLA ? 0 : TILE * V_ROW_BYTES;
    static constexpr int THREADS = (NWARPS + 1) * 32;
    static constexpr int CONSUMERS = NWARPS * 32;
    // shared memory map
    static constexpr int OFF_K = 0;
    static constexpr int OFF_V = OFF_K + STAGES * K_TILE_BYTES;
    static constexpr int PIPE_BYTES = OFF_V + STAGES * V_TILE_BYTES;
    static constexpr int MERGE_BYTES = NG * G * (DV + 2) * 4;  // end-of-CTA merge reuses the stage buffers
    static constexpr int OFF_P = (PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES);
    static constexpr int P_BYTES = NG * NV * 4;
    static constexpr int OFF_BAR = (OFF_P + P_BYTES + 15) / 16 * 16;
    static constexpr int SMEM_BYTES = OFF_BAR + 4 * STAGES * 8 + 16;
    static_assert(D % (8 * LANES) == 0 && DV % (8 * LANES) == 0, "head dims must split into 16-byte chunks per lane");
    static_assert((LANES & (LANES - 1)) == 0 && LANES <= 32, "LANES must be a power of two");
    static_assert((NV & (NV - 1)) == 0, "KPT*G must be a power of two");
    static_assert(!MLA || DV <= D, "latent-KV: V is a prefix of the K row");
    static_assert(K_ROW_BYTES % 16 == 0 && V_ROW_BYTES % 16 == 0, "rows are copied in 16-byte units");
};

constexpr int ilog2(int x) { return x <= 1 ? 0 : 1 + ilog2(x / 2); }

// Sum v[] over the LANES lanes of a group.  While more than one value is left each step also
// halves the number of values a lane keeps (reduce-scatter), so NV values cost about NV shuffles
// instead of NV*log2(LANES).  Afterwards lane c holds the totals of indices (c/REP)*RV .. +RV-1.
// v[] is indexed (key slot, head) = slot*G + head.  A step that halves over a key-slot bit needs no
// selects: the lanes with that lane bit set have walked their key slots in an order with that slot
// bit flipped (key_slot_permutation), so every lane keeps its lower register half and sends the
// upper one.  Steps over head bits select per lane.
template <int NV, int LANES, int G>
__device__ __forceinline__ void group_reduce_scatter(float (&v)[NV], int lane_in_group) {
    int cnt = NV;
#pragma unroll
    for (int off = LANES / 2; off >= 1; off >>= 1) {
        if (cnt > 1) {
            const int half = cnt / 2;
            if (half >= G) {  // a key-slot bit
#pragma unroll
                for (int j = 0; j < NV / 2; ++j) {
                    if (j < half) v[j] += __shfl_xor_sync(0xffffffffu, v[j + half], off);
                }
            } else {
                const bool upper = (lane_in_group & off) != 0;
#pragma unroll
                for (int j = 0; j < NV / 2; ++j) {
                    if (j < half) {
                        const float send = upper ? v[j] : v[j + half];
                        const float keep = upper ? v[j + half] : v[j];
                        v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                }
            }
            cnt = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
        }
    }
}
// XOR mask a lane applies to its key-slot index i (register slot i holds key slot i ^ mask).
template <int NV, int LANES, int G>
__device__ __forceinline__ int key_slot_permutation(int lane_in_group) {
    int perm = 0, cnt = NV;
#pragma unroll
    for (int off = LANES / 2; off >= 1; off >>= 1) {
        if (cnt > 1) {
            const int half = cnt / 2;
            if (half >= G && (lane_in_group & off)) perm |= half / G;
            cnt = half;
        }
    }
    return perm;
}

// arr[idx] for a run-time idx without sending the array to local memory.
template <int N>
__device__ __forceinline__ float pick(const float (&arr)[N], int idx) {
    float x = arr[0];
#pragma unroll
    for (int i = 1; i < N; ++i) x = (idx == i) ? arr[i] : x;
    return x;
}

constexpr float kLazyRaise = 8.0f;

// One K or V tile of a paged cache whose pages are shorter than the tile: one TMA box per page (whole
// tile) or one bulk copy per row (ragged tail), the page of every run or row looked up in the block table.
// Out of line, so that the common path's registers do not pay for it.  The caller has posted expect_tx.
// `my_page` (whole tiles): lane i holds the tile's i-th page, read by the caller with one coalesced load ahead of
// its wait for the stage -- one table look-up after another by a single lane, twice per tile (K and V), took
// longer than the two stages of a tile pipeline can hide (config 2 at 16-key pages: 464 us against 377 us packed).
static __device__ __noinline__ void load_tile_short_pages(const int *block_table, long long table_stride, int page_shift, int b, int key0,
                                                   int rows, int tile, bool whole, uint8_t *dst, int row_bytes,
                                                   const CUtensorMap *tm, int hk, const uint8_t *g_base,
                                                   long long g_row_bytes, uint64_t *bar, int lane, int my_page) {
    const int run = 1 << page_shift;
    const int *pages = block_table + (size_t)b * table_stride;
    if (whole) {
        for (int i = 0; i < (tile >> page_shift); ++i) {  // (tiles start on a page boundary)
            const int row = __shfl_sync(0xffffffffu, my_page, i) << page_shift;
            if (lane == 0) tma_load_tile_3d(dst + ((size_t)i << page_shift) * row_bytes, tm, 0, hk, row, bar);
        }
    } else {
        for (int r = lane; r < rows; r += 32) {
            const size_t row = ((size_t)pages[(key0 + r) >> page_shift] << page_shift) + ((key0 + r) & (run - 1));
            bulk_copy_g2s(dst + (size_t)r * row_bytes, g_base + row * g_row_bytes, (uint32_t)row_bytes, bar);
        }
    }
}

template <class C>
__global__ void __launch_bounds__(C::THREADS, C::MINB) da_split_kernel(const SplitParams p,
                                                              const __grid_constant__ CUtensorMap tm_k,
                                                              const __grid_constant__ CUtensorMap tm_v) {
    using T = typename C::T;
    constexpr int D = C::D, DV = C::DV, LANES = C::LANES, G = C::G, KPT = C::KPT, NG = C::NG, TILE = C::TILE;
    constexpr int NCH = C::NCH, NCHV = C::NCHV, NV = C::NV, RV = C::RV, REP = C::REP, STAGES = C::STAGES;
    extern __shared__ __align__(128) uint8_t smem[];

    pdl_launch_dependents();  // the merge kernel may be scheduled behind this grid's last CTAs
    const int split = blockIdx.x;
    const int hk = blockIdx.y / p.head_chunks;
    const int hc = blockIdx.y % p.head_chunks;
    if (p.batch_order) pdl_wait();  // written by the order kernel launched just before this one
    const int b = p.batch_order ? p.batch_order[blockIdx.z] : (int)blockIdx.z;
    const int h0 = hk * p.group + hc * G;  // first query head of this CTA
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;

    const int seq_begin = p.cu_seq_k[b];
    const int len = p.cu_seq_k[b + 1] - seq_begin;
    const int k_begin = split * p.chunk_keys;
    const int k_end = split_key_end(p, split, len);
    const float neg_inf = -INFINITY;

    if (k_begin >= k_end) {
        // Nothing to read.  With several splits the merge kernel skips this one; with a single split
        // the sequence is empty: the row is defined as zeros with LSE = -inf.
        if (p.num_splits == 1) {
            for (int idx = tid; idx < G * DV; idx += C::THREADS) {
                const int g = idx / DV, d = idx % DV;
                const size_t off = (size_t)b * p.o_row_stride + (size_t)(h0 + g) * DV + d;
                if (p.o) reinterpret_cast<T *>(p.o)[off] = from_float<T>(0.0f);
                if (p.o_f32) p.o_f32[((size_t)b * p.head_q + h0 + g) * DV + d] = 0.0f;
            }
            if (p.lse && tid < G) p.lse[(size_t)b * p.head_q + h0 + tid] = neg_inf;
        }
        return;
    }

    uint8_t *ks = smem + C::OFF_K;
    uint8_t *vs = C::MLA ? ks : smem + C::OFF_V;
    float *p_s = reinterpret_cast<float *>(smem + C::OFF_P);
    uint64_t *full_k = reinterpret_cast<uint64_t *>(smem + C::OFF_BAR);
    uint64_t *empty_k = full_k + STAGES;
    uint64_t *full_v = empty_k + STAGES;
    uint64_t *empty_v = full_v + STAGES;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty_v + STAGES);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_k[s], 1);
            mbar_init(&empty_k[s], C::NWARPS);
            mbar_init(&full_v[s], 1);
            mbar_init(&empty_v[s], C::NWARPS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    const int n_tiles = (k_end - k_begin + TILE - 1) / TILE;

    if (warp == C::NWARPS) {
        // ---------------- producer warp ----------------
        constexpr int EBITS = C::KV_BITS;  // element size of the cache, in bits (strides count elements)
        const uint8_t *kg = reinterpret_cast<const uint8_t *>(p.k) + (size_t)hk * D * EBITS / 8;
        const uint8_t *vg = reinterpret_cast<const uint8_t *>(p.v) + (size_t)hk * (C::MLA ? D : DV) * EBITS / 8;
        if (p.use_tmap && lane == 0) {
            tma_prefetch_desc(&tm_k);
            if (!C::MLA) tma_prefetch_desc(&tm_v);
        }
        bool ok = true;
        int armed_k = 0, armed_v = 0;  // tiles whose full barrier has been armed
        const bool short_pages = kv_run_keys(p, TILE) != TILE;  // paged cache with pages shorter than the tile
        for (int t = 0; t < n_tiles; ++t) {
            const int st = t % STAGES;
            const uint32_t ph = (uint32_t)(t / STAGES) & 1u;
            const int key0 = k_begin + t * TILE;
            const int rows = min(TILE, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            const bool whole = p.use_tmap && rows == TILE;  // a partial tile must not read past the sequence
            int my_page = 0;  // short pages: lane i reads the tile's i-th page from the block table, ahead of the wait
            if (short_pages && whole && lane < (TILE >> p.page_shift)) {
                my_page = p.block_table[(size_t)b * p.block_table_stride + (key0 >> p.page_shift) + lane];
            }
            if (t >= STAGES) ok = mbar_wait(&empty_k[st], ph ^ 1u, abort_flag);
            if (!ok) break;
            if (lane == 0) {
                mbar_arrive_expect_tx(&full_k[st], (uint32_t)rows * C::K_ROW_BYTES);
                if (whole && !short_pages) tma_load_tile_3d(ks + st * C::K_TILE_BYTES, &tm_k, 0, hk, (int)tok0, &full_k[st]);
            }
            __syncwarp();
            armed_k = t + 1;
            if (short_pages) {
                load_tile_short_pages(p.block_table, p.block_table_stride, p.page_shift, b, key0, rows, TILE, whole,
                                      ks + st * C::K_TILE_BYTES, C::K_ROW_BYTES, &tm_k, hk, kg,
                                      p.k_row_stride * (long long)EBITS / 8, &full_k[st], lane, my_page);
            } else if (!whole) {
                for (int r = lane; r < rows; r += 32) {
                    bulk_copy_g2s(ks + st * C::K_TILE_BYTES + r * C::K_ROW_BYTES, kg + (tok0 + r) * p.k_row_stride * EBITS / 8,
                                  C::K_ROW_BYTES, &full_k[st]);
                }
            }
            if (!C::MLA) {
                if (t >= STAGES) ok = mbar_wait(&empty_v[st], ph ^ 1u, abort_flag);
                if (!ok) break;
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full_v[st], (uint32_t)rows * C::V_ROW_BYTES);
                    if (whole && !short_pages) tma_load_tile_3d(vs + st * C::V_TILE_BYTES, &tm_v, 0, hk, (int)tok0, &full_v[st]);
                }
                __syncwarp();
                armed_v = t + 1;
                if (short_pages) {
                    load_tile_short_pages(p.block_table, p.block_table_stride, p.page_shift, b, key0, rows, TILE, whole,
                                          vs + st * C::V_TILE_BYTES, C::V_ROW_BYTES, &tm_v, hk, vg,
                                          p.v_row_stride * (long long)EBITS / 8, &full_v[st], lane, my_page);
                } else if (!whole) {
                    for (int r = lane; r < rows; r += 32) {
                        bulk_copy_g2s(vs + st * C::V_TILE_BYTES + r * C::V_ROW_BYTES,
                                      vg + (tok0 + r) * p.v_row_stride * EBITS / 8, C::V_ROW_BYTES, &full_v[st]);
                    }
                }
            }
        }
        if (!ok) {
            // A wait ran out.  Report it, then give the copies that are still in flight a bounded time
            // to land before this warp (the last user of the stage buffers) retires.
            if (lane == 0) report_timeout(p);
            for (int back = 1; back <= STAGES; ++back) {
                const int tk = armed_k - back, tv = armed_v - back;
                for (uint32_t spin = 0; tk >= 0 && spin < (1u << 20); ++spin)
                    if (mbar_try_wait(&full_k[tk % STAGES], (uint32_t)(tk / STAGES) & 1u)) break;
                for (uint32_t spin = 0; tv >= 0 && spin < (1u << 20); ++spin)
                    if (mbar_try_wait(&full_v[tv % STAGES], (uint32_t)(tv / STAGES) & 1u)) break;
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    const int c = lane % LANES;                     // lane in group = chunk index
    const int gi = warp * C::GPW + lane / LANES;    // group in CTA
    float *p_grp = p_s + gi * NV;

    // Q slice of this lane for the G heads, fp32.
    float qf[G][NCH][8];
    {
        const T *qg = reinterpret_cast<const T *>(p.q) + (size_t)b * p.q_row_stride + (size_t)h0 * D;
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int n = 0; n < NCH; ++n) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(qg + g * D + (c + n * LANES) * 8);
                unpack8<T>(raw, qf[g][n]);
            }
        }
    }

    // Which (key slot, head) pairs this lane owns after the reduce-scatter, and their ALiBi slopes.
    const int j0 = (c / REP) * RV;
    const int slot_perm = key_slot_permutation<NV, LANES, G>(c);
    float slope2[RV];  // slope * log2(e)
#pragma unroll
    for (int r = 0; r < RV; ++r) {
        const int g = (j0 + r) % G;
        slope2[r] = p.is_alibi ? exp2f(-8.0f * (float)(h0 + g + 1) / (float)p.head_q) * kLog2e : 0.0f;
    }
    const int pos_shift = (p.kv_pos_offset ? p.kv_pos_offset[b] : 0) - ((p.kv_total_len ? p.kv_total_len[b] : len) - 1);

    float m_run[G];      // running max per head (log2 domain), identical in every lane of the group
    float l_lane[RV];    // running sum of this lane's own probabilities
    float oacc[G][NCHV][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_run[g] = neg_inf;
#pragma unroll
        for (int n = 0; n < NCHV; ++n)
#pragma unroll
            for (int e = 0; e < 8; ++e) oacc[g][n][e] = 0.0f;
    }
#pragma unroll
    for (int r = 0; r < RV; ++r) l_lane[r] = 0.0f;

    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
        const int st = t % STAGES;
        const uint32_t ph = (uint32_t)(t / STAGES) & 1u;
        const int key0 = k_begin + t * TILE;
        const int rows = min(TILE, k_end - key0);

        // ---- S = Q K^T for this group's keys ----
        ok = mbar_wait(&full_k[st], ph, abort_flag);
        if (!ok) break;
        float sacc[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) sacc[j] = 0.0f;
        const uint8_t *kt = ks + st * C::K_TILE_BYTES;
#pragma unroll
        for (int i = 0; i < KPT; ++i) {
            const int kl = (i ^ slot_perm) * NG + gi;  // key slot in the tile (register slot i)
#pragma unroll
            for (int n = 0; n < NCH; ++n) {
                float kf[8];
                load_chunk8<T, C::KVQ>(kt + kl * C::K_ROW_BYTES + (c + n * LANES) * C::CHUNK_BYTES, kf);
#pragma unroll
                for (int g = 0; g < G; ++g) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) sacc[i * G + g] = fmaf(qf[g][n][e], kf[e], sacc[i * G + g]);
                }
            }
        }
        if (!C::MLA) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_k[st]);
        }
        group_reduce_scatter<NV, LANES, G>(sacc, c);

        // ---- scale, bias, mask; publish the scores of the group ----
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            const int j = j0 + r;
            const int kl = (j / G) * NG + gi;
            const int pos = key0 + kl;
            float s = sacc[r] * p.scale_log2 + slope2[r] * (float)(pos + pos_shift);
            sacc[r] = (kl < rows) ? s : neg_inf;
        }
        // ---- online softmax with a lazy reference: m_run is raised (and O, l rescaled) only when some
        // score of the group exceeds it by more than 2^kLazyRaise; otherwise p = 2^(s - m_run) <= 2^kLazyRaise.
        bool raise = false;
#pragma unroll
        for (int r = 0; r < RV; ++r) raise |= sacc[r] > pick<G>(m_run, (j0 + r) % G) + kLazyRaise;
        const unsigned grp_mask = LANES == 32 ? 0xffffffffu : (((1u << LANES) - 1u) << ((lane / LANES) * LANES));
        // the ballot also orders this tile's writes to p_grp after the previous tile's reads
        const bool grp_raise = (__ballot_sync(0xffffffffu, raise) & grp_mask) != 0u;
        if (grp_raise) {
#pragma unroll
            for (int r = 0; r < RV; ++r) p_grp[j0 + r] = sacc[r];
            __syncwarp(grp_mask);
            float alpha[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float m_new = m_run[g];
#pragma unroll
                for (int i = 0; i < KPT; ++i) m_new = fmaxf(m_new, p_grp[i * G + g]);
                const float m_use = (m_new == neg_inf) ? 0.0f : m_new;
                alpha[g] = exp2f(m_run[g] - m_use);
                m_run[g] = m_new;
            }
            __syncwarp(grp_mask);  // everybody of the group has read the raw scores
#pragma unroll
            for (int r = 0; r < RV; ++r) l_lane[r] *= pick<G>(alpha, (j0 + r) % G);
#pragma unroll
            for (int g = 0; g < G; ++g) {
#pragma unroll
                for (int n = 0; n < NCHV; ++n)
#pragma unroll
                    for (int e = 0; e < 8; ++e) oacc[g][n][e] *= alpha[g];
            }
        }
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            const float m_g = pick<G>(m_run, (j0 + r) % G);
            const float pr = exp2f(sacc[r] - ((m_g == neg_inf) ? 0.0f : m_g));
            l_lane[r] += pr;
            p_grp[j0 + r] = pr;
        }
        __syncwarp();

        // ---- O += P V ----
        if (!C::MLA) {
            ok = mbar_wait(&full_v[st], ph, abort_flag);
            if (!ok) break;
        }
        const uint8_t *vt = C::MLA ? kt : vs + st * C::V_TILE_BYTES;
        constexpr int VROW = C::MLA ? C::K_ROW_BYTES : C::V_ROW_BYTES;
#pragma unroll
        for (int i = 0; i < KPT; ++i) {
            const int kl = i * NG + gi;
            if (kl < rows) {
                float pg[G];
#pragma unroll
                for (int g = 0; g < G; ++g) pg[g] = p_grp[i * G + g];
#pragma unroll
                for (int n = 0; n < NCHV; ++n) {
                    float vf[8];
                    load_chunk8<T, C::KVQ>(vt + kl * VROW + (c + n * LANES) * C::CHUNK_BYTES, vf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) oacc[g][n][e] = fmaf(pg[g], vf[e], oacc[g][n][e]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(C::MLA ? &empty_k[st] : &empty_v[st]);
    }
    if (!ok && lane == 0) report_timeout(p);

    // ---------------- merge the groups of the CTA ----------------
    // Every consumer has passed its last full-barrier wait, so every copy has landed and the stage
    // buffers can be reused once all consumers are done reading them.
    named_bar_sync(1, C::CONSUMERS);
    float *red_m = reinterpret_cast<float *>(smem);  // [NG][G]
    float *red_l = red_m + NG * G;                    // [NG][G]
    float *red_o = red_l + NG * G;                    // [NG][G][DV]
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RV; ++r) p_grp[j0 + r] = l_lane[r];
    __syncwarp();
    if (c == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float l = 0.0f;
#pragma unroll
            for (int i = 0; i < KPT; ++i) l += p_grp[i * G + g];
            red_m[gi * G + g] = m_run[g];
            red_l[gi * G + g] = l;
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int n = 0; n < NCHV; ++n) {
            float4 *dst = reinterpret_cast<float4 *>(red_o + (size_t)(gi * G + g) * DV + (c + n * LANES) * 8);
            dst[0] = make_float4(oacc[g][n][0], oacc[g][n][1], oacc[g][n][2], oacc[g][n][3]);
            dst[1] = make_float4(oacc[g][n][4], oacc[g][n][5], oacc[g][n][6], oacc[g][n][7]);
        }
    }
    named_bar_sync(1, C::CONSUMERS);
    if (*abort_flag) return;  // a wait ran out somewhere in the CTA: the status word says so

    for (int idx = tid; idx < G * DV; idx += C::CONSUMERS) {
        const int g = idx / DV, d = idx % DV;
        float mx = neg_inf;
#pragma unroll
        for (int x = 0; x < NG; ++x) mx = fmaxf(mx, red_m[x * G + g]);
        float l = 0.0f, o = 0.0f;
#pragma unroll
        for (int x = 0; x < NG; ++x) {
            const float w = exp2f(red_m[x * G + g] - mx);  // mx is finite: the key range is not empty
            l = fmaf(red_l[x * G + g], w, l);
            o = fmaf(red_o[(size_t)(x * G + g) * DV + d], w, o);
        }
        const float out = o / l * p.out_scale;
        const int h = h0 + g;
        const float lse = (mx + log2f(l)) * kLn2;
        if (p.num_splits == 1) {
            if (p.o) reinterpret_cast<T *>(p.o)[(size_t)b * p.o_row_stride + (size_t)h * DV + d] = from_float<T>(out);
            if (p.o_f32) p.o_f32[((size_t)b * p.head_q + h) * DV + d] = out;
            if (p.lse && d == 0) p.lse[(size_t)b * p.head_q + h] = lse;
        } else {
            const size_t row = ((size_t)b * p.head_q + h) * p.num_splits + split;
            p.part_o[row * DV + d] = out;
            if (d == 0) p.part_lse[row] = lse;
        }
    }
}

// Host side.  `tm_k` / `tm_v` are rank-3 tensor maps [rows][head_k][dim] with box {dim, 1, TILE}
// (see make_kv_tensor_map in da_api.cu); they are ignored when p.use_tmap is 0.
template <class C>
cudaError_t launch_split(const SplitParams &p, const CUtensorMap &tm_k, const CUtensorMap &tm_v,
                         cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !attr_set[dev]) {
        err = cudaFuncSetAttribute(da_split_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (err != cudaSuccess) return err;
        attr_set[dev] = true;
    }
    dim3 grid(p.num_splits, p.head_k * p.head_chunks, p.batch);
    return launch_kernel(da_split_kernel<C>, grid, C::THREADS, C::SMEM_BYTES, stream, p.batch_order != nullptr, p, tm_k, tm_v);
}

}  // namespace da
