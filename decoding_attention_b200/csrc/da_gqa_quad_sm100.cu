// Grouped-query / multi-query decode attention for groups of at most 32 query heads per KV head (head
// dims 64, 96, 128) on the sm_100a tensor cores: four key streams, one per TMEM lane quadrant.
//
// An M = 128 tcgen05.mma tile whose rows are the query heads of one KV head (da_gqa_tc_sm100.cu) leaves
// 96 rows, and the softmax warps of three lane quadrants, idle when the group has 32 heads or fewer,
// and the kernel then runs at the pace of one quadrant's softmax chain (about 2 300 cycles of TMEM
// load / barrier / TMEM store latency per 64 keys and stream).  Here the group's Q rows are staged
// four times, rows 32 q .. 32 q + 31 = heads 0 .. 31, and the key range is dealt out in units of 64
// keys, unit j to quadrant j % 4:
//     S_q[128 x 64] = Q[128 x D] . K_unit[64 x D]^T     every row block computes it, block q's rows are read
//     O[128 x D]   += P_q[128 x 64] . V_unit[64 x D]     P_q is zero outside row block q
// so row block q of the one accumulator sums the units of quadrant q: four independent online-softmax
// streams over a quarter of the keys each, merged at the end like key-range splits.  The tensor pipe
// does four times the useful work and still idles; the softmax latency of four units overlaps.
// P_q lives in tensor memory (A operand of the second contraction): 4 x 32 columns whose lanes outside
// quadrant q are zeroed once.  Tensor memory: S 4 x 64 | P 4 x 32 | O D columns.
// K and V units travel through separate rings (a K unit is free after its S, a V unit waits for the
// softmax of its unit): K by TMA boxes, V by 16-byte cp.async of four loader warps.  Warps: 8 softmax (two per
// quadrant), TMA producer, S issuer, P.V issuer, 4 V loaders.  All P.V contractions are issued in unit order
// by one warp, so a quadrant that has to rescale its accumulator rows (rare: lazy reference max) only has to
// see the three units before its own retire: the next P.V cannot be issued before this quadrant delivers P.
// Under ALiBi the units are walked back to front, which keeps that path rare.  Every wait is bounded.  The reference runs this shape with one CTA per query head
// (csrc/kernel/decoding_attn/decoding_fwd_hd128_hdv128.cu:9-25), reading K and V once per head.
#include <type_traits>

#include "da_internal.h"
#include "da_tcgen05.cuh"

namespace da {
namespace {

constexpr int kRows = 128;                 // M of both contractions: 4 row blocks x 32 heads
constexpr int kUnit = 64;                  // keys per unit
constexpr int kQuads = 4;
constexpr int kQBlockBytes = kRows * 128;  // [128 rows x 64 dims]
constexpr int kKBlockBytes = kUnit * 128;  // [64 keys x 64 dims]
constexpr int kColsPer = 32;               // score columns per softmax thread (two threads per row)
constexpr int kTmemCols = 512;
constexpr int kColS = 0;                   // 4 x 64
constexpr int kColP = 256;                 // 4 x 32 (16-bit values in pairs)
constexpr int kColO = 384;                 // D <= 128 columns
constexpr int kSoftmaxWarps = 8, kProducerWarp = 8, kMmaWarp = 9, kPvWarp = 10, kLoaderWarp0 = 11, kLoaderWarps = 4;
constexpr int kThreads = (kSoftmaxWarps + 3 + kLoaderWarps) * 32;
constexpr int kVInFlight = 3;              // V units a loader warp keeps in flight
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct QuadCfg {
    static constexpr int kBlocks = D / 64;
    static constexpr int kUnitBytes = kBlocks * kKBlockBytes;  // a K unit; a V unit has the same size
    static constexpr int kNK = D == 128 ? 5 : 9;               // K ring, V ring (units)
    static constexpr int kNV = D == 128 ? 6 : 12;
    static constexpr int kStageStride = D + 4;                 // floats per staged output row (bank spread)
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + kBlocks * kQBlockBytes;
    static constexpr int kOffV = kOffK + kNK * kUnitBytes;
    static constexpr int kOffX = kOffV + kNV * kUnitBytes;     // row maxima [2 parities][4 quads][2 halves][32]
    static constexpr int kXFloats = 2 * kQuads * 2 * 32 + kQuads * 32 + kQuads * 2 * 32;  // + final m, final l
    static constexpr int kOffBar = kOffX + kXFloats * 4;
    // q_full, k_full/k_empty[kNK], v_full/v_empty[kNV], s_full/s_empty/p_full/pv_done/row_sync[4], p_zeroed, fin_sync, mma_done
    static constexpr int kNumBars = 1 + 2 * kNK + 2 * kNV + 5 * kQuads + 3;
    static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;
    static_assert(D == 64 || D == 128, "head dim");
    static_assert(kColO + D <= kTmemCols, "TMEM budget");
    static_assert(kQuads * 32 * kStageStride * 4 <= (kNK + kNV) * kUnitBytes, "output staging fits the idle rings");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// kShortPages: the cache is paged with pages shorter than a unit, which is then fetched page by page
// (a separate instantiation, so that the common case keeps its straight-line address arithmetic).
template <typename T, int D, bool kShortPages>
__global__ void __launch_bounds__(kThreads, 1)
da_gqa_quad_kernel(const SplitParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k) {
    using C = QuadCfg<D>;
    constexpr int kBlocks = C::kBlocks, kUnitBytes = C::kUnitBytes, kNK = C::kNK, kNV = C::kNV, kStageStride = C::kStageStride;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    if (threadIdx.x == kProducerWarp * 32) {  // descriptor fetches overlap the set-up below
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
    }
    pdl_launch_dependents();  // the merge kernel may be scheduled behind this grid's last CTAs
    const int split = blockIdx.x;
    const int hk = blockIdx.y;
    if (p.batch_order) pdl_wait();  // written by the order kernel launched just before this one
    const int b = p.batch_order ? p.batch_order[blockIdx.z] : (int)blockIdx.z;
    const int G = p.group;  // query heads of this KV head (at most 32): rows 0..G-1 of every row block
    const int h0 = hk * G;
    const int dreal = p.dim;  // 96 runs padded to 128: the tensor maps zero-fill columns 96..127
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq_begin = p.cu_seq_k[b];
    const int len = p.cu_seq_k[b + 1] - seq_begin;
    const int k_begin = split * p.chunk_keys;
    const int k_end = split_key_end(p, split, len);
    T *o_out = reinterpret_cast<T *>(p.o);
    if (launch_aborted(p)) return;  // an earlier CTA of this launch timed out: do not pile up

    if (k_begin >= k_end) {
        if (p.num_splits == 1) {  // empty sequence: zero rows, LSE = -inf
            for (int idx = tid; idx < G * dreal; idx += kThreads) {
                const int h = h0 + idx / dreal, d = idx % dreal;
                if (o_out) o_out[(size_t)b * p.o_row_stride + (size_t)h * dreal + d] = from_float<T>(0.0f);
                if (p.o_f32) p.o_f32[((size_t)b * p.head_q + h) * dreal + d] = 0.0f;
            }
            if (p.lse && tid < G) p.lse[(size_t)b * p.head_q + h0 + tid] = -INFINITY;
        }
        return;
    }
    const int n_units = (k_end - k_begin + kUnit - 1) / kUnit;
    // With ALiBi the bias grows towards the end of the sequence, and so does every head's row maximum: walked
    // front to back, every unit would raise the reference maximum of the steep heads and take the rescale path
    // (measured: config 3 43 us against 33 us without ALiBi).  Walked back to front the first units set the
    // maximum and the path stays rare.  `unit_of(j)` is the unit the j-th step works on.
    const bool backwards = p.is_alibi != 0;
    auto unit_of = [&](int j) { return backwards ? n_units - 1 - j : j; };

    uint8_t *q_s = smem + C::kOffQ;
    uint8_t *k_s = smem + C::kOffK;
    uint8_t *v_s = smem + C::kOffV;
    float *rowmax_s = reinterpret_cast<float *>(smem + C::kOffX);  // [2][4][2][32]
    float *m_fin = rowmax_s + 2 * kQuads * 2 * 32;                 // [4][32]
    float *l_fin = m_fin + kQuads * 32;                            // [4][2][32]
    float *stage = reinterpret_cast<float *>(k_s);                 // [4][32][kStageStride], once the rings are idle
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kOffBar);
    uint64_t *q_full = bars;
    uint64_t *k_full = bars + 1;
    uint64_t *k_empty = k_full + kNK;
    uint64_t *v_full = k_empty + kNK;
    uint64_t *v_empty = v_full + kNV;
    uint64_t *s_full = v_empty + kNV;
    uint64_t *s_empty = s_full + kQuads;
    uint64_t *p_full = s_empty + kQuads;
    uint64_t *pv_done = p_full + kQuads;
    uint64_t *row_sync = pv_done + kQuads;
    uint64_t *p_zeroed = row_sync + kQuads;
    uint64_t *fin_sync = p_zeroed + 1;
    uint64_t *mma_done = fin_sync + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + C::kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (tid < C::kNumBars) {
        // one barrier per thread; arrival counts: TMA / commit barriers 1, V units one per loader warp, the
        // softmax barriers the 64 threads of a quadrant or all 256
        uint64_t *bar = bars + tid;
        int count = 1;
        if (bar >= v_full && bar < v_empty) count = kLoaderWarps;
        if ((bar >= s_empty && bar < pv_done) || (bar >= row_sync && bar < p_zeroed)) count = 64;
        if (bar == p_zeroed || bar == fin_sync) count = kSoftmaxThreads;
        mbar_init(bar, count);
        if (tid == 0) *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kMmaWarp) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr uint32_t kIdescQK = instr_desc(kFmt, 0, kRows, kUnit);
    constexpr uint32_t kIdescPV = instr_desc(kFmt, 1, kRows, D);
    bool ok = true;

    if (warp == kProducerWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            // Heads h0 .. h0+31 of q into each of the four row blocks (the map's box holds min(32, head_q) rows;
            // rows past the group belong to the next KV head or read as zeros and feed rows nobody reads back).
            mbar_arrive_expect_tx(q_full, kQuads * kBlocks * min(32, p.head_q) * 128);
            for (int kb = 0; kb < kBlocks; ++kb) {
                for (int rb = 0; rb < kQuads; ++rb) {
                    tma_load_tile_3d(q_s + kb * kQBlockBytes + rb * (32 * 128), &tm_q, kb * 64, h0, b, q_full);
                }
            }
        }
        const T *k_g = reinterpret_cast<const T *>(p.k) + (size_t)hk * dreal;
        const int run = kShortPages ? kv_run_keys(p, kUnit) : kUnit;
        for (int j = 0; j < n_units && ok; ++j) {
            const int ks = j % kNK;
            const int key0 = k_begin + unit_of(j) * kUnit;
            const int rows = min(kUnit, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            auto row_of = [&](int r) { return kShortPages ? kv_tile_row(p, b, seq_begin, key0 + r) : tok0 + r; };
            uint8_t *kd = k_s + ks * kUnitBytes;
            int my_page = 0;
            if (kShortPages && rows == kUnit && lane < (kUnit >> p.page_shift)) {
                my_page = p.block_table[(size_t)b * p.block_table_stride + (key0 >> p.page_shift) + lane];
            }
            if (j >= kNK) ok = mbar_wait(&k_empty[ks], ((uint32_t)(j / kNK) & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            if (rows == kUnit) {
                if (lane == 0) mbar_arrive_expect_tx(&k_full[ks], kUnitBytes);
                for (int k0 = 0; k0 < kUnit; k0 += run) {  // one box per run of consecutive rows (a page, or the unit)
                    // (short pages: lane i has read the unit's i-th page, all lanes with one load; units start on a page boundary)
                    const int row = kShortPages ? (__shfl_sync(0xffffffffu, my_page, k0 >> p.page_shift) << p.page_shift) : (int)tok0;
                    if (lane == 0) {
                        for (int kb = 0; kb < kBlocks; ++kb) tma_load_tile_3d(kd + kb * kKBlockBytes + k0 * 128, &tm_k, kb * 64, hk, row, &k_full[ks]);
                    }
                }
            }
            if (rows < kUnit) {
                // Ragged last unit: 16-byte cp.async into the 128-byte-swizzled layout, rows past the end and
                // columns past the real head dim zero-filled (the tensor maps must not be asked for rows beyond the
                // sequence).  All of the warp's copies are in flight at once: one memory latency, where a loop of
                // loads and stores took 2-3 us, on the one unit the whole CTA waits for.
                constexpr int kChunks = D / 8;  // 16-byte chunks per row
                for (int i = lane; i < kUnit * kChunks; i += 32) {
                    const int r = i / kChunks, c = i % kChunks;
                    const bool real = r < rows && c * 8 < dreal;
                    const T *src = k_g + row_of(real ? r : 0) * p.k_row_stride + (real ? c * 8 : 0);
                    cp_async16(kd + (c >> 3) * kKBlockBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4), src, real ? 16u : 0u);
                }
                cp_async_commit();
                cp_async_wait<0>();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&k_full[ks]);
            }
            __syncwarp();
        }
    } else if (warp >= kLoaderWarp0) {
        // ---------------- V loaders: 16-byte cp.async straight into the swizzled layout the tensor maps produce.
        // One SM's TMA engine writes about 25 bytes per cycle; with V on the load/store path K and V arrive side
        // by side.  Rows past the end of the sequence and columns past the real head dim are zero-filled.  A unit's
        // barrier gets this warp's arrival once kVInFlight - 1 later units have been issued and its bytes have landed.
        const T *v_g = reinterpret_cast<const T *>(p.v) + (size_t)hk * dreal;
        const int lt = tid - kLoaderWarp0 * 32;  // 0..127: chunk lt & 7 of rows (lt >> 3) + 16 i of every 64-column block
        const int cc = lt & 7;
        for (int j = 0; j < n_units && ok; ++j) {
            const int vs = j % kNV;
            const int key0 = k_begin + unit_of(j) * kUnit;
            const int rows = min(kUnit, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            if (j >= kNV) ok = mbar_wait(&v_empty[vs], ((uint32_t)(j / kNV) & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            uint8_t *slot = v_s + vs * kUnitBytes;
#pragma unroll
            for (int ri = 0; ri < kUnit / 16; ++ri) {
                const int r = (lt >> 3) + 16 * ri;
                const int rr = min(r, rows - 1);
                const size_t trow = kShortPages ? kv_tile_row(p, b, seq_begin, key0 + rr) : tok0 + rr;
                const T *src = v_g + trow * p.v_row_stride + cc * 8;
#pragma unroll
                for (int kb = 0; kb < kBlocks; ++kb) {
                    const bool real = r < rows && kb * 64 + cc * 8 < dreal;
                    cp_async16(slot + kb * kKBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4), real ? src + kb * 64 : src, real ? 16u : 0u);  // 0: zero fill
                }
            }
            cp_async_commit();
            if (j >= kVInFlight - 1) {
                cp_async_wait<kVInFlight - 1>();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&v_full[(j - (kVInFlight - 1)) % kNV]);
            }
        }
        // the last units: every group has landed after the wait for all
        cp_async_wait<0>();
        fence_proxy_async();
        __syncwarp();
        if (ok && lane == 0) {
            for (int j = max(0, n_units - (kVInFlight - 1)); j < n_units; ++j) mbar_arrive(&v_full[j % kNV]);
        }
    } else if (warp == kMmaWarp) {
        // ---------------- issuer of the first contraction ----------------
        // S and P.V have an issuing warp each: with contractions this small the issue loop (barrier waits,
        // commits) sets the pace, not the tensor pipe, and one warp doing both took 1 420 cycles per unit.
        // (The whole warp walks the loop and an elected lane issues; the loop run by lane 0 alone is slower.)
        {
            const uint32_t leader = elect_one();
            const uint64_t q_desc0 = smem_desc(smem_u32(q_s), 16, 1024, 2);  // K-major, 8-row groups 1 KB apart
            const uint64_t k_desc0 = smem_desc(smem_u32(k_s), 16, 1024, 2);
            ok = mbar_wait(q_full, 0, abort_flag);
            for (int i = 0; i < n_units && ok; ++i) {
                // S of unit i into its quadrant's score columns.
                const int qd = i & 3, ks = i % kNK;
                ok = mbar_wait(&k_full[ks], (uint32_t)(i / kNK) & 1u, abort_flag);
                if (ok && i >= kQuads) ok = mbar_wait(&s_empty[qd], ((uint32_t)(i >> 2) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t kd = k_desc0 + (uint64_t)((ks * kUnitBytes) >> 4);
                const uint32_t d = tmem_base + kColS + qd * kUnit;
#pragma unroll
                for (int kb = 0; kb < kBlocks; ++kb) {
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        umma_ss(d, q_desc0 + (uint64_t)((kb * kQBlockBytes + s * 32) >> 4),
                                kd + (uint64_t)((kb * kKBlockBytes + s * 32) >> 4), kIdescQK, (kb | s) ? 1u : 0u, leader);
                    }
                }
                umma_commit(&s_full[qd], leader);
                umma_commit(&k_empty[ks], leader);
            }
        }
        __syncwarp();
    } else if (warp == kPvWarp) {
        // ---------------- issuer of the second contraction, in unit order ----------------
        {
            const uint32_t leader = elect_one();
            const uint64_t v_desc0 = smem_desc(smem_u32(v_s), kKBlockBytes, 1024, 2);  // MN-major: 64-col blocks LBO apart
            ok = mbar_wait(p_zeroed, 0, abort_flag);
            for (int j = 0; j < n_units && ok; ++j) {
                // O += P_q . V of unit j; row blocks other than q add zeros.  Unit 0 initialises all 128 rows.
                const int qd = j & 3, vs = j % kNV;
                ok = mbar_wait(&p_full[qd], (uint32_t)(j >> 2) & 1u, abort_flag);
                if (ok) ok = mbar_wait(&v_full[vs], (uint32_t)(j / kNV) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t pa = tmem_base + kColP + qd * 32;  // 16 keys = 8 columns of 16-bit pairs per step
                const uint64_t vd = v_desc0 + (uint64_t)((vs * kUnitBytes) >> 4);
#pragma unroll
                for (int s = 0; s < kUnit / 16; ++s) {
                    umma_ts(tmem_base + kColO, pa + s * 8, vd + (uint64_t)((s * 16 * 128) >> 4), kIdescPV, (j | s) ? 1u : 0u, leader);
                }
                umma_commit(&v_empty[vs], leader);
                umma_commit(&pv_done[qd], leader);
            }
            if (ok) umma_commit(mma_done, leader);  // (P of the last unit needed the last S: every contraction has finished)
        }
        __syncwarp();
    } else {
        // ------- softmax / epilogue: thread (quad, hf, lane) owns row 32 quad + lane (head `lane`) and the
        // score columns [32 hf, +32) of its quadrant's units j = quad, quad + 4, ... -------
        const int quad = warp & 3, hf = warp >> 2;
        const bool valid = lane < G;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t s_col = kColS + quad * kUnit + hf * kColsPer;
        const uint32_t p_col = kColP + quad * 32 + hf * 16;
        const float slope2 = p.is_alibi ? exp2f(-8.0f * (float)(h0 + lane + 1) / (float)p.head_q) * kLog2e : 0.0f;
        const int pos_shift = (p.kv_pos_offset ? p.kv_pos_offset[b] : 0) - ((p.kv_total_len ? p.kv_total_len[b] : len) - 1);
        float m_ref = -INFINITY, l = 0.0f;
        uint32_t buf[32];
        {
            // The rows of this quadrant are zero in the other quadrants' P (this thread's 16 columns of each).
            uint32_t z[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) z[j] = 0u;
            for (int qo = 0; qo < kQuads; ++qo) {
                if (qo != quad) tmem_st16(lane_base + kColP + qo * 32 + hf * 16, z);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(p_zeroed);
        }
        int n = 0;  // units this thread has finished (use count of its quadrant's barriers)
        for (int j = quad; j < n_units; j += kQuads, ++n) {
            const uint32_t par = (uint32_t)n & 1u;
            const int key0 = k_begin + unit_of(j) * kUnit + hf * kColsPer;
            const int cols = min(kUnit, k_end - (k_begin + unit_of(j) * kUnit)) - hf * kColsPer;  // valid columns of this thread
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[quad], par, abort_flag));
            if (!ok) break;
            tc_fence_after();
            tmem_ld32(lane_base + s_col, buf);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&s_empty[quad]);
            float s[kColsPer];
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < kColsPer; ++c) {
                const float x = __uint_as_float(buf[c]) * p.scale_log2 + slope2 * (float)(key0 + c + pos_shift);
                s[c] = (c < cols) ? x : -INFINITY;
                mx = fmaxf(mx, s[c]);
            }
            // The two threads of a row agree on the unit's row maximum (slots alternate with the unit's parity:
            // a thread may be a unit ahead of its partner's read).
            float *rm = rowmax_s + ((par * kQuads + quad) * 2) * 32;
            rm[hf * 32 + lane] = mx;
            mbar_arrive(&row_sync[quad]);
            ok = __all_sync(0xffffffffu, mbar_wait(&row_sync[quad], par, abort_flag));
            if (!ok) break;
            mx = fmaxf(mx, rm[(hf ^ 1) * 32 + lane]);
            const bool raise = mx > m_ref + kRescaleThreshold;
            float alpha = 1.0f;
            if (raise) {
                alpha = exp2f(m_ref - mx);  // 0 on the quadrant's first unit
                m_ref = mx;
                l *= alpha;
            }
            if (n >= 1) {
                // This quadrant's previous P.V (unit j - 4) has finished: its P columns are free again.
                ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[quad], (uint32_t)(n - 1) & 1u, abort_flag));
                if (!ok) break;
                if (__any_sync(0xffffffffu, raise && valid)) {
                    // Rare: the reference max of some row of this quadrant moved; rescale this thread's half of the
                    // row's accumulator columns in place.  Every P.V rewrites all 128 rows, so none may be in flight:
                    // those of units j-1, j-2, j-3 must have retired; the next one waits for this quadrant's P.
                    for (int d = 1; d < kQuads && ok; ++d) {
                        const int jj = j - d;
                        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[jj & 3], (uint32_t)(jj >> 2) & 1u, abort_flag));
                    }
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < D / 64; ++c) {
                        uint32_t ob[32];
                        tmem_ld32(lane_base + kColO + hf * (D / 2) + c * 32, ob);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) ob[e] = __float_as_uint(__uint_as_float(ob[e]) * alpha);
                        tmem_st32(lane_base + kColO + hf * (D / 2) + c * 32, ob);
                    }
                    tmem_wait_st();
                }
            }
            // P = exp2(S - m_ref), rounded to the input type, packed in pairs into this quadrant's P columns.
            float sum = 0.0f;
            uint32_t w[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float p0 = exp2f(s[2 * c] - m_ref), p1 = exp2f(s[2 * c + 1] - m_ref);
                sum += p0 + p1;
                if (std::is_same<T, __nv_bfloat16>::value) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    w[c] = *reinterpret_cast<uint32_t *>(&h);
                } else {
                    __half2 h = __floats2half2_rn(p0, p1);
                    w[c] = *reinterpret_cast<uint32_t *>(&h);
                }
            }
            tmem_st16(lane_base + p_col, w);
            l += sum;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&p_full[quad]);
        }
        // ---- merge the four streams and write the rows out ----
        if (ok) {
            l_fin[(quad * 2 + hf) * 32 + lane] = l;
            if (hf == 0) m_fin[quad * 32 + lane] = m_ref;
            mbar_arrive(fin_sync);
            ok = __all_sync(0xffffffffu, mbar_wait(fin_sync, 0, abort_flag));
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(mma_done, 0, abort_flag));  // every accumulator row is final, the rings are idle
        if (ok) {
            tc_fence_after();
            // Row `lane` (one head) over the four quadrants: weights against the common maximum.  Quadrant 0
            // always has a unit, so the maximum is finite; a quadrant without units has m = -inf and weight 0.
            float mm = -INFINITY;
#pragma unroll
            for (int qo = 0; qo < kQuads; ++qo) mm = fmaxf(mm, m_fin[qo * 32 + lane]);
            float lsum = 0.0f, w_own = 0.0f;
#pragma unroll
            for (int qo = 0; qo < kQuads; ++qo) {
                const float mq = m_fin[qo * 32 + lane];
                const float wq = (mq == -INFINITY) ? 0.0f : exp2f(mq - mm);
                lsum += (l_fin[(qo * 2) * 32 + lane] + l_fin[(qo * 2 + 1) * 32 + lane]) * wq;
                if (qo == quad) w_own = wq;
            }
            const float scale = w_own / lsum;
            float *dst_row = stage + (size_t)(quad * 32 + lane) * kStageStride + hf * (D / 2);
#pragma unroll
            for (int c = 0; c < D / 64; ++c) {
                uint32_t ob[32];
                tmem_ld32(lane_base + kColO + hf * (D / 2) + c * 32, ob);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    // (a quadrant without units never had its rows scaled by a finite P: force zeros)
                    const float4 v4 = w_own > 0.0f ? make_float4(__uint_as_float(ob[4 * e]) * scale, __uint_as_float(ob[4 * e + 1]) * scale,
                                                                 __uint_as_float(ob[4 * e + 2]) * scale, __uint_as_float(ob[4 * e + 3]) * scale)
                                                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    *reinterpret_cast<float4 *>(dst_row + c * 32 + 4 * e) = v4;
                }
            }
            tc_fence_before();
            if (quad == 0 && hf == 0 && valid) {
                const float lse = (mm + log2f(lsum)) * kLn2;
                const int h = h0 + lane;
                if (p.num_splits > 1) {
                    p.part_lse[((size_t)b * p.head_q + h) * p.num_splits + split] = lse;
                } else if (p.lse) {
                    p.lse[(size_t)b * p.head_q + h] = lse;
                }
            }
            mbar_arrive(fin_sync);
            ok = __all_sync(0xffffffffu, mbar_wait(fin_sync, 1, abort_flag));
        }
        if (ok) {
            // 256 threads sum the four staged copies of every head's row and store it, 4 columns at a time.
            const int quads_per_row = dreal / 4;
            for (int idx = tid; idx < G * quads_per_row; idx += kSoftmaxThreads) {
                const int hl = idx / quads_per_row, d0 = (idx % quads_per_row) * 4;
                float4 acc = *reinterpret_cast<const float4 *>(stage + (size_t)hl * kStageStride + d0);
#pragma unroll
                for (int qo = 1; qo < kQuads; ++qo) {
                    const float4 x = *reinterpret_cast<const float4 *>(stage + (size_t)(qo * 32 + hl) * kStageStride + d0);
                    acc.x += x.x, acc.y += x.y, acc.z += x.z, acc.w += x.w;
                }
                const int h = h0 + hl;
                if (p.num_splits > 1) {
                    const size_t row = ((size_t)b * p.head_q + h) * p.num_splits + split;
                    *reinterpret_cast<float4 *>(p.part_o + row * dreal + d0) = acc;
                } else {
                    if (o_out) {
                        alignas(8) T tmp[4] = {from_float<T>(acc.x), from_float<T>(acc.y), from_float<T>(acc.z), from_float<T>(acc.w)};
                        *reinterpret_cast<uint2 *>(o_out + (size_t)b * p.o_row_stride + (size_t)h * dreal + d0) = *reinterpret_cast<uint2 *>(tmp);
                    }
                    if (p.o_f32) *reinterpret_cast<float4 *>(p.o_f32 + ((size_t)b * p.head_q + h) * dreal + d0) = acc;
                }
            }
        }
    }

    if (!ok && lane == 0) report_timeout(p);
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int D>
cudaError_t launch_d(bool bf16, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k, cudaStream_t stream) {
    using C = QuadCfg<D>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !attr_set[dev]) {
        const void *kernels[4] = {(const void *)da_gqa_quad_kernel<__half, D, false>, (const void *)da_gqa_quad_kernel<__half, D, true>,
                                  (const void *)da_gqa_quad_kernel<__nv_bfloat16, D, false>,
                                  (const void *)da_gqa_quad_kernel<__nv_bfloat16, D, true>};
        for (const void *k : kernels) {
            err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
            if (err != cudaSuccess) return err;
        }
        attr_set[dev] = true;
    }
    dim3 grid(p.num_splits, p.head_k, p.batch);
    const bool overlap = p.batch_order != nullptr;
    const bool short_pages = p.block_table && (1 << p.page_shift) < kUnit;
    if (bf16) {
        return short_pages ? launch_kernel(da_gqa_quad_kernel<__nv_bfloat16, D, true>, grid, kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k)
                           : launch_kernel(da_gqa_quad_kernel<__nv_bfloat16, D, false>, grid, kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k);
    }
    return short_pages ? launch_kernel(da_gqa_quad_kernel<__half, D, true>, grid, kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k)
                       : launch_kernel(da_gqa_quad_kernel<__half, D, false>, grid, kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k);
}
}  // namespace

SplitVariantInfo split_info_gqa_quad() { return {kUnit, 32, 1}; }

// tm_q: rank-3 map of q [batch][head_q][dim], box {64, min(32, head_q), 1}; tm_k: rank-3 map
// [rows][head_k][dim], box {64, 1, 64 keys (or a page)}; both with the 128-byte swizzle (V needs no map).
// dim: 64 or 128 (96 runs as 128); at most 32 query heads per KV head.
cudaError_t launch_gqa_quad(bool bf16, int dim, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                            cudaStream_t stream) {
    if (p.group > 32) return cudaErrorInvalidValue;
    switch (dim) {
        case 64: return launch_d<64>(bf16, p, tm_q, tm_k, stream);
        case 128: return launch_d<128>(bf16, p, tm_q, tm_k, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace da
