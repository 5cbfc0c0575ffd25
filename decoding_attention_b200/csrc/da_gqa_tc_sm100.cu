// Grouped-query / multi-query decode attention (head dims 64, 96, 128, 256) on the sm_100a tensor cores,
// for KV heads that serve a group of query heads the CUDA-core kernel handles badly (more than 4, or
// not 1, 2 or 4; at most 128).
//
// With G query heads per KV head the path does 2*G flops per KV byte.  On CUDA cores
// (da_split_kernel.cuh, at most 4 heads per CTA) G = 32 is bound by instruction issue at about a
// tenth of the HBM rate -- the reference has the same shape of problem, one CTA per query head
// (csrc/kernel/decoding_attn/decoding_fwd_hd128_hdv128.cu:9-25).  Here the G heads of one KV head are
// rows of an M = 128 tcgen05.mma tile (rows >= G compute garbage that nobody reads; the tensor
// pipe is otherwise idle), so every K/V byte is read once and used for all G heads; for head dim D
//     S[128 x 64] = Q[128 x D] . K_tile[64 x D]^T      (D/16 MMAs  M128 N64 K16, operands K-major)
//     O[128 x D] += P[128 x 64] . V_tile[64 x D]        (4 MMAs     M128 N=D K16, V MN-major)
// One CTA = (sequence, KV head, key range).  Q, K and V tiles arrive by tiled TMA copies with the
// 128-byte swizzle; S (two buffers) and O live in tensor memory.
// Softmax/epilogue warps: a warp can only reach the TMEM lanes of its quadrant (warp % 4), so
// several warps share each block of 32 rows and split the 64 score columns (and the output columns)
// between them: with few valid rows per tile the softmax, not the tensor pipe, sets the pace, and
// its latency is per-thread serial work.  The threads of a row agree on the row maximum through
// shared memory once per tile.  Quadrants whose rows are all >= G stay out.
// Dims 64 and 128 run two independent softmax streams (even / odd tiles, one accumulator each,
// merged at the end): 16 softmax warps.  Dim 256 has room for one accumulator only and runs one
// stream over both S buffers: 8 softmax warps; its 64 KB tiles outlast a tile's softmax chain.
// Then one TMA producer warp, one warp for TMEM allocation + issue of S, one for the issue of P.V.  Lazy reference max as
// in the MLA kernel.  Every wait is bounded (the per-tile rendezvous of the softmax threads is an
// mbarrier).
#include <type_traits>

#include "da_internal.h"
#include "da_tcgen05.cuh"

namespace da {
namespace {

constexpr int kRows = 128;                            // M of both contractions (G valid rows)
constexpr int kTile = 64;                             // keys per tile
constexpr int kQBlockBytes = kRows * 128;             // [128 heads x 64 dims]
constexpr int kKBlockBytes = kTile * 128;             // [64 keys x 64 dims]
constexpr int kPBytes = kRows * kTile * 2;
constexpr int kColsPer = 32;                          // score columns per thread
constexpr int kTmemCols = 512;
constexpr int kColS = 0;      // 2 x 64: the two S buffers
constexpr int kColO = 128;    // one accumulator of D columns per stream

// Per head dim D: 64 and 128 run two softmax streams (two accumulators of D columns), 256 runs one (its
// 64 KB tiles keep the pipe and the memory system busy longer than the softmax chain of a tile takes).
template <int D>
struct GqaCfg {
    static constexpr int kBlocks = D / 64;                    // 64-element (128-byte) column blocks of a row
    static constexpr int kStreams = D <= 128 ? 2 : 1;
    static constexpr int kStages = D == 64 ? 8 : (D == 128 ? 4 : 2);
    static constexpr int kKStageBytes = kBlocks * kKBlockBytes;  // K tile; the V tile has the same size
    static constexpr int kColSplit = 2 * kStreams;            // softmax threads per row: streams x 2 column halves
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + kBlocks * kQBlockBytes;
    static constexpr int kOffV = kOffK + kStages * kKStageBytes;
    static constexpr int kOffP = kOffV + kStages * kKStageBytes;
    static constexpr int kOffRowMax = kOffP + kStreams * kPBytes;  // partial row maxima / sums, stream maxima
    static constexpr int kOffBar = kOffRowMax + 2 * kColSplit * kRows * 4 + 1024;
    // q_full, kv_full/kv_empty[kStages], s_full[2], s_empty[2], p_full[2], pv_done[2], row_sync[2], fin_sync
    static constexpr int kNumBars = 1 + 2 * kStages + 11;
    static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;
    static constexpr int kSoftmaxWarps = 4 * kColSplit;
    static constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1, kPvWarp = kSoftmaxWarps + 2;
    static constexpr int kThreads = (kSoftmaxWarps + 3) * 32;
    static constexpr int kOutPer = D / kColSplit;             // output columns per thread in the epilogue
    static_assert(D == 64 || D == 128 || D == 256, "head dim");
    static_assert(kColO + kStreams * D <= kTmemCols, "TMEM budget");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};
constexpr float kRescaleThreshold = 8.0f;


// kShortPages: the cache is paged with pages shorter than a key tile, which is then fetched page by page
// (a separate instantiation, so that the common case keeps its straight-line address arithmetic).
template <typename T, int D, bool kShortPages>
__global__ void __launch_bounds__(GqaCfg<D>::kThreads, 1)
da_gqa_tc_kernel(const SplitParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v) {
    using C = GqaCfg<D>;
    constexpr int kDim = D, kBlocks = C::kBlocks, kStreams = C::kStreams, kStages = C::kStages, kKStageBytes = C::kKStageBytes;
    constexpr int kColSplit = C::kColSplit, kThreads = C::kThreads, kProducerWarp = C::kProducerWarp, kMmaWarp = C::kMmaWarp;
    constexpr int kOffQ = C::kOffQ, kOffK = C::kOffK, kOffV = C::kOffV, kOffP = C::kOffP, kOffRowMax = C::kOffRowMax;
    constexpr int kOffBar = C::kOffBar, kNumBars = C::kNumBars, kOutPer = C::kOutPer;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    pdl_launch_dependents();  // the merge kernel may be scheduled behind this grid's last CTAs
    const int split = blockIdx.x;
    const int hk = blockIdx.y;
    if (p.batch_order) pdl_wait();  // written by the order kernel launched just before this one
    const int b = p.batch_order ? p.batch_order[blockIdx.z] : (int)blockIdx.z;
    const int G = p.group;            // query heads of this KV head: rows 0..G-1 of the tile
    const int h0 = hk * G;
    // The head dim the caller's tensors have.  It equals D except for head dim 96, which runs on the D = 128
    // instantiation: the tensor maps declare 96 columns, so the second 64-column box of every row arrives with
    // its last 32 columns zero-filled, S and O come out as for 128 columns of which the last 32 are zero.
    const int dreal = p.dim;
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
    const int n_tiles = (k_end - k_begin + kTile - 1) / kTile;
    // With ALiBi the bias, and with it every head's row maximum, grows towards the end of the sequence: walked
    // front to back, every tile would raise the reference maximum of the steep heads and take the rescale path.
    // Walked back to front the first tiles set the maximum.  `tile_of(t)` is the tile the t-th step works on.
    const bool backwards = p.is_alibi != 0;
    auto tile_of = [&](int t) { return backwards ? n_tiles - 1 - t : t; };
    const int active_quads = (G + 31) / 32;                   // 32-row blocks that hold valid rows
    const int participants = active_quads * 2 * 32;           // softmax threads at work on one stream

    uint8_t *q_s = smem + kOffQ;
    uint8_t *k_s = smem + kOffK;
    uint8_t *v_s = smem + kOffV;
    uint8_t *p_s = smem + kOffP;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    uint64_t *q_full = bars;
    uint64_t *kv_full = bars + 1;
    uint64_t *kv_empty = kv_full + kStages;
    uint64_t *s_full = kv_empty + kStages;
    uint64_t *s_empty = s_full + 2;
    uint64_t *p_full = s_empty + 2;
    uint64_t *pv_done = p_full + 2;
    uint64_t *row_sync = pv_done + 2;
    uint64_t *fin_sync = row_sync + 2;
    float *rowmax_s = reinterpret_cast<float *>(smem + kOffRowMax);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_empty[s], participants);
            mbar_init(&p_full[s], participants);
            mbar_init(&pv_done[s], 1);
            mbar_init(&row_sync[s], participants);
        }
        mbar_init(fin_sync, kStreams * participants);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kMmaWarp) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr uint32_t kIdescQK = instr_desc(kFmt, 0, kRows, kTile);
    constexpr uint32_t kIdescPV = instr_desc(kFmt, 1, kRows, kDim);
    bool ok = true;

    if (warp == kProducerWarp) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            tma_prefetch_desc(&tm_v);
            // Rows h0 .. h0+127 of q: rows past this KV head's group (or past head_q: zero-filled) only
            // feed tile rows that are never read back.
            // (the map's box holds min(128, head_q) rows; the transaction count is the box size).
            mbar_arrive_expect_tx(q_full, kBlocks * min(kRows, p.head_q) * 128);
            for (int kb = 0; kb < kBlocks; ++kb) tma_load_tile_3d(q_s + kb * kQBlockBytes, &tm_q, kb * 64, h0, b, q_full);
        }
        const T *k_g = reinterpret_cast<const T *>(p.k) + (size_t)hk * dreal;
        const T *v_g = reinterpret_cast<const T *>(p.v) + (size_t)hk * dreal;
        const int run = kShortPages ? kv_run_keys(p, kTile) : kTile;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int st = t % kStages;
            const uint32_t ph = (uint32_t)(t / kStages) & 1u;
            const int key0 = k_begin + tile_of(t) * kTile;
            const int rows = min(kTile, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            auto row_of = [&](int r) { return kShortPages ? kv_tile_row(p, b, seq_begin, key0 + r) : tok0 + r; };
            if (t >= kStages) ok = mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag);
            if (!ok) break;
            uint8_t *kd = k_s + st * kKStageBytes, *vd = v_s + st * kKStageBytes;
            if (rows == kTile) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(&kv_full[st], 2 * kKStageBytes);
                    for (int k0 = 0; k0 < kTile; k0 += run) {  // one box per run of consecutive rows (a page, or the tile)
                        const int row = (int)row_of(k0);
                        for (int kb = 0; kb < kBlocks; ++kb) {
                            tma_load_tile_3d(kd + kb * kKBlockBytes + k0 * 128, &tm_k, kb * 64, hk, row, &kv_full[st]);
                            tma_load_tile_3d(vd + kb * kKBlockBytes + k0 * 128, &tm_v, kb * 64, hk, row, &kv_full[st]);
                        }
                    }
                }
            } else {
                // Ragged tail: 16-byte cp.async into the 128-byte-swizzled layout, rows past the end and columns past
                // the real head dim zero-filled (the tensor maps must not be asked for rows beyond the sequence).
                // All of the warp's copies are in flight at once: one memory latency, where a loop of loads and
                // stores took 2-3 us, on the one tile the whole CTA waits for.
                constexpr int kChunks = kDim / 8;  // 16-byte chunks per row
                for (int i = lane; i < kTile * kChunks; i += 32) {
                    const int r = i / kChunks, c = i % kChunks;
                    const bool real = r < rows && c * 8 < dreal;
                    const size_t row = row_of(real ? r : 0);
                    const int col = real ? c * 8 : 0;
                    const int off = (c >> 3) * kKBlockBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                    cp_async16(kd + off, k_g + row * p.k_row_stride + col, real ? 16u : 0u);
                    cp_async16(vd + off, v_g + row * p.v_row_stride + col, real ? 16u : 0u);
                }
                cp_async_commit();
                cp_async_wait<0>();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&kv_full[st]);
            }
            __syncwarp();
        }
    } else if (warp == kMmaWarp) {
        // ---------------- issuer of S = Q.K^T ----------------
        // S and P.V have an issuing warp each (this one and kPvWarp): with contractions this small the issue loop --
        // barrier waits, commits -- sets the pace, and one warp doing both needed about 1 500 cycles per tile.
        const uint32_t leader = elect_one();
        const uint64_t q_desc0 = smem_desc(smem_u32(q_s), 16, 1024, 2);  // K-major, 8-row groups 1 KB apart
        const uint64_t k_desc0 = smem_desc(smem_u32(k_s), 16, 1024, 2);
        ok = mbar_wait(q_full, 0, abort_flag);
        for (int t = 0; t < n_tiles && ok; ++t) {
            ok = mbar_wait(&kv_full[t % kStages], (uint32_t)(t / kStages) & 1u, abort_flag);
            if (ok && t >= 2) ok = mbar_wait(&s_empty[t & 1], ((uint32_t)(t / 2) & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t kd = k_desc0 + (uint64_t)(((t % kStages) * kKStageBytes) >> 4);
            const uint32_t d = tmem_base + kColS + (t & 1) * kTile;
#pragma unroll
            for (int kb = 0; kb < kBlocks; ++kb) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    umma_ss(d, q_desc0 + (uint64_t)((kb * kQBlockBytes + ks * 32) >> 4),
                            kd + (uint64_t)((kb * kKBlockBytes + ks * 32) >> 4), kIdescQK, (kb | ks) ? 1u : 0u, leader);
                }
            }
            umma_commit(&s_full[t & 1], leader);
        }
        __syncwarp();
    } else if (warp == C::kPvWarp) {
        // ---------------- issuer of O += P.V ----------------
        const uint32_t leader = elect_one();
        const uint64_t v_desc0 = smem_desc(smem_u32(v_s), kKBlockBytes, 1024, 2);  // MN-major: 64-col blocks LBO apart
        const uint64_t p_desc0 = smem_desc(smem_u32(p_s), kRows * 16, 128, 0);     // core matrices, 8-key chunks 2 KB apart
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int st = t % kStages;
            ok = mbar_wait(&p_full[t & 1], (uint32_t)(t / 2) & 1u, abort_flag);
            if (ok) ok = mbar_wait(&kv_full[st], (uint32_t)(t / kStages) & 1u, abort_flag);  // (long complete: this warp's own view of the V tile)
            if (!ok) break;
            tc_fence_after();
            const uint64_t pd = p_desc0 + (uint64_t)((((kStreams == 2) ? (t & 1) : 0) * kPBytes) >> 4);
            const uint64_t vd = v_desc0 + (uint64_t)((st * kKStageBytes) >> 4);
#pragma unroll
            for (int ks = 0; ks < kTile / 16; ++ks) {
                umma_ss(tmem_base + kColO + ((kStreams == 2) ? (t & 1) : 0) * kDim, pd + (uint64_t)((ks * 2 * (kRows * 16)) >> 4),
                        vd + (uint64_t)((ks * 16 * 128) >> 4), kIdescPV, (t >= kStreams || ks > 0) ? 1u : 0u, leader);
            }
            umma_commit(&kv_empty[st], leader);
            umma_commit(&pv_done[t & 1], leader);
        }
        __syncwarp();
    } else if ((warp & 3) < active_quads) {
        // ------- softmax / epilogue -------
        // Two independent online-softmax streams run interleaved: even tiles (S buffer 0, P buffer 0,
        // accumulator O0) and odd tiles (buffer 1, O1), each with its own reference max and sum; they
        // are merged at the end like two key-range splits.  That keeps two tiles' worth of the
        // (latency-bound) softmax chain in flight.  Thread (quad, strm, hf, lane) owns row 32 quad + lane
        // of stream strm and its score columns [32 hf, +32).
        const int quad = warp & 3, cp = warp >> 2, strm = (kStreams == 2) ? (cp >> 1) : 0, hf = cp & 1;
        const int r = quad * 32 + lane;
        const bool valid = r < G;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t o_col = kColO + strm * kDim;
        const float slope2 = p.is_alibi ? exp2f(-8.0f * (float)(h0 + r + 1) / (float)p.head_q) * kLog2e : 0.0f;
        const int pos_shift = (p.kv_pos_offset ? p.kv_pos_offset[b] : 0) - ((p.kv_total_len ? p.kv_total_len[b] : len) - 1);
        float m_ref = -INFINITY, l = 0.0f;
        uint32_t buf[32];
        float *rm = rowmax_s + strm * (2 * kRows);  // [2 halves][128] partial row maxima of this stream
        int last_t = -1;
        int n_done = 0;  // tiles this thread has finished (use count of its stream's row_sync barrier)
        for (int t = strm; t < n_tiles; t += kStreams, ++n_done) {
            const int sb = (kStreams == 2) ? strm : (t & 1);  // S buffer of this tile (= t & 1) and the barriers that go with it
            const int it = t >> 1;  // use count of those barriers
            const int key0 = k_begin + tile_of(t) * kTile + hf * kColsPer;
            const int rows = min(kTile, k_end - (k_begin + tile_of(t) * kTile)) - hf * kColsPer;  // valid columns of this thread
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[sb], (uint32_t)it & 1u, abort_flag));
            if (!ok) break;
            tc_fence_after();
            tmem_ld32(lane_base + kColS + sb * kTile + hf * kColsPer, buf);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&s_empty[sb]);
            float s[kColsPer];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < kColsPer; ++j) {
                const float x = __uint_as_float(buf[j]) * p.scale_log2 + slope2 * (float)(key0 + j + pos_shift);
                s[j] = (j < rows) ? x : -INFINITY;
                mx = fmaxf(mx, s[j]);
            }
            // The two threads of a row agree on the tile's row maximum.
            rm[hf * kRows + r] = mx;
            mbar_arrive(&row_sync[strm]);
            ok = __all_sync(0xffffffffu, mbar_wait(&row_sync[strm], (uint32_t)n_done & 1u, abort_flag));
            if (!ok) break;
            mx = fmaxf(mx, rm[(hf ^ 1) * kRows + r]);
            const bool raise = mx > m_ref + kRescaleThreshold;
            float alpha = 1.0f;
            if (raise) {
                alpha = exp2f(m_ref - mx);  // 0 on the stream's first tile
                m_ref = mx;
                l *= alpha;
            }
            if (n_done >= 1) {
                // This stream's previous P.V (tile t - kStreams) has finished: its P buffer and its accumulator are idle.
                const int tp = t - kStreams;
                ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(kStreams == 2) ? strm : (tp & 1)], (uint32_t)(tp >> 1) & 1u, abort_flag));
                if (!ok) break;
                if (__any_sync(0xffffffffu, raise && valid)) {
                    // Rare: the reference max of some row of this quadrant moved; rescale this thread's half
                    // of the row's accumulator columns in place.
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < kDim / 64; ++c) {
                        uint32_t ob[32];
                        tmem_ld32(lane_base + o_col + hf * (kDim / 2) + c * 32, ob);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) ob[j] = __float_as_uint(__uint_as_float(ob[j]) * alpha);
                        tmem_st32(lane_base + o_col + hf * (kDim / 2) + c * 32, ob);
                    }
                    tmem_wait_st();
                }
            }
            // P = exp2(S - m_ref), rounded to the input type, into the A-operand layout (8-key chunks).
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < kColsPer / 8; ++c) {
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
                *reinterpret_cast<uint4 *>(p_s + strm * kPBytes + (hf * (kColsPer / 8) + c) * (kRows * 16) + r * 16) =
                    make_uint4(w[0], w[1], w[2], w[3]);
            }
            l += sum;
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&p_full[sb]);
            last_t = t;
        }
        // ---- merge the streams and write the row out ----
        float *l_part = rowmax_s + kStreams * 2 * kRows;  // [kColSplit threads of a row][128]
        float *m_strm = l_part + kColSplit * kRows;        // [kStreams][128]
        if (ok) {
            l_part[cp * kRows + r] = l;
            if (hf == 0) m_strm[strm * kRows + r] = m_ref;
            mbar_arrive(fin_sync);
            ok = __all_sync(0xffffffffu, mbar_wait(fin_sync, 0, abort_flag));
        }
        // every accumulator must be final: the last P.V that went through either S buffer
        for (int sb = 0; sb < 2 && ok; ++sb) {
            const int last = ((n_tiles - 1) & 1) == sb ? n_tiles - 1 : n_tiles - 2;
            if (last >= 0) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[sb], (uint32_t)(last >> 1) & 1u, abort_flag));
        }
        (void)last_t;
        if (ok) {
            tc_fence_after();
            const float m0 = m_strm[r];
            const float m1 = (kStreams == 2) ? m_strm[kRows + r] : -INFINITY;
            const float l0 = l_part[0 * kRows + r] + l_part[1 * kRows + r];
            const float l1 = (kStreams == 2) ? l_part[2 * kRows + r] + l_part[3 * kRows + r] : 0.0f;
            const float mm = fmaxf(m0, m1);                      // stream 0 always has a tile: finite
            const float w0 = exp2f(m0 - mm), w1 = (m1 == -INFINITY) ? 0.0f : exp2f(m1 - mm);
            const float lsum = l0 * w0 + l1 * w1;
            const float inv = 1.0f / lsum;
            const float lse = (mm + log2f(lsum)) * kLn2;
            const int h = h0 + r;
            const size_t row = ((size_t)b * p.head_q + h) * p.num_splits + split;
            constexpr int CW = kOutPer < 32 ? kOutPer : 32;  // columns per TMEM load: 16 (dim 64) or 32
#pragma unroll
            for (int c = 0; c < kOutPer / CW; ++c) {
                const int d0 = cp * kOutPer + c * CW;  // this thread's output columns [d0, d0 + CW)
                float out[CW];
                uint32_t oa[CW], ob[CW];
                if constexpr (CW == 32) {
                    tmem_ld32(lane_base + kColO + d0, oa);                          // stream 0
                    if (kStreams == 2) tmem_ld32(lane_base + kColO + kDim + d0, ob);  // stream 1 (never written if it had no tile)
                } else {
                    tmem_ld16(lane_base + kColO + d0, oa);
                    if (kStreams == 2) tmem_ld16(lane_base + kColO + kDim + d0, ob);
                }
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < CW; ++j) {
                    const float a0 = __uint_as_float(oa[j]) * w0;
                    const float a1 = (kStreams == 2 && w1 > 0.0f) ? __uint_as_float(ob[j]) * w1 : 0.0f;
                    out[j] = (a0 + a1) * inv;
                }
                if (!valid || d0 >= dreal) continue;  // (a head dim run padded has whole column groups of zeros)
                if (p.num_splits > 1) {
                    float4 *dst = reinterpret_cast<float4 *>(p.part_o + row * dreal + d0);
#pragma unroll
                    for (int j = 0; j < CW / 4; ++j) dst[j] = make_float4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
                } else {
                    if (o_out) {
                        uint4 *dst = reinterpret_cast<uint4 *>(o_out + (size_t)b * p.o_row_stride + (size_t)h * dreal + d0);
#pragma unroll
                        for (int j = 0; j < CW / 8; ++j) {
                            alignas(16) T tmp[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) tmp[e] = from_float<T>(out[8 * j + e]);
                            dst[j] = *reinterpret_cast<uint4 *>(tmp);
                        }
                    }
                    if (p.o_f32) {
                        float *dst = p.o_f32 + ((size_t)b * p.head_q + h) * dreal + d0;
#pragma unroll
                        for (int j = 0; j < CW; ++j) dst[j] = out[j];
                    }
                }
            }
            if (valid && cp == 0) {
                if (p.num_splits > 1) {
                    p.part_lse[row] = lse;
                } else if (p.lse) {
                    p.lse[(size_t)b * p.head_q + h] = lse;
                }
            }
            tc_fence_before();
        }
    }

    if (!ok && lane == 0) report_timeout(p);
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace


SplitVariantInfo split_info_gqa_tc() { return {kTile, kRows, 1}; }

namespace {
template <int D>
cudaError_t launch_d(bool bf16, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k, const CUtensorMap &tm_v,
                     cudaStream_t stream) {
    using C = GqaCfg<D>;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !attr_set[dev]) {
        const void *kernels[4] = {(const void *)da_gqa_tc_kernel<__half, D, false>, (const void *)da_gqa_tc_kernel<__half, D, true>,
                                  (const void *)da_gqa_tc_kernel<__nv_bfloat16, D, false>,
                                  (const void *)da_gqa_tc_kernel<__nv_bfloat16, D, true>};
        for (const void *k : kernels) {
            err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
            if (err != cudaSuccess) return err;
        }
        attr_set[dev] = true;
    }
    dim3 grid(p.num_splits, p.head_k, p.batch);
    const bool overlap = p.batch_order != nullptr;
    const bool short_pages = p.block_table && (1 << p.page_shift) < kTile;
    if (bf16) {
        return short_pages ? launch_kernel(da_gqa_tc_kernel<__nv_bfloat16, D, true>, grid, C::kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k, tm_v)
                           : launch_kernel(da_gqa_tc_kernel<__nv_bfloat16, D, false>, grid, C::kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k, tm_v);
    }
    return short_pages ? launch_kernel(da_gqa_tc_kernel<__half, D, true>, grid, C::kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k, tm_v)
                       : launch_kernel(da_gqa_tc_kernel<__half, D, false>, grid, C::kThreads, C::kSmemBytes, stream, overlap, p, tm_q, tm_k, tm_v);
}
}  // namespace

// tm_q: rank-3 map of q [batch][head_q][dim], box {64, min(128, head_q), 1}; tm_k / tm_v: rank-3 maps
// [rows][head_k][dim], box {64, 1, 64 keys}; all with the 128-byte swizzle.  dim: 64, 128 or 256.
cudaError_t launch_gqa_tc(bool bf16, int dim, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                          const CUtensorMap &tm_v, cudaStream_t stream) {
    switch (dim) {
        case 64: return launch_d<64>(bf16, p, tm_q, tm_k, tm_v, stream);
        case 128: return launch_d<128>(bf16, p, tm_q, tm_k, tm_v, stream);
        case 256: return launch_d<256>(bf16, p, tm_q, tm_k, tm_v, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace da
