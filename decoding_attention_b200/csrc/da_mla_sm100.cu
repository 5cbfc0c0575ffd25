// Latent-KV (MLA) decode attention on the sm_100a tensor cores: tcgen05.mma with accumulators in
// tensor memory (TMEM), operands staged by TMA.
//
// Shape: up to 128 query heads (rows past head_q are padding) share one KV head whose rows hold 576
// values; V is the first 512 of them
// (the reference runs this shape through its generic kernel, one CTA per query head:
// csrc/kernel/decoding_attn/decoding_fwd_hd576_hdv512.cu:9-17, so every K row is fetched 128
// times).  Here the 128 heads are the M dimension of two dense contractions per 64-key tile:
//     S[128 x 64]   = Q[128 x 576] . K_tile[64 x 576]^T         (both operands K-major)
//     O[128 x 256] += P[128 x 64]  . V_tile[64 x 256]            (V = the same smem bytes, MN-major)
// TMEM holds 128 lanes x 512 fp32 columns, which the 128 x 512 output alone would fill, so one CTA
// owns one half of the output columns (256 TMEM columns); the two CTAs of a (sequence, key range)
// each compute S themselves and never talk to each other.
//
// An M=128 tcgen05.mma step costs the same for N = 64 keys as for N = 32, so tiles are 64 keys.  A
// 64-key tile is 72 KB and Q is 144 KB, more than shared memory holds twice over, hence:
//   * Q: four 64-column blocks live in TMEM (A operand read from TMEM), five in shared memory;
//   * P never touches shared memory: it is written over its own S columns in TMEM (16-bit pairs)
//     and read from there as the A operand of P.V;
//   * K tiles are not staged whole.  Of the nine 64-column blocks of a tile only the four that make
//     up this CTA's half of V are needed again for P.V; they go to a ring of three 32 KB slots.  The
//     other five are dead once S has consumed them and stream through a ring of six 8 KB slots,
//     each released by a tcgen05.commit right after its four MMAs.
// TMEM columns: S0 | S1 (64 each, P aliased) | O (256) | Q (4 x 32).
//
// Warp roles (320 threads): warps 0-3 = softmax/epilogue, thread r owns TMEM lane r = head r, so
// row maxima, sums and the rare rescale of O need no cross-thread traffic; warp 4 = TMA producer
// (Q and the streamed blocks); warp 5 = TMEM allocation and MMA issue (one elected lane); warps
// 6-9 = loaders of the V quarter-tiles with 16-byte cp.async, because one SM's TMA engine alone
// moves only about 21 B/clk.  The MMA pipe executes in issue
// order S(0) S(1) PV(0) S(2) PV(1) ..., which is what makes the S/P aliasing safe: S(t+2) is issued
// after PV(t), and PV(t) after the softmax threads have replaced S(t) by P(t).
// Online softmax with a lazy reference: the running reference max m_ref of a row is only raised
// when a score exceeds it by more than 8 (log2 domain), so O is rescaled a handful of times.
// Every wait is bounded; on expiry the CTA records kStatusWaitTimeout and still frees its TMEM.
#include <type_traits>

#include "da_internal.h"
#include "da_tcgen05.cuh"

namespace da {
namespace {

constexpr int kHeads = 128;       // M of both contractions
constexpr int kDim = 576;         // K of S = Q K^T
constexpr int kDimV = 512;
constexpr int kHalfV = 256;       // output columns per CTA
constexpr int kTile = 64;         // keys per tile (N of S, K of O)
constexpr int kBlocks = kDim / 64;                    // 64-element (128-byte) column blocks of a row
constexpr int kVBlocks = 4;                           // blocks of a tile that are this CTA's V columns
constexpr int kABlocks = kBlocks - kVBlocks;          // blocks only S needs
constexpr int kQTmemBlocks = 4;   // Q blocks kept in TMEM: those that meet the first four streamed blocks
constexpr int kQSmemBlocks = kBlocks - kQTmemBlocks;
constexpr int kQBlockBytes = kHeads * 128;            // 16 KB: [128 heads x 64 dims], 128B-swizzled
constexpr int kKBlockBytes = kTile * 128;             // 8 KB: [64 keys x 64 dims], 128B-swizzled
constexpr int kASlots = 6;                            // ring of streamed blocks
constexpr int kVSlots = 3;                            // ring of V quarter-tiles
constexpr int kVSlotBytes = kVBlocks * kKBlockBytes;
constexpr int kOffQ = 0;
constexpr int kOffA = kOffQ + kQSmemBlocks * kQBlockBytes;
constexpr int kOffV = kOffA + kASlots * kKBlockBytes;
constexpr int kOffBar = kOffV + kVSlots * kVSlotBytes;
// q_full, q_tmem, a_full/a_empty[kASlots], v_full/v_empty[kVSlots], s_full[2], p_full[2], pv_done[2]
constexpr int kNumBars = 2 + 2 * kASlots + 2 * kVSlots + 2 + 2 + 2;
constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16 + 1024;  // + tmem slot/abort flag + alignment slack
constexpr int kLoaderWarps = 4;                       // warps that fetch the V quarter-tiles through the load/store unit
constexpr int kLoaderThreads = kLoaderWarps * 32;
constexpr int kThreads = 192 + kLoaderThreads;
constexpr int kTmemCols = 512;
constexpr int kColS = 0;      // two S buffers of kTile columns; P(t) overwrites the first half of S(t)
constexpr int kColO = 128;    // 256 output columns
constexpr int kColQ = 384;    // kQTmemBlocks * 32 columns: Q as packed 16-bit pairs, row r in lane r
static_assert(kColQ + kQTmemBlocks * 32 <= kTmemCols, "TMEM budget");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
constexpr float kRescaleThreshold = 8.0f;

// Column block of the j-th streamed block (j < kABlocks) and of the j-th V block for output half h.
__device__ __forceinline__ int a_block(int h, int j) { return j < 4 ? (h ? j : 4 + j) : 8; }
__device__ __forceinline__ int v_block(int h, int j) { return 4 * h + j; }


// One [64 keys x 64 dims] block of the latent cache into a 128-byte-swizzled 8 KB slot.  Whole
// tiles go by TMA (lane 0 issues; the bytes are counted on `bar`, whose expect_tx the caller has
// posted); a ragged last tile is read with plain loads, rows past the end zeroed, because the
// tensor map must not be asked for rows beyond the sequence.
template <typename T, typename RowOf>
__device__ __forceinline__ void load_block(uint8_t *dst, const CUtensorMap *tm, const T *k_g, size_t k_row_stride, int block,
                                           RowOf row_of, int run, int rows, uint64_t *bar, int lane) {
    if (rows == kTile) {
        if (lane == 0) {
            for (int k0 = 0; k0 < kTile; k0 += run) tma_load_2d(dst + k0 * 128, tm, block * 64, (int)row_of(k0), bar);
        }
    } else {
        for (int i = lane; i < kTile * 8; i += 32) {
            const int r = i >> 3, cc = i & 7;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows) v = *reinterpret_cast<const uint4 *>(k_g + row_of(r) * k_row_stride + block * 64 + cc * 8);
            *reinterpret_cast<uint4 *>(dst + r * 128 + ((cc ^ (r & 7)) << 4)) = v;
        }
    }
}

// kShortPages: the cache is paged with pages shorter than a key tile, which is then fetched page by page.
// A separate instantiation, so that the common case keeps its straight-line address arithmetic.
template <typename T, bool kShortPages>
__global__ void __launch_bounds__(kThreads, 1)
da_mla_tc_kernel(const SplitParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    pdl_launch_dependents();  // the merge kernel may be scheduled behind this grid's last CTAs
    const int split = blockIdx.x;
    const int half = blockIdx.y;  // which 256 output columns
    if (p.batch_order) pdl_wait();  // written by the order kernel launched just before this one
    const int b = p.batch_order ? p.batch_order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq_begin = p.cu_seq_k[b];
    const int len = p.cu_seq_k[b + 1] - seq_begin;
    const int k_begin = split * p.chunk_keys;
    const int k_end = split_key_end(p, split, len);
    T *o_out = reinterpret_cast<T *>(p.o);
    if (launch_aborted(p)) return;  // an earlier CTA of this launch timed out: do not pile up

    if (k_begin >= k_end) {
        if (p.num_splits == 1) {  // empty sequence: zero row, LSE = -inf
            for (int idx = tid; idx < p.head_q * kHalfV; idx += kThreads) {
                const int h = idx / kHalfV, d = half * kHalfV + idx % kHalfV;
                if (o_out) o_out[(size_t)b * p.o_row_stride + (size_t)h * kDimV + d] = from_float<T>(0.0f);
                if (p.o_f32) p.o_f32[((size_t)b * p.head_q + h) * kDimV + d] = 0.0f;
            }
            if (p.lse && half == 0 && tid < p.head_q) p.lse[(size_t)b * p.head_q + tid] = -INFINITY;
        }
        return;
    }
    const int n_tiles = (k_end - k_begin + kTile - 1) / kTile;

    uint8_t *q_s = smem + kOffQ;
    uint8_t *a_s = smem + kOffA;
    uint8_t *v_s = smem + kOffV;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    uint64_t *q_full = bars;
    uint64_t *q_tmem = bars + 1;
    uint64_t *a_full = bars + 2;
    uint64_t *a_empty = a_full + kASlots;
    uint64_t *v_full = a_empty + kASlots;
    uint64_t *v_empty = v_full + kVSlots;
    uint64_t *s_full = v_empty + kVSlots;
    uint64_t *p_full = s_full + 2;
    uint64_t *pv_done = p_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBars);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (tid == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_tmem, kHeads);
        for (int s = 0; s < kASlots; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < kVSlots; ++s) {
            mbar_init(&v_full[s], kLoaderThreads);
            mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], kHeads);
            mbar_init(&pv_done[s], 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr uint32_t kFmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr uint32_t kIdescQK = instr_desc(kFmt, 0, kHeads, kTile);
    constexpr uint32_t kIdescPV = instr_desc(kFmt, 1, kHeads, kHalfV);
    bool ok = true;

    if (warp == 4) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            // Q blocks for shared memory: slot 0 meets the last streamed block, slots 1-4 the V blocks.
            // (the map's box holds head_q <= 128 rows; rows past them keep whatever shared memory held and only
            // feed tile rows that are never read back)
            mbar_arrive_expect_tx(q_full, kQSmemBlocks * p.head_q * 128);
            tma_load_tile_3d(q_s, &tm_q, a_block(half, kABlocks - 1) * 64, 0, b, q_full);
            for (int j = 0; j < kVBlocks; ++j) {
                tma_load_tile_3d(q_s + (1 + j) * kQBlockBytes, &tm_q, v_block(half, j) * 64, 0, b, q_full);
            }
        }
        const T *k_g = reinterpret_cast<const T *>(p.k);
        const int run = kShortPages ? kv_run_keys(p, kTile) : kTile;
        int a_slot = 0;
        uint32_t a_round = 0;  // how many times the streamed ring has wrapped
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int key0 = k_begin + t * kTile;
            const int rows = min(kTile, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            // rows of the tile are consecutive in the cache, except across the pages of a short-page cache
            auto row_of = [&](int r) { return kShortPages ? kv_tile_row(p, b, seq_begin, key0 + r) : tok0 + r; };
            const bool whole = rows == kTile;
            // the five streamed blocks, each into the next slot of the ring (the V blocks come from the loader warps)
            for (int j = 0; j < kABlocks && ok; ++j) {
                if (a_round > 0) ok = mbar_wait(&a_empty[a_slot], (a_round & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                if (whole && lane == 0) mbar_arrive_expect_tx(&a_full[a_slot], kKBlockBytes);
                load_block<T>(a_s + a_slot * kKBlockBytes, &tm_k, k_g, p.k_row_stride, a_block(half, j), row_of, run, rows,
                              &a_full[a_slot], lane);
                if (!whole) {
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[a_slot]);
                }
                if (++a_slot == kASlots) {
                    a_slot = 0;
                    ++a_round;
                }
            }
            __syncwarp();
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        {
            const uint32_t leader = elect_one();
            // Descriptors differ from slot to slot only in their start-address field (low 14 bits, in
            // 16-byte units): build them once and add offsets, so that the unrolled issue sequence is
            // one add per operand and the MMA itself.  (A single thread issues these; every extra
            // dependent instruction here is tensor-pipe idle time.)
            const uint64_t q_desc0 = smem_desc(smem_u32(q_s), 16, 1024, 2);
            const uint64_t a_desc0 = smem_desc(smem_u32(a_s), 16, 1024, 2);
            const uint64_t vk_desc0 = smem_desc(smem_u32(v_s), 16, 1024, 2);            // V slot as K-major rows (for S)
            const uint64_t vn_desc0 = smem_desc(smem_u32(v_s), kKBlockBytes, 1024, 2);  // V slot MN-major (for P.V)
            const uint32_t q_tmem_addr = tmem_base + kColQ;
            int a_slot = 0;
            uint32_t a_round = 0;
            auto issue_qk = [&](int t) -> bool {
                const uint32_t d = tmem_base + kColS + (t & 1) * kTile;
#pragma unroll
                for (int j = 0; j < kABlocks; ++j) {
                    if (!mbar_wait(&a_full[a_slot], a_round & 1u, abort_flag)) return false;
                    tc_fence_after();
                    const uint64_t bd = a_desc0 + (uint64_t)((a_slot * kKBlockBytes) >> 4);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        if (j < kQTmemBlocks) {
                            umma_ts(d, q_tmem_addr + j * 32 + ks * 8, bd + (uint64_t)(ks * 2), kIdescQK, (j | ks) ? 1u : 0u, leader);
                        } else {
                            umma_ss(d, q_desc0 + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), kIdescQK, 1u, leader);
                        }
                    }
                    umma_commit(&a_empty[a_slot], leader);
                    if (++a_slot == kASlots) {
                        a_slot = 0;
                        ++a_round;
                    }
                }
                if (!mbar_wait(&v_full[t % kVSlots], (uint32_t)(t / kVSlots) & 1u, abort_flag)) return false;
                tc_fence_after();
                const uint64_t vd = vk_desc0 + (uint64_t)(((t % kVSlots) * kVSlotBytes) >> 4);
#pragma unroll
                for (int j = 0; j < kVBlocks; ++j) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        umma_ss(d, q_desc0 + (uint64_t)(((1 + j) * kQBlockBytes + ks * 32) >> 4),
                                vd + (uint64_t)((j * kKBlockBytes + ks * 32) >> 4), kIdescQK, 1u, leader);
                    }
                }
                umma_commit(&s_full[t & 1], leader);
                return true;
            };
            ok = mbar_wait(q_full, 0, abort_flag);
            if (ok) ok = mbar_wait(q_tmem, 0, abort_flag);
            if (ok) {
                tc_fence_after();
                ok = issue_qk(0);
            }
            for (int t = 0; t < n_tiles && ok; ++t) {
                if (t + 1 < n_tiles) {
                    ok = issue_qk(t + 1);
                    if (!ok) break;
                }
                ok = mbar_wait(&p_full[t & 1], (uint32_t)(t / 2) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const int vs = t % kVSlots;
                const uint32_t d = tmem_base + kColO;
                // A = P from TMEM: 16 keys = 8 columns of 16-bit pairs per step.
                // B = V, MN-major: 64-column blocks kKBlockBytes apart (LBO), 8-key groups 1 KB apart (SBO).
                const uint32_t pa = tmem_base + kColS + (t & 1) * kTile;
                const uint64_t vd = vn_desc0 + (uint64_t)((vs * kVSlotBytes) >> 4);
#pragma unroll
                for (int ks = 0; ks < kTile / 16; ++ks) {
                    umma_ts(d, pa + ks * 8, vd + (uint64_t)((ks * 16 * 128) >> 4), kIdescPV, (t | ks) ? 1u : 0u, leader);
                }
                umma_commit(&v_empty[vs], leader);
                umma_commit(&pv_done[t & 1], leader);
            }
        }
        __syncwarp();
    } else if (warp >= 6) {
        // ---------------- V loaders: 16-byte cp.async through the load/store unit ----------------
        // The TMA engine of an SM moves about 21 B/clk (measured with bulk copies, L2-resident source, any
        // depth); 16-byte loads from many threads reach 85-97 B/clk on the same data.  The four V blocks of
        // a tile (32 KB of its 72 KB) therefore bypass the TMA engine: 128 threads x 16 cp.async, written
        // straight into the 128-byte-swizzled layout; a tile is published (wait_group, proxy fence, arrive)
        // once the next one has been issued, so two are in flight.
        const int lt = tid - 6 * 32;  // 0..127
        const T *k_g = reinterpret_cast<const T *>(p.k);
        const int run = kShortPages ? kv_run_keys(p, kTile) : kTile;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int key0 = k_begin + t * kTile;
            const int rows = min(kTile, k_end - key0);
            const size_t tok0 = kv_tile_row(p, b, seq_begin, key0);
            const int vs = t % kVSlots;
            if (t >= kVSlots) ok = mbar_wait(&v_empty[vs], ((uint32_t)(t / kVSlots) & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            uint8_t *slot = v_s + vs * kVSlotBytes;
            if (!kShortPages) {  // the tile's rows are consecutive in the cache
#pragma unroll
                for (int n = 0; n < kVBlocks * kTile * 8 / kLoaderThreads; ++n) {
                    const int i = lt + n * kLoaderThreads;
                    const int j = i >> 9, r = (i >> 3) & 63, cc = i & 7;
                    const T *src = k_g + (tok0 + min(r, rows - 1)) * p.k_row_stride + v_block(half, j) * 64 + cc * 8;
                    cp_async16(slot + j * kKBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4), src, r < rows ? 16u : 0u);  // 0: zero fill
                }
            } else {  // pages shorter than the tile: at most four of them, looked up once per tile
                size_t page_row[4];
#pragma unroll
                for (int g = 0; g < 4; ++g) page_row[g] = g * run < rows ? kv_tile_row(p, b, seq_begin, key0 + g * run) : 0;
#pragma unroll
                for (int n = 0; n < kVBlocks * kTile * 8 / kLoaderThreads; ++n) {
                    const int i = lt + n * kLoaderThreads;
                    const int j = i >> 9, r = (i >> 3) & 63, cc = i & 7;
                    const int rr = min(r, rows - 1);
                    const int g = rr / run;  // run is 16 or 32
                    const size_t base = g == 0 ? page_row[0] : (g == 1 ? page_row[1] : (g == 2 ? page_row[2] : page_row[3]));
                    const T *src = k_g + (base + (rr - g * run)) * p.k_row_stride + v_block(half, j) * 64 + cc * 8;
                    cp_async16(slot + j * kKBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4), src, r < rows ? 16u : 0u);
                }
            }
            cp_async_commit();
            if (t >= 1) {  // the tile issued one iteration ago has landed: publish it to the tensor pipe
                cp_async_wait<1>();
                fence_proxy_async();
                mbar_arrive(&v_full[(t - 1) % kVSlots]);
            }
        }
        cp_async_wait<0>();
        fence_proxy_async();
        if (ok) mbar_arrive(&v_full[(n_tiles - 1) % kVSlots]);
    } else {
        // ---------------- softmax / epilogue: thread r <-> TMEM lane r <-> head r ----------------
        const int r = tid;
        const bool valid = r < p.head_q;  // with fewer than 128 heads the remaining rows are padding
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        const float slope2 = p.is_alibi ? exp2f(-8.0f * (float)(r + 1) / (float)p.head_q) * kLog2e : 0.0f;
        const int pos_shift = (p.kv_pos_offset ? p.kv_pos_offset[b] : 0) - ((p.kv_total_len ? p.kv_total_len[b] : len) - 1);
        float m_ref = -INFINITY, l = 0.0f;
        uint32_t buf[32];
        {
            // The Q columns that meet the first four streamed blocks go to TMEM as packed 16-bit pairs.
            const T *q_row = reinterpret_cast<const T *>(p.q) + (size_t)b * p.q_row_stride + (size_t)r * kDim;
#pragma unroll 1
            for (int j = 0; j < kQTmemBlocks; ++j) {
                const T *src = q_row + a_block(half, j) * 64;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 v = valid ? *reinterpret_cast<const uint4 *>(src + i * 8) : make_uint4(0, 0, 0, 0);
                    buf[4 * i] = v.x, buf[4 * i + 1] = v.y, buf[4 * i + 2] = v.z, buf[4 * i + 3] = v.w;
                }
                tmem_st32(lane_base + kColQ + j * 32, buf);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(q_tmem);
        }
        for (int t = 0; t < n_tiles; ++t) {
            const int key0 = k_begin + t * kTile;
            const int rows = min(kTile, k_end - key0);
            const uint32_t s_addr = lane_base + kColS + (t & 1) * kTile;
            ok = mbar_wait(&s_full[t & 1], (uint32_t)(t / 2) & 1u, abort_flag);
            if (!ok) break;
            tc_fence_after();
            float s[kTile];
            float mx = -INFINITY;
#pragma unroll
            for (int c0 = 0; c0 < kTile; c0 += 32) {
                tmem_ld32(s_addr + c0, buf);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float x = __uint_as_float(buf[j]) * p.scale_log2 + slope2 * (float)(key0 + c0 + j + pos_shift);
                    s[c0 + j] = (c0 + j < rows) ? (valid ? x : 0.0f) : -INFINITY;
                    mx = fmaxf(mx, s[c0 + j]);
                }
            }
            const bool raise = mx > m_ref + kRescaleThreshold;
            float alpha = 1.0f;
            if (raise) {
                alpha = exp2f(m_ref - mx);  // 0 on the first tile
                m_ref = mx;
                l *= alpha;
            }
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
            // P = exp2(S - m_ref), rounded to the input type, packed in pairs over the first half of S(t).
            // (The tile that used these columns before, t-2, is past its P.V: S(t) was issued after it.)
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < kTile / 2; ++j) {
                const float p0 = exp2f(s[2 * j] - m_ref), p1 = exp2f(s[2 * j + 1] - m_ref);
                sum += p0 + p1;
                if (std::is_same<T, __nv_bfloat16>::value) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    buf[j] = *reinterpret_cast<uint32_t *>(&h);
                } else {
                    __half2 h = __floats2half2_rn(p0, p1);
                    buf[j] = *reinterpret_cast<uint32_t *>(&h);
                }
            }
            tmem_st32(s_addr, buf);
            l += sum;
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&p_full[t & 1]);
        }
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
                const int d0 = half * kHalfV + c * 32;
                if (!valid) continue;  // padding row: nothing to write (the loads above are warp-wide)
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
            if (half == 0 && valid) {
                if (p.num_splits > 1) {
                    p.part_lse[row] = lse;
                } else if (p.lse) {
                    p.lse[(size_t)b * p.head_q + r] = lse;
                }
            }
            tc_fence_before();
        }
    }

    if (!ok && lane == 0) report_timeout(p);
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace


SplitVariantInfo split_info_mla_tc() { return {kTile, kHeads, 1}; }

// tm_q: rank-3 map over q [batch][128][576], box {64, 128, 1}, 128-byte swizzle;
// tm_k: rank-2 map over the latent cache [rows][576], box {64, kTile}, 128-byte swizzle.
cudaError_t launch_mla_tc(bool bf16, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                          cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !attr_set[dev]) {
        const void *kernels[4] = {(const void *)da_mla_tc_kernel<__half, false>, (const void *)da_mla_tc_kernel<__half, true>,
                                  (const void *)da_mla_tc_kernel<__nv_bfloat16, false>,
                                  (const void *)da_mla_tc_kernel<__nv_bfloat16, true>};
        for (const void *k : kernels) {
            err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (err != cudaSuccess) return err;
        }
        attr_set[dev] = true;
    }
    dim3 grid(p.num_splits, 2, p.batch);
    const bool overlap = p.batch_order != nullptr;
    const bool short_pages = p.block_table && (1 << p.page_shift) < kTile;
    if (bf16) {
        return short_pages ? launch_kernel(da_mla_tc_kernel<__nv_bfloat16, true>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k)
                           : launch_kernel(da_mla_tc_kernel<__nv_bfloat16, false>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k);
    }
    return short_pages ? launch_kernel(da_mla_tc_kernel<__half, true>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k)
                       : launch_kernel(da_mla_tc_kernel<__half, false>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k);
}

}  // namespace da
