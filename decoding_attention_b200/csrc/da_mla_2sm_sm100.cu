// Latent-KV (MLA) decode attention on the sm_100a tensor cores, two SMs per key range:
// tcgen05.mma.cta_group::2 with accumulators in tensor memory (TMEM), operands staged by TMA and
// cp.async.
//
// Shape: up to 128 query heads share one KV head whose rows hold 576 values, V being the first 512
// of them (the reference runs this shape through its generic kernel, one CTA per query head:
// csrc/kernel/decoding_attn/decoding_fwd_hd576_hdv512.cu:9-17, so every K row is fetched once per
// head).  A cluster of two CTAs owns one (sequence, key range) and walks it in tiles of 128 keys:
//     S[128 heads x 128 keys]  = Q[128 x 576] . K_tile[128 x 576]^T     36 MMAs  M128 N128 K16
//     O[128 heads x 512]      += P[128 x 128] . V_tile[128 x 512]       16 MMAs  M128 N256 K16
// Both are pair MMAs: CTA c holds heads 64c..64c+63 (its rows of Q, S, P and O) and supplies one half
// of every B operand from its own shared memory -- keys 64c..64c+63 of the tile for S, 256 of the 512
// V columns (dims 256c..256c+255) of all 128 keys for P.V.  Nothing is computed twice, every K row is
// read by one CTA for S, and the 128 x 512 fp32 output fits because a CTA's 64 x 512 share is 128
// TMEM lanes x 256 columns.  What a CTA reads per tile: its 64 keys x 576 dims for S (nine 8 KB
// blocks streamed by TMA through a ring of nine slots, released three at a time by a tcgen05.commit right after
// their twelve MMAs) and 128 keys x 256 dims for P.V (two 32 KB half-tile slots, cp.async), 136 KB against
// 2 x 72 KB for a kernel whose two CTAs work apart; the second reader of a row hits L2.
// What bounds it (measured with per-tile cycle stamps, batch 128 x 4096 keys, 150 us): the K ring never made
// the issuing warp wait; the issue loops and the softmax chain did.  A barrier wait costs the issuing warp 100-200
// cycles even when the phase is complete, a commit 60-90, so S and P.V have an issuing warp each, the ring's
// barriers cover three blocks, and P / P.V are tracked per 64-key half of a tile so that the next tile's P block 0
// is written while P.V still reads block 1.  A tile takes about 2 950 cycles against 2 176 cycles of MMAs.
//
// TMEM columns per CTA: S0 | S1 (64 each: lanes 0-63 keys 0-63 of the tile, lanes 64-127 keys 64-127,
// rows = this CTA's heads) | O (256: lanes 0-63 dims 0-255, lanes 64-127 dims 256-511) | Q (4 x 32:
// the first four 64-dim blocks of Q as 16-bit pairs, head r in lanes r and r + 64, read as the A operand).
// Warp roles (480 threads): warps 0-7 softmax/epilogue, two per TMEM lane quadrant -- thread (ch, l) works on
// lane l, i.e. head (l & 63) and key half (l >> 6), and on 32 of the lane's 64 score columns; the four threads
// of a head swap their tile maxima through shared memory, keep one reference max, and write P (16-bit,
// 128-byte-swizzled K-major) to shared memory; warp 8 TMA producer (Q blocks, streamed K blocks); warp 9 TMEM
// allocation and, in the rank-0 CTA, issue of S for the pair; warps 10-13 V loaders (16-byte cp.async straight
// into the swizzled layout, because one SM's TMA engine alone moves only about 21 B/clk); warp 14, in the
// rank-0 CTA, issue of P.V.
// Barriers the issuing warps wait on live in the rank-0 CTA and count arrivals / bytes from both CTAs;
// barriers that release buffers or publish S are signalled in both CTAs by one multicast commit.
// Online softmax with a lazy reference max (raised only when exceeded by 2^8), so O is rescaled a
// handful of times.  Every wait is bounded; on expiry the CTA records the timeout and still frees
// its TMEM.
#include <type_traits>

#include "da_internal.h"
#include "da_tcgen05.cuh"

namespace da {
namespace {

constexpr int kHeads = 128;        // M of both contractions (pair)
constexpr int kRows = 64;          // heads per CTA
constexpr int kDim = 576;
constexpr int kDimV = 512;
// Keys per pair tile.  (64-key tiles were measured at 307 us against 187 us: a tile's cost is mostly fixed, so
// halving the tile doubles the number of softmax hand-overs.)
constexpr int kTile = 128;
constexpr int kHalf = kTile / 2;   // keys per CTA in S / per V half-tile slot
constexpr int kBlocks = kDim / 64; // 64-element (128-byte) column blocks of a row
constexpr int kVBlocks = 4;        // V blocks per CTA (256 of the 512 output dims)
constexpr int kQTmemBlocks = 4;                 // Q blocks 0 .. kQTmemBlocks-1 live in TMEM
constexpr int kQSmemBlocks = kBlocks - kQTmemBlocks;
constexpr int kQBlockBytes = 64 * 128;     // [64 heads x 64 dims], 128-byte swizzle: a Q block (and a 64-key block of P)
constexpr int kKBlockBytes = kHalf * 128;  // [kHalf keys x 64 dims]: a K block of one CTA
constexpr int kASlots = 9;                      // ring of TMA-streamed K blocks: one tile
constexpr int kGroup = 3;                       // K blocks per ring barrier: the issue loop pays per barrier wait and commit
constexpr int kAGroups = kASlots / kGroup;
static_assert(kASlots % kGroup == 0 && (kDim / 64) % kGroup == 0, "blocks travel in groups");
constexpr int kTileGroups = (kDim / 64) / kGroup;   // groups per tile
constexpr int kRingTiles = kAGroups / kTileGroups;  // the ring holds a whole number of tiles: a group's slot is static
static_assert(kAGroups % kTileGroups == 0, "the K ring holds whole tiles");
constexpr int kVSlots = 3;                      // ring of V half-tiles
constexpr int kVSlotBytes = kVBlocks * kKBlockBytes;
constexpr int kPBufs = 1;                       // P tiles in shared memory
constexpr int kPBytes = (kTile / 64) * kQBlockBytes;  // [64 heads x kTile keys]
constexpr int kQStageSlots = (kQTmemBlocks * kQBlockBytes + kVSlotBytes - 1) / kVSlotBytes;  // V slots that stage Q at first
constexpr int kOffQ = 0;
constexpr int kOffA = kOffQ + kQSmemBlocks * kQBlockBytes;
constexpr int kOffV = kOffA + kASlots * kKBlockBytes;
constexpr int kOffP = kOffV + kVSlots * kVSlotBytes;
constexpr int kOffBar = kOffP + kPBufs * kPBytes;
// q_full, q_tmem, q_stage_full, q_copied, a_full/a_empty[kASlots], v_full/v_empty[kVSlots], s_full[2], p_full[2][2], pv_done[2][2], s_empty[2], o_stable[2]
constexpr int kNumBars = 4 + 2 * kAGroups + 2 * kVSlots + 14;
constexpr int kOffMisc = kOffBar + kNumBars * 8;          // tmem slot, abort flag
constexpr int kOffXch = kOffMisc + 16;                    // bf16 [2][256] tile maxima, later float [256] row sums
constexpr int kSmemBytes = kOffXch + 256 * 4 + 1024;      // + alignment slack
constexpr int kLoaderWarps = 4;
constexpr int kLoaderThreads = kLoaderWarps * 32;
constexpr int kSoftmaxWarps = 8;                   // two per TMEM lane quadrant
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr int kProducerWarp = kSoftmaxWarps, kSWarp = kSoftmaxWarps + 1, kLoaderWarp0 = kSoftmaxWarps + 2;
constexpr int kPvWarp = kLoaderWarp0 + kLoaderWarps;
constexpr int kThreads = (kPvWarp + 1) * 32;
constexpr int kTmemCols = 512;
constexpr int kColS = 0;              // two S buffers of kHalf columns
constexpr int kColO = 2 * kHalf;      // 256 output columns
constexpr int kColQ = kColO + 256;    // kQTmemBlocks * 32 columns
static_assert(kColQ + kQTmemBlocks * 32 <= kTmemCols, "TMEM budget");
static_assert(kQStageSlots < kVSlots, "the Q blocks bound for TMEM are staged in the last V slots");
static_assert(kTile == 128 && kQTmemBlocks % 2 == 0, "tile");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert(kSoftmaxThreads * (128 * 4 + 16) <= kOffP - kOffA, "the epilogue stages its output in the idle rings");
constexpr float kRescaleThreshold = 8.0f;

// kShortPages: the cache is paged in pages shorter than the kHalf keys one CTA stages at a time; a block is then
// fetched page by page (one TMA box per page) and the V loaders look every row's page up.  A separate
// instantiation, so that the common case keeps its straight-line address arithmetic.
template <typename T, bool kShortPages>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
da_mla_2sm_kernel(const SplitParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    pdl_launch_dependents();  // the merge kernel may be scheduled behind this grid's last CTAs
    const uint32_t rank = cluster_ctarank();
    const int split = blockIdx.y;
    if (p.batch_order) pdl_wait();  // written by the order kernel launched just before this one
    const int b = p.batch_order ? p.batch_order[blockIdx.z] : (int)blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq_begin = p.cu_seq_k[b];
    const int len = p.cu_seq_k[b + 1] - seq_begin;
    const int k_begin = split * p.chunk_keys;
    const int k_end = split_key_end(p, split, len);
    T *o_out = reinterpret_cast<T *>(p.o);
    const int head0 = (int)rank * kRows;  // first head of this CTA
    // (both CTAs of a pair take the same branch here: the conditions do not depend on the rank)
    if (launch_aborted(p)) return;  // an earlier CTA of this launch timed out: do not pile up

    if (k_begin >= k_end) {
        if (p.num_splits == 1) {  // empty sequence: zero rows, LSE = -inf
            const int nh = min(kRows, p.head_q - head0);
            for (int idx = tid; idx < nh * kDimV; idx += kThreads) {
                const int h = head0 + idx / kDimV, d = idx % kDimV;
                if (o_out) o_out[(size_t)b * p.o_row_stride + (size_t)h * kDimV + d] = from_float<T>(0.0f);
                if (p.o_f32) p.o_f32[((size_t)b * p.head_q + h) * kDimV + d] = 0.0f;
            }
            if (p.lse && tid < nh) p.lse[(size_t)b * p.head_q + head0 + tid] = -INFINITY;
        }
        return;
    }
    const int n_tiles = (k_end - k_begin + kTile - 1) / kTile;
    // With ALiBi the bias, and with it every head's row maximum, grows towards the end of the sequence: walked
    // front to back, every tile would raise the reference maximum of the steep heads and take the rescale path.
    // Walked back to front the first tiles set the maximum.  `tile_of(t)` is the tile the t-th step works on.
    const bool backwards = p.is_alibi != 0;
    auto tile_of = [&](int t) { return backwards ? n_tiles - 1 - t : t; };

    uint8_t *q_s = smem + kOffQ;
    uint8_t *a_s = smem + kOffA;
    uint8_t *v_s = smem + kOffV;
    uint8_t *p_s = smem + kOffP;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBar);
    uint64_t *q_full = bars;       // rank 0: Q blocks of both CTAs are in shared memory
    uint64_t *q_tmem = bars + 1;   // rank 0: Q blocks of both CTAs are in TMEM
    uint64_t *q_stage_full = bars + 2;  // this CTA: Q blocks 0..3 landed in the staging slot
    uint64_t *q_copied = bars + 3;      // this CTA: the softmax warps have moved them to TMEM
    uint64_t *a_full = bars + 4;   // rank 0: streamed K block landed in both CTAs
    uint64_t *a_empty = a_full + kAGroups;
    uint64_t *v_full = a_empty + kAGroups;  // rank 0: V half-tile landed in both CTAs
    uint64_t *v_empty = v_full + kVSlots;
    uint64_t *s_full = v_empty + kVSlots;
    // P and P.V are tracked per 64-key half of a tile, [tile parity][half]: the threads of key half h write P
    // block h as soon as the first / second half of the previous tile's P.V has read it, and the P.V issuer
    // starts on block 0 while block 1 is still being written.
    uint64_t *p_full = s_full + 2;         // rank 0: P block written by both CTAs
    uint64_t *pv_done = p_full + 4;
    uint64_t *s_empty = pv_done + 4;       // rank 0: every softmax warp of the pair has read its S columns
    uint64_t *o_stable = s_empty + 2;      // rank 0: no softmax warp of the pair is rescaling its accumulator rows for this tile
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    __nv_bfloat16 *x_max = reinterpret_cast<__nv_bfloat16 *>(smem + kOffXch);  // [2][256] tile maxima, rounded up
    float *x_sum = reinterpret_cast<float *>(smem + kOffXch);                   // [256] row sums, after the last tile

    if (tid == 0) {
        mbar_init(q_full, 2);
        mbar_init(q_tmem, 2 * kSoftmaxWarps);
        mbar_init(q_stage_full, 1);
        mbar_init(q_copied, kSoftmaxWarps);
        for (int s = 0; s < kAGroups; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < kVSlots; ++s) {
            mbar_init(&v_full[s], 2 * kLoaderWarps);
            mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&s_full[s], 1);
            mbar_init(&s_empty[s], 2 * kSoftmaxWarps);
            mbar_init(&o_stable[s], 2 * kSoftmaxWarps);
            for (int h = 0; h < 2; ++h) {
                mbar_init(&p_full[2 * s + h], kSoftmaxWarps);  // the four warps of key half h, in both CTAs
                mbar_init(&pv_done[2 * s + h], 1);
            }
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kSWarp) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    cluster_sync_all();  // both CTAs' barriers exist before anybody arrives on them remotely
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // shared::cluster addresses of the rank-0 CTA's barriers (what the peer arrives on)
    auto lead = [&](uint64_t *bar) { return map_to_cta(smem_u32(bar), 0); };

    constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
    constexpr uint32_t kIdescQK = instr_desc(kFmt, 0, kHeads, kTile);
    constexpr uint32_t kIdescPV = instr_desc(kFmt, 1, kHeads, 256);
    bool ok = true;
    const T *k_g = reinterpret_cast<const T *>(p.k);

    if (warp == kProducerWarp) {
        // ---------------- TMA producer: Q blocks 4..8, then this CTA's 64 keys of every tile ----------------
        const int q_rows = min(kRows, p.head_q - head0);  // rows the Q box holds (<= 0: this CTA is all padding)
        if (lane == 0) {
            tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(&tm_k);
            if (q_rows > 0) {
                // a box always delivers its full size: rows past head_q arrive as zeros
                mbar_arrive_expect_tx_remote(lead(q_full), (uint32_t)(kQSmemBlocks * min(p.head_q, kRows) * 128));
                for (int j = 0; j < kQSmemBlocks; ++j)
                    tma2_load_3d(q_s + j * kQBlockBytes, &tm_q, (kQTmemBlocks + j) * 64, head0, b, lead(q_full));
                // blocks 0..3 pass through the last V slot on their way to TMEM
                mbar_arrive_expect_tx(q_stage_full, (uint32_t)(kQTmemBlocks * min(p.head_q, kRows) * 128));
                for (int j = 0; j < kQTmemBlocks; ++j)
                    tma_load_tile_3d(v_s + (kVSlots - kQStageSlots) * kVSlotBytes + j * kQBlockBytes, &tm_q, j * 64, head0, b, q_stage_full);
            } else {
                mbar_arrive_remote(lead(q_full));
            }
        }
        int gs = 0;
        uint32_t round = 0;
        for (int t = 0; t < n_tiles && ok; ++t) {
            const int key0 = k_begin + tile_of(t) * kTile + (int)rank * kHalf;  // this CTA's first key of the tile
            const int rows = max(0, min(kHalf, k_end - key0));
            const size_t tok0 = rows > 0 ? kv_tile_row(p, b, seq_begin, key0) : 0;
            // rows of the tile are consecutive in the cache, except across the pages of a short-page cache
            auto row_of = [&](int r) { return kShortPages ? kv_tile_row(p, b, seq_begin, key0 + r) : tok0 + r; };
            const int run = kShortPages ? (1 << p.page_shift) : kHalf;  // consecutive rows: a page, or the whole half tile
            // Short pages: lane i reads the i-th page of this CTA's half tile from the block table once per tile, all
            // lanes with one load (a look-up per page and group by the issuing lane alone took twelve dependent loads
            // per tile, longer than the tile itself).
            int my_page = 0;
            if (kShortPages && rows == kHalf && lane < (kHalf >> p.page_shift)) {
                my_page = p.block_table[(size_t)b * p.block_table_stride + (key0 >> p.page_shift) + lane];
            }
            for (int g = 0; g < kBlocks / kGroup && ok; ++g) {
                if (round > 0) ok = mbar_wait(&a_empty[gs], (round & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                uint8_t *dst = a_s + gs * kGroup * kKBlockBytes;
                // a_full[gs] of the rank-0 CTA takes ONE arrival per use, rank 0's, which also announces the
                // bytes: its own blocks when they come by TMA, and always the peer's -- delivered by the
                // peer's TMA copies, or counted by hand when the peer had to write ragged blocks with stores.
                // (No remote arrival per group: a cluster-scope release costs about a thousand cycles.)
                if (rows == kHalf) {
                    if (lane == 0 && rank == 0) mbar_arrive_expect_tx(&a_full[gs], 2 * kGroup * kKBlockBytes);
                    for (int k0 = 0; k0 < kHalf; k0 += run) {
                        // (half tiles start on a page boundary: a page's first row is page << page_shift)
                        const int row = kShortPages ? (__shfl_sync(0xffffffffu, my_page, k0 >> p.page_shift) << p.page_shift) : (int)tok0;
                        if (lane == 0) {
#pragma unroll
                            for (int jj = 0; jj < kGroup; ++jj)
                                tma2_load_2d(dst + jj * kKBlockBytes + k0 * 128, &tm_k, (g * kGroup + jj) * 64, row, lead(&a_full[gs]));
                        }
                    }
                } else {
                    // ragged end of the key range (the tensor map must not be asked for rows beyond the sequence)
                    // (16-byte cp.async, all of the warp's copies in flight at once; rows past the end zero-filled)
                    for (int i = lane; i < kGroup * kHalf * 8; i += 32) {
                        const int jj = i / (kHalf * 8), r = (i >> 3) % kHalf, cc = i & 7;
                        const bool real = r < rows;
                        const T *src = k_g + (real ? row_of(r) * p.k_row_stride + (g * kGroup + jj) * 64 + cc * 8 : 0);
                        cp_async16(dst + jj * kKBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4), src, real ? 16u : 0u);
                    }
                    cp_async_commit();
                    cp_async_wait<0>();
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (rank == 0) {
                            mbar_arrive_expect_tx(&a_full[gs], kGroup * kKBlockBytes);
                        } else {
                            fence_acq_rel_cluster();
                            mbar_complete_tx_remote(lead(&a_full[gs]), kGroup * kKBlockBytes);
                        }
                    }
                }
                if (++gs == kAGroups) {
                    gs = 0;
                    ++round;
                }
            }
            __syncwarp();
        }
    } else if (warp == kSWarp) {
        // ---------------- issuer of S = Q.K^T (the rank-0 CTA issues for the pair) ----------------
        // The two contractions have an issuing warp each (this one and warp kPvWarp): per K block the issue loop
        // costs a barrier wait, four MMAs and a commit, about as long as those MMAs run, so one warp issuing S
        // and P.V in turn keeps the tensor pipe waiting for its next instruction.  The whole warp walks the loop
        // and one elected lane issues: the same loop run by lane 0 alone was measured 55 % slower.
        if (rank == 0) {
            const uint32_t leader = elect_one();
            const uint64_t q_desc0 = smem_desc(smem_u32(q_s), 16, 1024, 2);
            const uint64_t a_desc0 = smem_desc(smem_u32(a_s), 16, 1024, 2);
            const uint32_t q_tmem_addr = tmem_base + kColQ;
            ok = mbar_wait(q_full, 0, abort_flag);
            if (ok) ok = mbar_wait(q_tmem, 0, abort_flag);
            if (ok) tc_fence_after();
            for (int t = 0; t < n_tiles && ok; ++t) {
                // S(t) goes where S(t-2) was, once the softmax threads have loaded that.
                if (t >= 2) ok = mbar_wait(&s_empty[t & 1], (uint32_t)((t - 2) / 2) & 1u, abort_flag);
                if (!ok) break;
                const uint32_t d = tmem_base + kColS + (t & 1) * kHalf;
                const int gs0 = (t % kRingTiles) * kTileGroups;       // first ring slot of this tile's groups
                const uint32_t a_par = (uint32_t)(t / kRingTiles) & 1u;
                // (unrolled over the tile's groups: slots, barriers and descriptors are compile-time offsets, which
                // keeps the issue loop -- the pace-setter of the kernel -- short; one barrier wait and one commit per group)
#pragma unroll
                for (int g = 0; g < kTileGroups; ++g) {
                    ok = mbar_wait(&a_full[gs0 + g], a_par, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int jj = 0; jj < kGroup; ++jj) {
                        const int j = g * kGroup + jj;
                        const uint64_t bd = a_desc0 + (uint64_t)(((gs0 + g) * kGroup + jj) * (kKBlockBytes >> 4));
                        if (j < kQTmemBlocks) {
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                umma2_ts(d, q_tmem_addr + j * 32 + ks * 8, bd + (uint64_t)(ks * 2), kIdescQK, (j | ks) ? 1u : 0u, leader);
                        } else {
                            const uint64_t qd = q_desc0 + (uint64_t)(((j - kQTmemBlocks) * kQBlockBytes) >> 4);
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                umma2_ss(d, qd + (uint64_t)(ks * 2), bd + (uint64_t)(ks * 2), kIdescQK, (j | ks) ? 1u : 0u, leader);
                        }
                    }
                    umma2_commit_both(&a_empty[gs0 + g], leader);
                }
                if (!ok) break;
                umma2_commit_both(&s_full[t & 1], leader);
            }
        }
        __syncwarp();
    } else if (warp == kPvWarp) {
        // ---------------- issuer of O += P.V (rank-0 CTA), tile by tile ----------------
        if (rank == 0) {
            const uint32_t leader = elect_one();
            const uint64_t p_desc0 = smem_desc(smem_u32(p_s), 16, 1024, 2);
            const uint64_t v_desc0 = smem_desc(smem_u32(v_s), kKBlockBytes, 1024, 2);  // V slot, MN-major
            for (int t = 0; t < n_tiles && ok; ++t) {
                ok = mbar_wait(&p_full[2 * (t & 1)], (uint32_t)(t / 2) & 1u, abort_flag);
                // P block 0 is complete once the warps of key half 0 have written it; the warps of key half 1 may
                // still be rescaling their lanes' accumulator columns (the rare raised reference maximum), and
                // every P.V rewrites all of O: wait until every softmax warp of the pair is past that point.
                if (ok) ok = mbar_wait(&o_stable[t & 1], (uint32_t)(t / 2) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d = tmem_base + kColO;
                const uint64_t pd = p_desc0 + (uint64_t)((((t % kPBufs) * kPBytes)) >> 4);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int i = 2 * t + h;
                    const int vs = i % kVSlots;
                    if (h == 1) ok = mbar_wait(&p_full[2 * (t & 1) + 1], (uint32_t)(t / 2) & 1u, abort_flag);
                    if (ok) ok = mbar_wait(&v_full[vs], (uint32_t)(i / kVSlots) & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t vd = v_desc0 + (uint64_t)((vs * kVSlotBytes) >> 4);
#pragma unroll
                    for (int ks = 0; ks < kHalf / 16; ++ks) {
                        // A = P[64 heads x 16 keys]: keys h * kHalf + ks * 16 .. of the tile, in 64-key swizzled blocks;
                        // B = V[16 keys x 128 dims] per CTA, blocks {0,1} then {2,3}
                        const int key = h * kHalf + ks * 16;
                        const uint64_t ad = pd + (uint64_t)(((key / 64) * kQBlockBytes + (key % 64) * 2) >> 4);
                        const uint64_t bd = vd + (uint64_t)((ks * 16 * 128) >> 4);
                        umma2_ss(d, ad, bd, kIdescPV, (t | h | ks) ? 1u : 0u, leader);
                        umma2_ss(d + 128, ad, bd + (uint64_t)((2 * kKBlockBytes) >> 4), kIdescPV, (t | h | ks) ? 1u : 0u, leader);
                    }
                    umma2_commit_both(&v_empty[vs], leader);
                    umma2_commit_both(&pv_done[2 * (t & 1) + h], leader);
                }
                if (!ok) break;
            }
        }
        __syncwarp();
    } else if (warp >= kLoaderWarp0 && warp < kLoaderWarp0 + kLoaderWarps) {
        // ---------------- V loaders: this CTA's 256 dims of all 128 keys of a tile, half-tile by half-tile ----------------
        // Jobs of 32 KB each, in the order the tensor pipe needs them: K blocks 5..8 of tile 0, then per tile t
        // the same blocks of tile t+1 and the two V half-tiles of tile t.  A job is published (its barrier in the
        // rank-0 CTA gets this warp's arrival) once the next one has been issued and its own bytes have landed,
        // so two jobs are in flight.
        // One copy of the copy code for every half-tile (the kernel's unrolled loops share the instruction cache: a
        // version of this loop that was inlined four times made the whole kernel 30 % slower).  A half-tile's
        // barrier gets this warp's arrival once the next one has been issued and its own bytes have landed: two
        // half-tiles are in flight.
        const int lt = tid - kLoaderWarp0 * 32;  // 0..127
        const int n_halves = 2 * n_tiles;
        for (int i = 0; i < n_halves && ok; ++i) {
            const int key0 = k_begin + tile_of(i >> 1) * kTile + (i & 1) * kHalf;
            const int rows = max(0, min(kHalf, k_end - key0));
            const size_t tok0 = rows > 0 ? kv_tile_row(p, b, seq_begin, key0) : 0;
            const int vs = i % kVSlots;
            if (i >= kVSlots) ok = mbar_wait(&v_empty[vs], ((uint32_t)(i / kVSlots) & 1u) ^ 1u, abort_flag);
            if (ok && i >= kVSlots - kQStageSlots && i < kVSlots) ok = mbar_wait(q_copied, 0, abort_flag);  // the slot staged Q blocks
            if (!ok) break;
            uint8_t *slot = v_s + vs * kVSlotBytes;
            // thread lt copies the 16-byte chunk (lt & 7) of rows (lt >> 3) + 16 i for each of the four blocks
#pragma unroll
            for (int ri = 0; ri < kHalf / 16; ++ri) {
                const int r = (lt >> 3) + 16 * ri, cc = lt & 7;
                const int rr = max(0, min(r, rows - 1));
                const size_t trow = kShortPages ? (rows > 0 ? kv_tile_row(p, b, seq_begin, key0 + rr) : 0) : tok0 + rr;
                const T *src = k_g + trow * p.k_row_stride + (int)rank * kVBlocks * 64 + cc * 8;
#pragma unroll
                for (int j = 0; j < kVBlocks; ++j) {
                    cp_async16(slot + j * kKBlockBytes + r * 128 + ((cc ^ (r & 7)) << 4), src + j * 64, r < rows ? 16u : 0u);  // 0: zero fill
                }
            }
            cp_async_commit();
            if (i >= 1) {  // the half-tile issued one iteration ago has landed: publish it to the tensor pipe
                cp_async_wait<1>();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote_cta(lead(&v_full[(i - 1) % kVSlots]));
            }
        }
        cp_async_wait<0>();
        fence_proxy_async();
        __syncwarp();
        if (ok && lane == 0) mbar_arrive_remote_cta(lead(&v_full[(n_halves - 1) % kVSlots]));
    } else {
        // ---------------- softmax / epilogue: two warps per TMEM lane quadrant.  Thread (ch, l) works on lane l,
        // i.e. head l & 63 and key half l >> 6, and on 32 of the lane's 64 score columns (ch = 0 / 1): the softmax
        // chain of a tile is per-thread serial work, and with one thread per lane it set the kernel's pace. ----------
        const int tl = tid & 127, ch = tid >> 7;
        const int r = tl & 63, kh = tl >> 6;
        const int head = head0 + r;
        const bool valid = head < p.head_q;  // rows past head_q are padding
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const float slope2 = p.is_alibi ? exp2f(-8.0f * (float)(head + 1) / (float)p.head_q) * kLog2e : 0.0f;
        const int pos_shift = (p.kv_pos_offset ? p.kv_pos_offset[b] : 0) - ((p.kv_total_len ? p.kv_total_len[b] : len) - 1);
        float m_ref = -INFINITY, l = 0.0f;
        uint32_t buf[32];
        {
            // Q blocks 0..3 go to TMEM as packed 16-bit pairs, head r in lane r AND lane r + 64: a pair MMA reads an
            // A operand that lives in TMEM lane by lane, lanes 64-127 for the second half of the N columns.  The
            // blocks arrive by TMA in the last V slot (which the loaders leave alone until q_copied completes) and
            // each thread moves its own row: 16-byte loads of one row per lane straight from global memory would
            // cost one L1 wavefront per lane and instruction, about four thousand cycles per CTA.
            const uint8_t *q_stage = v_s + (kVSlots - kQStageSlots) * kVSlotBytes;
            const bool have_q = head0 < p.head_q;
            if (have_q) ok = __all_sync(0xffffffffu, mbar_wait(q_stage_full, 0, abort_flag)) != 0;
#pragma unroll
            for (int jj = 0; jj < kQTmemBlocks / 2; ++jj) {
                const int j = ch * (kQTmemBlocks / 2) + jj;  // this warp's half of the blocks
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 v = (valid && ok) ? *reinterpret_cast<const uint4 *>(q_stage + j * kQBlockBytes + r * 128 + ((i ^ (r & 7)) << 4))
                                                  : make_uint4(0, 0, 0, 0);
                    buf[4 * i] = v.x, buf[4 * i + 1] = v.y, buf[4 * i + 2] = v.z, buf[4 * i + 3] = v.w;
                }
                tmem_st32(lane_base + kColQ + j * 32, buf);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(q_copied);
                if (ok) mbar_arrive_remote_cta(lead(q_tmem));
            }
        }
        // `ok` is kept warp-uniform, and a warp that has given up still walks the loop so that the named
        // barriers below always see all 256 threads.
        auto wait_all = [&](uint64_t *bar, uint32_t parity) {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
        };
        for (int t = 0; t < n_tiles; ++t) {
            const int key0 = k_begin + tile_of(t) * kTile + kh * kHalf + ch * 32;  // first key of this thread's 32 columns
            const int rows = k_end - key0;                                 // columns >= rows are past the end
            const uint32_t s_addr = lane_base + kColS + (t & 1) * kHalf + ch * 32;
            if (ok) ok = wait_all(&s_full[t & 1], (uint32_t)(t / 2) & 1u);
            float s[32];
            float mx = -INFINITY;
            if (ok) {
                tc_fence_after();
                tmem_ld32(s_addr, buf);
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote_cta(lead(&s_empty[t & 1]));
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float x0 = __uint_as_float(buf[j]) * p.scale_log2 + slope2 * (float)(key0 + j + pos_shift);
                    s[j] = (j < rows) ? (valid ? x0 : 0.0f) : -INFINITY;
                    mx = fmaxf(mx, s[j]);
                }
            }
            // One reference per head: its four threads swap their maxima, rounded up to 16 bits (any common
            // reference at or above the true maximum serves; every thread uses the rounded values, its own too).
            x_max[(t & 1) * 256 + tid] = __float2bfloat16_ru(mx);
            named_bar_sync(1, kSoftmaxThreads);
            if (!ok) continue;
            {
                const __nv_bfloat16 *xm = x_max + (t & 1) * 256;
                mx = fmaxf(fmaxf(__bfloat162float(xm[tid]), __bfloat162float(xm[tid ^ 64])),
                           fmaxf(__bfloat162float(xm[tid ^ 128]), __bfloat162float(xm[tid ^ 192])));
            }
            const bool raise = mx > m_ref + kRescaleThreshold;
            float alpha = 1.0f;
            if (raise) {
                alpha = exp2f(m_ref - mx);  // 0 on the first tile
                m_ref = mx;
                l *= alpha;
            }
            const bool rescale = t >= 1 && __any_sync(0xffffffffu, raise);
            if (rescale) {
                // Rare: the reference max of some row in this warp moved.  O must be idle (P.V of tile
                // t-1 complete, P.V of this tile held back by o_stable) while its rows are rescaled in place.
                ok = wait_all(&pv_done[2 * ((t - 1) & 1) + 1], (uint32_t)((t - 1) / 2) & 1u);
                if (!ok) continue;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < 128 / 32; ++c) {  // this thread's half of the lane's 256 columns
                    tmem_ld32(lane_base + kColO + ch * 128 + c * 32, buf);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) buf[j] = __float_as_uint(__uint_as_float(buf[j]) * alpha);
                    tmem_st32(lane_base + kColO + ch * 128 + c * 32, buf);
                }
                tmem_wait_st();
                tc_fence_before();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_remote_cta(lead(&o_stable[t & 1]));  // this warp's accumulator rows are as P.V(t) may find them
            if (!rescale && kPBufs == 1 && t >= 1) {
                // this thread's block of the single P buffer is still being read by its half of P.V of tile t-1
                ok = wait_all(&pv_done[2 * ((t - 1) & 1) + kh], (uint32_t)((t - 1) / 2) & 1u);
                if (!ok) continue;
            }
            // P = exp2(S - m_ref), rounded to the input type: row r, keys kh * kHalf .. of the tile, K-major in 64-key
            // swizzled blocks
            const int pkey = kh * kHalf + ch * 32;
            uint8_t *p_row = p_s + (t % kPBufs) * kPBytes + (pkey / 64) * kQBlockBytes + r * 128;
            float sum = 0.0f;
#pragma unroll
            for (int cc = 0; cc < 32 / 8; ++cc) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = exp2f(s[cc * 8 + 2 * j] - m_ref), p1 = exp2f(s[cc * 8 + 2 * j + 1] - m_ref);
                    sum += p0 + p1;
                    if (std::is_same<T, __nv_bfloat16>::value) {
                        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                        w[j] = *reinterpret_cast<uint32_t *>(&hh);
                    } else {
                        __half2 hh = __floats2half2_rn(p0, p1);
                        w[j] = *reinterpret_cast<uint32_t *>(&hh);
                    }
                }
                const int chunk = (pkey % 64) / 8 + cc;  // 16-byte chunk of the 128-byte row
                *reinterpret_cast<uint4 *>(p_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            l += sum;
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote_cta(lead(&p_full[2 * (t & 1) + kh]));
        }
        if (ok) ok = wait_all(&pv_done[2 * ((n_tiles - 1) & 1) + 1], (uint32_t)((n_tiles - 1) / 2) & 1u);
        named_bar_sync(1, kSoftmaxThreads);  // the last tile's maxima have been read: the row sums take their place
        x_sum[tid] = l;
        named_bar_sync(1, kSoftmaxThreads);
        if (ok) {
            tc_fence_after();
            l = (x_sum[tid] + x_sum[tid ^ 64]) + (x_sum[tid ^ 128] + x_sum[tid ^ 192]);
            const float inv = 1.0f / l;
            const float lse = (m_ref + log2f(l)) * kLn2;
            const size_t row = ((size_t)b * p.head_q + head) * p.num_splits + split;
            // This thread's 128 output values (half of its lane's 256 columns) are staged in shared memory (the rings are idle now: every MMA
            // of the pair has finished) and leave as one bulk copy per destination, so the writes reach
            // memory as whole lines whatever the row pitch.  Regions are 16 bytes longer than their data:
            // the float4 / uint4 stores of a quarter warp then fall into different banks.
            uint8_t *stage = smem + kOffA;
            const int d_first = kh * 256 + ch * 128;
            const uint32_t o_addr = lane_base + kColO + ch * 128;
            auto stage_f32 = [&](float *dst_g) {
                float *mine = reinterpret_cast<float *>(stage + (size_t)tid * (128 * 4 + 16));
                uint32_t buf2[32];
#pragma unroll 1
                for (int c = 0; c < 128 / 32; c += 2) {
                    tmem_ld32(o_addr + c * 32, buf);
                    tmem_ld32(o_addr + c * 32 + 32, buf2);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        reinterpret_cast<float4 *>(mine + c * 32)[j] =
                            make_float4(__uint_as_float(buf[4 * j]) * inv, __uint_as_float(buf[4 * j + 1]) * inv,
                                        __uint_as_float(buf[4 * j + 2]) * inv, __uint_as_float(buf[4 * j + 3]) * inv);
                        reinterpret_cast<float4 *>(mine + c * 32 + 32)[j] =
                            make_float4(__uint_as_float(buf2[4 * j]) * inv, __uint_as_float(buf2[4 * j + 1]) * inv,
                                        __uint_as_float(buf2[4 * j + 2]) * inv, __uint_as_float(buf2[4 * j + 3]) * inv);
                    }
                }
                fence_proxy_async();
                if (valid) bulk_store_s2g(dst_g, mine, 128 * 4);
                bulk_store_commit();
            };
            auto stage_t = [&](T *dst_g) {
                uint8_t *mine = stage + (size_t)tid * (128 * 2 + 16);
                uint32_t buf2[32];
#pragma unroll 1
                for (int c = 0; c < 128 / 32; c += 2) {
                    tmem_ld32(o_addr + c * 32, buf);
                    tmem_ld32(o_addr + c * 32 + 32, buf2);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        alignas(16) T tmp[8], tmp2[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            tmp[e] = from_float<T>(__uint_as_float(buf[8 * j + e]) * inv);
                            tmp2[e] = from_float<T>(__uint_as_float(buf2[8 * j + e]) * inv);
                        }
                        reinterpret_cast<uint4 *>(mine + c * 64)[j] = *reinterpret_cast<uint4 *>(tmp);
                        reinterpret_cast<uint4 *>(mine + c * 64 + 64)[j] = *reinterpret_cast<uint4 *>(tmp2);
                    }
                }
                fence_proxy_async();
                if (valid) bulk_store_s2g(dst_g, mine, 128 * 2);
                bulk_store_commit();
            };
            float *dst_f32 = p.num_splits > 1 ? p.part_o + row * kDimV + d_first
                                              : (p.o_f32 ? p.o_f32 + ((size_t)b * p.head_q + head) * kDimV + d_first : nullptr);
            const bool want_t = p.num_splits == 1 && o_out != nullptr;
            if (dst_f32) {
                stage_f32(dst_f32);
                if (want_t) bulk_store_wait_read();  // the staging bytes are about to be reused
            }
            if (want_t) stage_t(o_out + (size_t)b * p.o_row_stride + (size_t)head * kDimV + d_first);
            bulk_store_wait_read();
            if (kh == 0 && ch == 0 && valid) {
                if (p.num_splits > 1) {
                    p.part_lse[row] = lse;
                } else if (p.lse) {
                    p.lse[(size_t)b * p.head_q + head] = lse;
                }
            }
            tc_fence_before();
        }
    }

    if (!ok && lane == 0) report_timeout(p);
    __syncthreads();
    if (*abort_flag) {
        // give copies that may still be in flight a bounded time to land before the CTA retires
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) {
        }
    }
    tc_fence_before();
    cluster_sync_all();  // the peer may still read this CTA's shared memory (pair MMAs) or arrive on its barriers
    if (warp == kSWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace


SplitVariantInfo split_info_mla_2sm() { return {kTile, kHeads, 1}; }

// tm_q: rank-3 map over q [batch][head_q][576], box {64, min(64, head_q), 1}; tm_k: rank-2 map over the latent
// cache [rows][576], box {64, half a tile of keys, or a page when pages are shorter}; both with the 128-byte swizzle.  Grid (2, splits, batch) in clusters of
// two along x: the two CTAs of a key range.
cudaError_t launch_mla_2sm(bool bf16, const SplitParams &p, const CUtensorMap &tm_q, const CUtensorMap &tm_k,
                           cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 64 && !attr_set[dev]) {
        const void *kernels[4] = {(const void *)da_mla_2sm_kernel<__half, false>, (const void *)da_mla_2sm_kernel<__half, true>,
                                  (const void *)da_mla_2sm_kernel<__nv_bfloat16, false>,
                                  (const void *)da_mla_2sm_kernel<__nv_bfloat16, true>};
        for (const void *k : kernels) {
            err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (err != cudaSuccess) return err;
        }
        attr_set[dev] = true;
    }
    dim3 grid(2, p.num_splits, p.batch);
    const bool overlap = p.batch_order != nullptr;
    const bool short_pages = p.block_table && (1 << p.page_shift) < kHalf;
    if (bf16) {
        return short_pages ? launch_kernel(da_mla_2sm_kernel<__nv_bfloat16, true>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k)
                           : launch_kernel(da_mla_2sm_kernel<__nv_bfloat16, false>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k);
    }
    return short_pages ? launch_kernel(da_mla_2sm_kernel<__half, true>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k)
                       : launch_kernel(da_mla_2sm_kernel<__half, false>, grid, kThreads, kSmemBytes, stream, overlap, p, tm_q, tm_k);
}

}  // namespace da
