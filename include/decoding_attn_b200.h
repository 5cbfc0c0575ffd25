/* C ABI of the B200 (sm_100a) decode-attention library, libdecoding_attn_b200.so.
 *
 * Plain pointers and sizes only: every pointer marked "device" is a CUDA device pointer that the
 * caller owns and lends for the call; nothing here takes or returns a framework type.  All calls
 * are asynchronous on `stream` and make no host synchronisation.  Functions return DA_OK (0) or a
 * DA_ERR_* code; da_last_error() gives the message of the calling thread's last failure.
 *
 * Each entry point names the interface of Bruce-Lee-LY/decoding_attention that it stands in for.
 */
#ifndef DECODING_ATTN_B200_H_
#define DECODING_ATTN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum da_status {
    DA_OK = 0,
    DA_ERR_INVALID_ARG = 1, /* null pointer, bad size, misaligned pointer or stride */
    DA_ERR_UNSUPPORTED = 2, /* (dim, dim_v) pair or layout the kernels do not cover */
    DA_ERR_WORKSPACE = 3,   /* caller workspace too small, or the internal one could not grow */
    DA_ERR_CUDA = 4,        /* a CUDA runtime call failed; message in da_last_error() */
    DA_ERR_TIMEOUT = 5      /* a kernel's bounded wait ran out (reported by da_device_status) */
} da_status_t;

/* Arguments of one decode-attention call: o[b,h,:] = softmax(scale * q[b,h,:] . K_b^T + alibi) . V_b
 * for one query token per sequence over a packed variable-length KV cache.
 *
 * Replaces the argument list of decoding_attn() (csrc/ops/decoding_attn.h:29-30) and the kernel
 * parameter block DecodingParams that set_dmha_fwd_params() derives from it
 * (csrc/ops/decoding_attn.cpp:13-62, csrc/kernel/decoding_attn/decoding.h:11-51).  Zero-initialise
 * the struct, set struct_size = sizeof(da_decode_args_t), then fill what you need: every field the
 * reference does not have is optional and 0 / NULL selects the reference's behaviour.
 */
typedef struct da_decode_args {
    uint32_t struct_size;
    int32_t is_bf16;  /* 0: fp16, 1: bf16 (all of q, k, v, o) */
    int32_t is_alibi; /* add slope(h) * (key_pos - (len - 1)), slope(h) = 2^(-8 (h+1) / head_q) */
    int32_t num_splits; /* key-range splits per sequence; 0 = chosen by the library */

    const void *q;           /* device [batch, head_q, dim] */
    const void *k;           /* device [total_k, head_k, dim]; latent-KV cache for MLA */
    const void *v;           /* device [total_k, head_k, dim_v]; NULL = MLA: V is k[..., :dim_v] */
    void *o;                 /* device [batch, head_q, dim_v]; may be NULL if o_f32 is given */
    const int32_t *cu_seq_k; /* device [batch + 1], cumulative sequence lengths */

    int64_t max_seq_k; /* expected longest sequence: sizes the key-range splits.  Longer sequences are
                        * still read to their end (by their last split), only less evenly balanced;
                        * with a block table, its rows must cover every real length. */
    int64_t batch, head_q, head_k, dim, dim_v;

    /* Row strides in elements (distance between consecutive tokens); 0 = packed, i.e. what the
     * reference always assumes (csrc/ops/decoding_attn.cpp:32-46).  Heads are contiguous in a row. */
    int64_t q_row_stride, k_row_stride, v_row_stride, o_row_stride;

    float softmax_scale; /* <= 0 selects 1/sqrt(dim) (csrc/ops/decoding_attn.cpp:54) */
    uint32_t total_k; /* optional hint: rows of k that belong to the batch's sequences (for a packed cache, its row
                       * count), 0 = unknown.  With it the split planner can tell a ragged batch (mean length well
                       * below max_seq_k) from a uniform one; results do not depend on it. */

    float *lse;   /* optional device [batch, head_q]: natural-log sum-exp of the scaled scores */
    float *o_f32; /* optional device [batch, head_q, dim_v] packed: the result before rounding */

    /* Optional device [batch]: this KV range is keys [kv_pos_offset, kv_pos_offset + len) of a
     * sequence of kv_total_len keys held elsewhere (key-range sharding); only ALiBi uses them. */
    const int32_t *kv_pos_offset;
    const int32_t *kv_total_len;

    void *workspace;        /* optional device scratch for split partials; NULL = library-owned */
    size_t workspace_bytes; /* size of `workspace` */

    void *stream; /* cudaStream_t */

    /* Paged cache (optional; NULL = packed, the reference's layout).  k and v then point to page
     * pools [num_pages * page_size, head_k, dim] and key j of sequence b lives in row
     * block_table[b * block_table_stride + j / page_size] * page_size + j % page_size.
     * Lengths still come from cu_seq_k (differences only).  page_size: a power of two >= 16 (pages
     * shorter than a 64-key tile are fetched one TMA box per page).
     * The reference has no paged input; its Python benchmark builds this layout for the libraries
     * it compares against (benchmarks/python/benchmark_decoding_attn.py:129-151, :182-190). */
    const int32_t *block_table; /* device [batch, block_table_stride] */
    int64_t block_table_stride; /* elements per row, >= ceil(longest sequence / page_size) */
    int32_t page_size;

    /* Quantised cache (optional).  kv_dtype 0: k and v hold the type of q (the reference's only case).
     * DA_KV_FP8_E4M3 / DA_KV_INT8: one byte per element (FP8 e4m3, or a signed 8-bit integer);
     * DA_KV_INT4: signed 4-bit integers, two per byte, the element with the even index in the low nibble.
     * The tensors stand for k * k_scale and v * v_scale (one scale per tensor; <= 0 selects 1).  q, o
     * and all arithmetic stay as they are; strides and dims still count elements (row strides: multiples
     * of 16 bytes).  Supported with v given and (dim, dim_v) one of (64,64) (96,96) (128,128) (256,256);
     * the latent-KV shape returns DA_ERR_UNSUPPORTED.  The reference lists KV-cache quantisation as not
     * done (README.md:154-156). */
    int32_t kv_dtype;
    float k_scale, v_scale;
} da_decode_args_t;

enum { DA_KV_SAME_AS_Q = 0, DA_KV_FP8_E4M3 = 1, DA_KV_INT8 = 2, DA_KV_INT4 = 3 };

/* Runs decode attention.  Stands in for decoding_attn() (csrc/ops/decoding_attn.h:29-30,
 * csrc/ops/decoding_attn.cpp:70-76) and everything below it: run_dmha_fwd / DA_FP16_SWITCH /
 * DA_HEADDIM_SWITCH (csrc/ops/decoding_attn.cpp:64-68, csrc/common/common.h:62-96), the per-shape
 * run_dmha_fwd_<T,HD,HDV> (csrc/kernel/decoding_attn/decoding_fwd_hd*.cu), the launcher
 * (decoding_fwd_launch_template.h:11-31) and the kernel (decoding_fwd_kernel.h:13-236).
 * Supported (dim, dim_v): (64,64) (96,96) (128,128) (256,256) and (576,512) with v == NULL, as in
 * the reference; any other pair returns DA_ERR_UNSUPPORTED instead of silently doing nothing.
 * A zero-length sequence gives a zero row (LSE = -inf) instead of an unwritten one.
 * With workspace == NULL the library keeps one grow-only scratch buffer per device; calls that may
 * overlap on one device (different streams) must then pass their own workspace, and so must a call
 * made during stream capture (growing the buffer calls cudaMalloc).
 * Bounded waits: a kernel whose wait runs out records it for da_device_status(); the CTAs of that
 * same launch that have not started yet retire at once, later launches are not affected.  A replayed
 * CUDA graph repeats its launch ids: after a timeout inside a replay, read da_device_status() (which
 * clears the record) before replaying again. */
int da_decode_fwd(const da_decode_args_t *args);

/* The same call for a caller whose tensors live in HOST memory (q, k, v, o, cu_seq_k, lse are host
 * pointers, packed rows; pinned memory gives full copy speed).  Copies the inputs to device
 * buffers the library keeps per device, runs da_decode_fwd on `stream`, copies o (and lse) back
 * and returns after the stream has drained.  This is the shape of the reference's own benchmark
 * harness, which owns host and device copies of every tensor and moves them around the call
 * (csrc/common/tensor.h:26-38, :74-83; csrc/common/tester.h:98-119). */
int da_decode_fwd_host(const da_decode_args_t *host_args);

/* da_decode_fwd for a caller that cannot allocate device memory and has no buffer to lend: the
 * split partials go to a fixed 16 MiB array inside the library image (da_static_scratch_bytes()).
 * Meant for hosts whose memory is fully planned by someone else -- an engine that gave all of HBM
 * to its KV-cache pool, code running where calls into the CUDA allocator are forbidden.  Leave
 * args->workspace NULL.  Returns DA_ERR_WORKSPACE, without launching anything, when the call would
 * need more than the array holds (num_splits = 1 needs at most 4 bytes per sequence and always
 * fits).  It calls no cudaMalloc / cudaFree.  The first call on a device looks up the array's
 * device address (cudaGetSymbolAddress), which is also the moment the runtime puts the array on
 * that device (device code is loaded lazily): make that first call at start-up, before the host
 * commits the rest of the memory, and outside any stream capture.  All calls on a device share the
 * array, which keeps the previous call's bytes (nothing in it needs clearing): calls that overlap
 * on the GPU race, so keep them on one stream.
 * This entry point has no counterpart in the reference, whose kernel keeps its only scratch in
 * shared memory. */
int da_decode_fwd_static(const da_decode_args_t *args);
size_t da_static_scratch_bytes(void);

/* Scratch bytes da_decode_fwd needs for these arguments: the split partials (none when it will not
 * split) plus, for grids of more than one wave, 4 bytes per sequence for the launch order.  No reference
 * counterpart: the reference kernel keeps its only scratch, the score row, in shared memory
 * (decoding_fwd_launch_template.h:14-18). */
size_t da_decode_workspace_bytes(const da_decode_args_t *args);

/* The split count da_decode_fwd will use for these arguments (diagnostics / benchmarks). */
int da_decode_num_splits(const da_decode_args_t *args);
/* The same for a device with `sm_count` SMs, without touching any device (no pointer is dereferenced): what the
 * host-side tests pin the planner's decisions with.  -1 on invalid arguments. */
int da_plan_num_splits(const da_decode_args_t *args, int sm_count);

/* Merges `num_parts` partial results of the same rows, each computed over a disjoint key range:
 *   o = sum_r exp(lse_r - LSE) o_r,  LSE = log sum_r exp(lse_r).
 * part_o: device fp32, part r row i at part_o + r*part_stride_o + i*row_stride_o (dim_v contiguous);
 * part_lse: device fp32, at part_lse + r*part_stride_lse + i*row_stride_lse.  rows = batch*head_q.
 * o (type per is_bf16, row i at o + i*dim_v), o_f32 and lse are optional outputs.
 * No reference counterpart (the reference never splits a row); it is the second step of key-range
 * sharding across GPUs, run after the (o_r, lse_r) records have been gathered. */
int da_merge_partials(const float *part_o, const float *part_lse, int32_t num_parts, int64_t rows, int32_t dim_v,
                      int64_t part_stride_o, int64_t row_stride_o, int64_t part_stride_lse, int64_t row_stride_lse,
                      void *o, float *o_f32, float *lse, int32_t is_bf16, void *stream);

/* Key-range sharding without a collective library: one kernel per rank that (1) stores this rank's
 * record `rec` (o fp32 [rows, dim_v] followed by lse fp32 [rows]) into every peer's gather buffer
 * with peer stores and raises a flag there, (2) waits -- bounded -- for all peers' flags of this
 * step in its own buffer, (3) merges the `world` records into o [rows, dim_v] (+ optional lse).
 * peer_bufs[r] is the device address, valid on THIS device, of rank r's gather buffer (a symmetric
 * allocation of da_exchange_buffer_bytes(world, rows, dim_v) bytes, zero-filled once before the
 * first step; peer_bufs[rank] is the local one).  `epoch` numbers the steps: 1, 2, 3, ... the same
 * on every rank.  All ranks must call it once per step, each on its own GPU, and be running
 * concurrently.  A peer that never shows up makes the wait run out: the rows are left unwritten
 * and da_device_status() reports DA_ERR_TIMEOUT.  No reference counterpart (single-GPU library). */
int da_exchange_merge(const float *rec, void *const *peer_bufs, int32_t world, int32_t rank, int64_t rows,
                      int32_t dim_v, uint32_t epoch, void *o, float *lse, int32_t is_bf16, void *stream);
size_t da_exchange_buffer_bytes(int32_t world, int64_t rows, int32_t dim_v);
/* The same with the bound of the wait for the peers' flags given in SM clocks (0 = the default, about a
 * quarter of a second).  A short bound lets a host that watches its peers give up on a dead one quickly;
 * the tests use it to run the give-up path (a peer that never posts) without stalling a GPU.
 * No reference counterpart. */
int da_exchange_merge_bounded(const float *rec, void *const *peer_bufs, int32_t world, int32_t rank, int64_t rows,
                              int32_t dim_v, uint32_t epoch, void *o, float *lse, int32_t is_bf16, void *stream,
                              int64_t max_wait_cycles);

/* Profiling hook for the calling thread: while both are non-NULL, da_decode_fwd records the CUDA
 * event `start_event` on the stream just before its main (key-streaming) kernel and `stop_event`
 * just after it, so a benchmark can time that kernel apart from the merge kernel.  Pass NULLs to
 * switch it off.  The reference times whole calls only (CudaTimer, csrc/common/cuda_timer.h:10-52). */
void da_set_profile_events(void *start_event, void *stop_event);

/* Reads and clears the current device's kernel status word (synchronises the device).  Returns
 * DA_OK, or DA_ERR_TIMEOUT if a kernel gave up a bounded wait since the last call.  The reference
 * has no counterpart: its kernel has no waits and its host checks exit() (common.h:17-49). */
int da_device_status(void);

/* Launches a one-warp kernel that waits, with a bound of about a millisecond, on a barrier nobody
 * will ever arrive on, and gives up the way the attention kernels' bounded waits do.  Afterwards
 * da_device_status() returns DA_ERR_TIMEOUT once (and clears the word); the context stays usable.
 * For testing the failure path without faulting or hanging a GPU.  No reference counterpart. */
int da_selftest_wait_timeout(void *stream);

const char *da_status_string(int status);
const char *da_last_error(void);

/* Number of kernels this library has launched from the calling process (all threads). */
uint64_t da_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* DECODING_ATTN_B200_H_ */
