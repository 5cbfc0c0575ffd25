// TEST INFRASTRUCTURE ONLY -- CPU oracle for single-query ("decode") attention.
//
// This file restates, step for step, the CPU attention that the reference project uses to check
// its GPU kernel: Tester<T>::attn_cpu in csrc/common/tester.h:133-259 of
// Bruce-Lee-LY/decoding_attention.  It is the checker for the CUDA path of this repository and the
// timed CPU baseline of the benchmark; the product path never links, imports or calls it.
//
// Parity pin: oracle/ref_attn_cpu.cpp compiles the reference's own tester.h (where it lies in a
// checkout of the reference) into oracle/_ref/, and tests/test_oracle.py requires this restatement
// to be bit-identical to it on fixed-length inputs; committed golden vectors made by the reference
// test-suite's torch_attn (tests/test_decoding_attn.py:35-57) pin it a second time.
//
// What is kept from tester.h (line numbers of that file):
//   * S = q.k accumulated in fp32, sequentially over d, multiply then add (no fused multiply-add)
//     (:166-176);
//   * tmp = S * scale, scale = 1/sqrt(dim) computed in double and narrowed to float (:186, :201);
//   * ALiBi: slope(h) = 1 / exp2(8 (h+1) / head_q) in double, narrowed to float (:193); the bias
//     slope * (sk - sq - row_shift), row_shift = seq_k - seq_q, is added for sk < sq + row_shift
//     (:202-205) -- with seq_q = 1 the excluded last key would get bias 0 anyway;
//   * max over the row, expf(tmp - max), sequential fp32 sum, divide (:206-219);
//   * O = sum_sk P * V in fp32, sequentially over sk, multiply then add, V addressed with row pitch
//     head_k * dim (:244, :247), V = K when no V tensor is given (:149) and d_v = dim_v (:142);
//   * one rounding to fp16 / bf16, round-to-nearest-even (:250-254).
// Deliberate deviations (none changes a result the reference can produce):
//   * score/probability scratch is per (batch, head) row.  The reference indexes shared S/P buffers
//     with the *current* sequence's length as pitch (:176, :201, :218), so rows of different
//     sequences overlap when lengths differ; its harness only builds equal lengths (:122-129);
//   * inputs are passed in as raw 16-bit patterns; nothing is allocated with CUDA;
//   * rows are independent, so they are spread over OpenMP threads (bit-identical per row);
//   * the O = P.V loop nest runs sk outermost and d innermost: every o[d] still sees the same
//     sequence of additions, but the inner loop vectorises;
//   * optional extras used by the tests of this repository: natural-log LSE = max + log(sum) per row,
//     a caller-supplied softmax scale, and a (position offset, total length) pair so that a shard
//     of a longer sequence gets the ALiBi bias of the whole sequence;
//   * a zero-length sequence yields a zero output row and LSE = -inf (the reference leaves the row
//     unwritten, csrc/kernel/decoding_attn/decoding_fwd_kernel.h:16-18).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float half_bits_to_float(uint16_t h) {
    // IEEE binary16 -> binary32, exact (what __half2float does).
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t float_to_half_bits(float f) {
    // binary32 -> binary16, round-to-nearest-even (what __float2half does).
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t abs = x & 0x7fffffffu;
    if (abs >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((abs > 0x7f800000u) ? 0x200u | ((abs >> 13) & 0x3ffu) : 0u));
    }
    if (abs >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (abs < 0x38800000u) {  // result is subnormal or zero
        if (abs < 0x33000000u) return (uint16_t)sign;  // < 2^-25 -> 0
        int e = (int)(abs >> 23);
        uint32_t man = (abs & 0x7fffffu) | 0x800000u;
        int shift = 126 - e;  // 14..24
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) ++half_man;
        return (uint16_t)(sign | half_man);
    }
    uint32_t man = abs & 0x7fffffu;
    uint32_t e = (abs >> 23) - 112u;
    uint32_t out = (e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (out & 1u))) ++out;
    return (uint16_t)(sign | out);
}

inline float bf16_bits_to_float(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t float_to_bf16_bits(float f) {
    // round-to-nearest-even, NaN kept quiet (what __float2bfloat16 does).
    uint32_t x;
    std::memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

template <bool kBf16>
inline float load_elem(const uint16_t *p) {
    return kBf16 ? bf16_bits_to_float(*p) : half_bits_to_float(*p);
}

template <bool kBf16>
void attn_cpu_impl(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *o, float *o_f32, float *lse,
                   const int32_t *cu_seq_k, int64_t batch, int64_t head_q, int64_t head_k, int64_t dim, int64_t dim_v,
                   int is_alibi, float scale, const int32_t *kv_pos_offset, const int32_t *kv_total_len,
                   int64_t batch_begin, int64_t batch_end) {
    const int64_t head_ratio = head_q / head_k;
    const uint16_t *vv = v ? v : k;
    const int64_t kv_pitch = head_k * dim;  // tester.h:244 -- V rows use the K pitch
    const int64_t rows = (batch_end - batch_begin) * head_q;
    (void)batch;

#pragma omp parallel
    {
        std::vector<float> s;
        std::vector<float> qf((size_t)dim);
        std::vector<float> acc((size_t)dim_v);
#pragma omp for schedule(dynamic, 1)
        for (int64_t row = 0; row < rows; ++row) {
            const int64_t b = batch_begin + row / head_q;
            const int64_t h = row % head_q;
            const int64_t h_k = h / head_ratio;
            const int64_t sum_seq_k = cu_seq_k[b];
            const int64_t seq_k = (int64_t)cu_seq_k[b + 1] - sum_seq_k;
            uint16_t *o_row = o ? o + (b * head_q + h) * dim_v : nullptr;
            float *of_row = o_f32 ? o_f32 + (b * head_q + h) * dim_v : nullptr;
            if (seq_k <= 0) {
                for (int64_t d = 0; d < dim_v; ++d) {
                    if (o_row) o_row[d] = 0;
                    if (of_row) of_row[d] = 0.0f;
                }
                if (lse) lse[b * head_q + h] = -std::numeric_limits<float>::infinity();
                continue;
            }
            s.resize((size_t)seq_k);
            for (int64_t d = 0; d < dim; ++d) qf[d] = load_elem<kBf16>(q + (b * head_q + h) * dim + d);

            // S = Q K^T  (tester.h:158-180)
            for (int64_t sk = 0; sk < seq_k; ++sk) {
                const uint16_t *k_row = k + (sum_seq_k + sk) * kv_pitch + h_k * dim;
                float a = 0.0f;
                for (int64_t d = 0; d < dim; ++d) {
                    a += qf[d] * load_elem<kBf16>(k_row + d);
                }
                s[sk] = a;
            }

            // P = softmax(S * scale + alibi)  (tester.h:187-229)
            const float h_slope = is_alibi ? (float)(1.0 / exp2(8.0 * (double)(h + 1) / (double)head_q)) : 0.0f;
            const int64_t pos0 = kv_pos_offset ? kv_pos_offset[b] : 0;
            const int64_t total = kv_total_len ? kv_total_len[b] : seq_k;
            const int64_t row_shift = total - 1;
            float max_s = -std::numeric_limits<float>::max();
            for (int64_t sk = 0; sk < seq_k; ++sk) {
                float t = s[sk] * scale;
                if (is_alibi && (pos0 + sk) < row_shift) {
                    t += h_slope * (float)((int)(pos0 + sk) - (int)row_shift);
                }
                s[sk] = t;
                max_s = std::max(max_s, t);
            }
            float sum_s = 0.0f;
            for (int64_t sk = 0; sk < seq_k; ++sk) {
                s[sk] = std::exp(s[sk] - max_s);
                sum_s += s[sk];
            }
            for (int64_t sk = 0; sk < seq_k; ++sk) s[sk] = s[sk] / sum_s;
            if (lse) lse[b * head_q + h] = max_s + std::log(sum_s);

            // O = P V  (tester.h:232-258)
            for (int64_t d = 0; d < dim_v; ++d) acc[d] = 0.0f;
            for (int64_t sk = 0; sk < seq_k; ++sk) {
                const uint16_t *v_row = vv + (sum_seq_k + sk) * kv_pitch + h_k * dim;
                const float p = s[sk];
                for (int64_t d = 0; d < dim_v; ++d) {
                    acc[d] += p * load_elem<kBf16>(v_row + d);
                }
            }
            for (int64_t d = 0; d < dim_v; ++d) {
                if (o_row) o_row[d] = kBf16 ? float_to_bf16_bits(acc[d]) : float_to_half_bits(acc[d]);
                if (of_row) of_row[d] = acc[d];
            }
        }
    }
}

}  // namespace

extern "C" {

// q [batch, head_q, dim], k [total_k, head_k, dim], v [total_k, head_k, dim_v] or NULL (then V = the
// first dim_v elements of each K row), o [batch, head_q, dim_v] (may be NULL), all 16-bit patterns.
// o_f32 (optional) receives the unrounded fp32 result, lse (optional) the natural-log LSE.
// scale <= 0 selects the reference's 1/sqrt(dim).  kv_pos_offset / kv_total_len (optional, per
// sequence) place a shard inside a longer sequence for the ALiBi bias.  Only sequences
// [batch_begin, batch_end) are computed.  threads <= 0 keeps the OpenMP default.
int oracle_attn_cpu(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *o, float *o_f32, float *lse,
                    const int32_t *cu_seq_k, int64_t batch, int64_t head_q, int64_t head_k, int64_t dim,
                    int64_t dim_v, int is_alibi, int is_bf16, float scale, const int32_t *kv_pos_offset,
                    const int32_t *kv_total_len, int64_t batch_begin, int64_t batch_end, int threads) {
    if (!q || !k || !cu_seq_k || head_k <= 0 || head_q % head_k != 0 || dim <= 0 || dim_v <= 0) return 1;
    if (v && dim_v != dim) return 2;  // the reference addresses V with the K pitch (tester.h:244)
    if (!v && dim_v > dim) return 2;
    if (batch_begin < 0 || batch_end > batch || batch_begin > batch_end) return 3;
    if (!(scale > 0.0f)) scale = (float)(1.0 / std::sqrt((double)dim));
#ifdef _OPENMP
    int saved = omp_get_max_threads();
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
    if (is_bf16) {
        attn_cpu_impl<true>(q, k, v, o, o_f32, lse, cu_seq_k, batch, head_q, head_k, dim, dim_v, is_alibi, scale,
                            kv_pos_offset, kv_total_len, batch_begin, batch_end);
    } else {
        attn_cpu_impl<false>(q, k, v, o, o_f32, lse, cu_seq_k, batch, head_q, head_k, dim, dim_v, is_alibi, scale,
                             kv_pos_offset, kv_total_len, batch_begin, batch_end);
    }
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(saved);
#endif
    return 0;
}

int oracle_num_procs(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

// Conversions exported so that tests can check them against torch's.
float oracle_half_to_float(uint16_t h) { return half_bits_to_float(h); }
float oracle_bf16_to_float(uint16_t h) { return bf16_bits_to_float(h); }
uint16_t oracle_float_to_half(float f) { return float_to_half_bits(f); }
uint16_t oracle_float_to_bf16(float f) { return float_to_bf16_bits(f); }
}
