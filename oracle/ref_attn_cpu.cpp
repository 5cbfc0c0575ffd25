// TEST INFRASTRUCTURE ONLY -- runs the reference project's own CPU attention, unmodified.
//
// This translation unit #includes csrc/common/tester.h from a checkout of
// Bruce-Lee-LY/decoding_attention (the include path is given on the compiler command line by
// oracle/Makefile; no reference source is copied here) and calls its private member
// Tester<T>::attn_cpu (tester.h:133-259) on caller-supplied tensors.  The built library goes to
// oracle/_ref/ and is used (a) to pin oracle/attn_cpu.cpp bit-for-bit and (b) as the timed
// "reference" CPU baseline of the benchmark.
//
// tester.h allocates every tensor twice -- host and device (tensor.h:26-28) -- and fills it from an
// unseeded std::random_device (tensor.h:31-36).  Neither needs a GPU for the CPU path, so the CUDA
// runtime calls it makes are satisfied by oracle/fake_cudart.c (host malloc/memcpy), and the random
// host contents are overwritten with the caller's inputs before attn_cpu runs.  The harness only
// builds equal-length batches (tester.h:122-129); the entry point therefore takes one seq_k.
//
// The reference is single-threaded.  `threads` > 1 runs that many independent Tester instances on
// disjoint slices of the batch, each executing the unmodified attn_cpu.
#include <cuda_runtime_api.h>
#include <fcntl.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <ctime>
#include <functional>
#include <limits>
#include <memory>
#include <mutex>
#include <numeric>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#define private public
#include "tester.h"
#undef private

namespace {

// The harness logs every allocation to stderr (tensor.h:40).  While any call is in flight stderr is
// parked on /dev/null; calls may overlap (one per host thread), hence the count.
std::mutex g_quiet_mu;
int g_quiet_users = 0, g_saved_err = -1;
void quiet_enter() {
    std::lock_guard<std::mutex> lock(g_quiet_mu);
    if (g_quiet_users++ == 0) {
        fflush(stderr);
        g_saved_err = dup(2);
        int devnull = open("/dev/null", O_WRONLY);
        if (g_saved_err >= 0 && devnull >= 0) dup2(devnull, 2);
        if (devnull >= 0) close(devnull);
    }
}
void quiet_leave() {
    std::lock_guard<std::mutex> lock(g_quiet_mu);
    if (--g_quiet_users == 0 && g_saved_err >= 0) {
        fflush(stderr);
        dup2(g_saved_err, 2);
        close(g_saved_err);
        g_saved_err = -1;
    }
}

template <typename T>
void run_slice(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *o, size_t b0, size_t nb,
               size_t seq_k, size_t head_q, size_t head_k, size_t dim, size_t dim_v, bool is_alibi) {
    Tester<T> t(nb, 1, seq_k, head_q, head_k, dim, dim_v, false, is_alibi, nullptr, 1, 10, 100, false);
    std::memcpy((void *)t.m_Q->getHostPtr(), q + b0 * head_q * dim, nb * head_q * dim * 2);
    std::memcpy((void *)t.m_K->getHostPtr(), k + b0 * seq_k * head_k * dim, nb * seq_k * head_k * dim * 2);
    if (t.m_V) {
        std::memcpy((void *)t.m_V->getHostPtr(), v + b0 * seq_k * head_k * dim_v, nb * seq_k * head_k * dim_v * 2);
    }
    t.attn_cpu(t.m_Q, t.m_K, t.m_V, t.m_base, t.m_cu_seq_k, seq_k, dim_v, false, is_alibi);
    std::memcpy(o + b0 * head_q * dim_v, (const void *)t.m_base->getHostPtr(), nb * head_q * dim_v * 2);
}

}  // namespace

extern "C" int ref_attn_cpu(const uint16_t *q, const uint16_t *k, const uint16_t *v, uint16_t *o, int64_t batch,
                            int64_t seq_k, int64_t head_q, int64_t head_k, int64_t dim, int64_t dim_v, int is_alibi,
                            int is_bf16, int threads) {
    if (!q || !k || !o || batch <= 0 || seq_k <= 0) return 1;
    if ((dim == dim_v) != (v != nullptr)) return 2;  // tester.h:66 builds V only when dim == dim_v
    int n = std::max(1, std::min<int>(threads, (int)batch));
    quiet_enter();
    std::vector<std::thread> pool;
    for (int i = 0; i < n; ++i) {
        size_t b0 = (size_t)batch * i / n, b1 = (size_t)batch * (i + 1) / n;
        if (b1 == b0) continue;
        auto fn = [=]() {
            if (is_bf16) {
                run_slice<__nv_bfloat16>(q, k, v, o, b0, b1 - b0, seq_k, head_q, head_k, dim, dim_v, is_alibi);
            } else {
                run_slice<half>(q, k, v, o, b0, b1 - b0, seq_k, head_q, head_k, dim, dim_v, is_alibi);
            }
        };
        if (n == 1) {
            fn();
        } else {
            pool.emplace_back(fn);
        }
    }
    for (auto &t : pool) t.join();
    quiet_leave();
    return 0;
}
