// da_decode_fwd_static(): decode attention for callers that must not allocate device memory.
//
// Who needs it: a host that runs inside somebody else's memory plan -- a serving engine that has
// handed every byte of HBM to its own KV-cache pool, a plugin called from a region where the CUDA
// allocator is off limits (library code invoked under a caller-owned allocator lock, a real-time
// loop that forbids calls which may block on the driver's allocation path) -- cannot let this
// library call cudaMalloc for the split-KV partials, and may not have a spare buffer to lend as
// `workspace` either.  For them the partials live in a fixed array that is part of the library
// image: kStaticScratchBytes on every GPU that uses this entry point.  The CUDA runtime loads a
// module's device code lazily, so the array is materialised on a device by the first call there
// (the cudaGetSymbolAddress below), not when the library is loaded: a host that is about to commit
// all of its memory should make one call per device at start-up, while the memory is still there,
// and nothing is allocated by any later call.
//
// The array is shared by all calls on a device and keeps whatever the last call left in it.  That
// is harmless here: the split kernels write every partial (row, split) that the merge kernel will
// read, and the merge kernel derives from cu_seq_k which splits exist, so nothing has to start at
// zero and nothing is cleared.  Two calls that overlap on one GPU (different streams) would write
// the same bytes and race; serialise them or give the second one its own `workspace` through
// da_decode_fwd.
#include <cstdio>
#include <mutex>

#include "../../include/decoding_attn_b200.h"
#include "da_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB per GPU

// In host code this name is only a handle for the runtime (its host-side shadow); the address the
// kernels need comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void *g_scratch_ptr[64] = {};

}  // namespace

extern "C" int da_decode_fwd_static(const da_decode_args_t *args) {
    if (!args) return da::report_error(DA_ERR_INVALID_ARG, "args is NULL");
    if (args->workspace || args->workspace_bytes) {
        return da::report_error(DA_ERR_INVALID_ARG,
                                "da_decode_fwd_static uses the library's static scratch: leave workspace NULL");
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return da::report_error(DA_ERR_CUDA, "cudaGetDevice failed");
    void *ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!g_scratch_ptr[dev]) {
            // First call on this device (it is current): resolve the device address of the array.
            e = cudaGetSymbolAddress(&g_scratch_ptr[dev], g_static_scratch);
            if (e != cudaSuccess) {
                g_scratch_ptr[dev] = nullptr;
                return da::report_error(DA_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed");
            }
        }
        ptr = g_scratch_ptr[dev];
    }
    const size_t need = da_decode_workspace_bytes(args);
    if (need > kStaticScratchBytes) {
        char msg[256];
        snprintf(msg, sizeof(msg),
                 "this call needs %zu bytes of split scratch but the static scratch holds %zu: lower num_splits "
                 "(1 needs none) or use da_decode_fwd with a workspace",
                 need, kStaticScratchBytes);
        return da::report_error(DA_ERR_WORKSPACE, msg);
    }
    da_decode_args_t a = *args;
    a.workspace = ptr;
    a.workspace_bytes = kStaticScratchBytes;
    return da_decode_fwd(&a);
}

extern "C" size_t da_static_scratch_bytes(void) { return kStaticScratchBytes; }
