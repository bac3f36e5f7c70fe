// Backward entry point for callers that are not allowed to allocate device memory.
//
// Some hosts cannot call cudaMalloc at the point where they need the backward pass:
// code running inside a memory pool that is already fully handed out, plugins that
// are only given their input / output buffers, or hosts that forbid allocation after
// start-up.  The fused backward needs a small scratch buffer (one float per
// (batch, query, head): delta = rowsum(out * dout) - dlse).  Here that scratch is a
// fixed array inside the library image, so the caller passes inputs and outputs only.
//
// Limits and rules
//   * the array is 4 MiB per GPU that loads the library, held until the process exits; a problem
//     fits when natten_workspace_bytes(params, NATTEN_OP_FUSED_BWD) <= 4 MiB: one accumulator per
//     (batch, query, head) -- 4 bytes, 8 in double precision -- plus the partial sums of the
//     additional tokens' gradients when there are any (1 048 576 rows in the plain 4-byte case);
//     larger problems are rejected with NATTEN_E_TOO_LARGE and nothing is launched;
//   * the first call on each device looks up the array's device address (no
//     allocation, but a runtime query): make that first call before any stream capture;
//   * every call on a device uses the same array, so two calls whose kernels may run
//     at the same time (different streams) race on it -- keep them on one stream or
//     order them with events.  Nothing in the array has to start at zero: each call
//     overwrites every entry it later reads.
#include "../../include/natten_b200.h"

#include <cuda_runtime.h>
#include <mutex>

namespace {

constexpr size_t kStaticRows = 1u << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_scratch[kStaticRows];

std::mutex g_mutex;
void* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the array on the current device.  In host code the array's name
// is only a handle; the address the kernels need comes from cudaGetSymbolAddress.
int scratch_for_current_device(void** out)
{
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= kMaxDevices) return NATTEN_E_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (err != cudaSuccess) return (int)err;
        if (!p) return NATTEN_E_UNSUPPORTED;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return NATTEN_OK;
}

} // namespace

extern "C" {

size_t natten_static_scratch_bytes(void) { return kStaticRows * sizeof(float); }

int natten_fused_bwd_static(const natten_params_t* params, const void* q, const void* k, const void* v,
                            const void* extra_k, const void* extra_v, const void* out, const void* lse,
                            const void* dout, const void* dlse, void* dq, void* dk, void* dv,
                            void* dextra_k, void* dextra_v, void* stream)
{
    if (!params) return NATTEN_E_INVALID;
    const size_t need = natten_workspace_bytes(params, NATTEN_OP_FUSED_BWD);
    if (need > natten_static_scratch_bytes()) return NATTEN_E_TOO_LARGE;
    void* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != NATTEN_OK) return rc;
    return natten_fused_bwd(params, q, k, v, extra_k, extra_v, out, lse, dout, dlse, dq, dk, dv,
                            dextra_k, dextra_v, scratch, natten_static_scratch_bytes(), stream);
}

} // extern "C"
