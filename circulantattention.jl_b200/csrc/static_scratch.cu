// ca_attention_fwd_static: the fused forward for callers that cannot allocate.
//
// Some hosts of this library may not call cudaMalloc (or any allocating
// routine) at the point where they need the forward pass: code running inside
// a memory pool they do not own, real-time loops with a fixed memory budget,
// plugins that are handed device pointers and nothing else.  The normal entry
// point, ca_attention_fwd, asks such a caller for a workspace (the packed copy
// of k and v that the tiled kernels stream from, or the score buffer of the
// entmax path).  This variant needs none: the workspace is a fixed array that
// lives in the library's own device image.
//
// Consequences the caller must know:
//   * every GPU that loads the library holds kStaticScratchBytes of device
//     memory until the process exits, whether or not this entry point is used;
//   * problems whose workspace exceeds that size are rejected with
//     CA_ERR_TOO_LARGE (use ca_attention_fwd with a caller workspace instead);
//   * all calls on one GPU share the one array, which keeps whatever the last
//     call left there.  Nothing in it has to start at zero (the pack kernel
//     rewrites every byte the forward kernel reads, padding included), but two
//     calls that overlap on the GPU -- different streams, or the same stream
//     from two host threads without ordering -- race on it;
//   * the first call on each device resolves the array's device address
//     (a host-side set-up step); make that first call before any stream
//     capture is begun.
#include "common.cuh"

#include <mutex>

namespace ca {
namespace {

constexpr size_t kStaticScratchBytes = (size_t)64 << 20;   // 64 MiB

// File-scope device array.  In host code this name is only a handle for the
// runtime, not a device address: the address is obtained once per device with
// cudaGetSymbolAddress below and that pointer is what kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the current device (resolved on first use).
int static_scratch(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices) {
        set_error("device ordinal %d is outside the supported range 0..%d", dev, kMaxDevices - 1);
        return CA_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return CA_OK;
}

}  // namespace
}  // namespace ca

extern "C" {

size_t ca_static_scratch_bytes(void) { return ca::kStaticScratchBytes; }

int ca_attention_fwd_static(const ca_desc* d, const void* q, const void* k, const void* v,
                            void* y, float* nz, float* stats, void* stream) {
    if (!d) { ca::set_error("descriptor is NULL"); return CA_ERR_NULL; }
    const size_t need = ca_attention_fwd_workspace(d, nz != nullptr);
    if (need > ca::kStaticScratchBytes) {
        ca::set_error("this problem needs a workspace of %zu bytes but the built-in scratch array holds %zu; "
                      "call ca_attention_fwd with a caller-provided workspace",
                      need, ca::kStaticScratchBytes);
        return CA_ERR_TOO_LARGE;
    }
    void* scratch = nullptr;
    if (need > 0) {
        int rc = ca::static_scratch(&scratch);
        if (rc) return rc;
    }
    return ca_attention_fwd(d, q, k, v, y, nz, stats, scratch, stream);
}

}  // extern "C"
