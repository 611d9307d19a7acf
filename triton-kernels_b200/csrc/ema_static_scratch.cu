// Backward pass that allocates nothing: the partial sums of the decay gradient live in a fixed array
// in device memory that is part of this library's image, instead of a workspace the caller provides.
//
// Who needs this.  ema_b200_bwd() asks its caller for a workspace, and the Python layer gets one from
// torch's caching allocator.  Some callers cannot do that at the moment of the call:
//   * a host that binds the C interface directly and has handed all of device memory to its own arena at
//     start-up, so that a later cudaMalloc would fail or fragment the arena;
//   * a latency-critical loop, where cudaMalloc / cudaFree synchronise the whole device and stall every
//     other stream of the process;
//   * code running while the framework's allocator must not be entered (inside one of its callbacks,
//     or on a thread that holds its lock).
// For those, this entry point needs only the input and output tensors.  The price is a size limit and
// the loss of concurrency described below.
//
// The array is reserved once per device when the library's image is loaded there; the call itself never
// calls cudaMalloc, cudaFree, or any library routine that allocates.
#include <mutex>

#include "ema_b200.h"
#include "ema_common.cuh"

namespace {

// 8 MiB: enough for a per-head decay at b*h*ceil(d/16)*ceil(L/128) <= 262,000 or so (e.g. b=16, h=2,
// d=1024, L=8192 needs 4 MiB), and for a per-step decay at b*h*ceil(d/16)*ceil(L/128)*128 <= 2,097,152.
constexpr size_t kScratchFloats = size_t(2) << 20;
constexpr size_t kScratchBytes = kScratchFloats * sizeof(float);

static __device__ __align__(256) float g_static_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float *g_scratch_ptr[kMaxDevices];  // device address of g_static_scratch, per device; null until looked up

// Looks the array's address up on the current device (first call on that device only).
int scratch_for_current_device(float **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { ema::set_last_cuda_error(e); return EMA_ERR_CUDA; }
    if (dev < 0 || dev >= kMaxDevices) return EMA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
        float *ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch);
        if (e != cudaSuccess || !ptr) { ema::set_last_cuda_error(e); return EMA_ERR_CUDA; }
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return EMA_OK;
}

}  // namespace

extern "C" size_t ema_b200_static_scratch_limit(void) { return kScratchBytes; }

extern "C" int ema_b200_bwd_static_scratch(const ema_b200_problem *p, const void *x, const float *decay,
                                           const void *dy, const float *tile_states, void *dx, float *ddecay,
                                           void *stream) {
    if (!p) return EMA_ERR_BADARG;
    const size_t need = ema_b200_bwd_workspace_bytes(p);
    if (need == 0) return EMA_ERR_BADARG;              // the problem description itself is invalid
    if (need > kScratchBytes) return EMA_ERR_SCRATCH_LIMIT;  // nothing was launched
    float *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    // Nothing in the scratch has to start at zero: the backward kernel writes every partial sum that the
    // reduction kernels read afterwards, in the same stream, and ddecay is overwritten, not accumulated.
    // The scratch pointer reaches the kernels as their partial-sum buffer.
    return ema_b200_bwd(p, x, decay, dy, tile_states, dx, ddecay, /*dfinal_state=*/nullptr,
                        /*dinit_state=*/nullptr, /*stop_below=*/0.f, scratch, kScratchBytes, stream);
}
