// Shared device/host helpers for the EMA kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ema_b200.h"
#include "ema_bounds.cuh"

namespace ema {

// Everything a fused launch needs.  Strides are in elements, as in ema_b200_problem.
struct FusedParams {
    const void *x;
    const float *decay;
    // forward only, optional: per-step input weights [b, L, h] replacing the convention's (1 - a or 1), and per-step
    // output weights applied to what is written (the states stay unweighted); both with the decay's strides
    const float *in_weight;
    const float *out_weight;
    const void *dy;
    void *out;  // y (forward) or dx (backward)
    float *chunk_states;
    float *tile_states;
    const float *init_state;
    float *final_state;
    float *log_decay_sum;
    const float *dfinal_state;
    float *dinit_state;
    float *da_partial;
    int64_t weighted_partial_stride;   // weighted backward: floats between the partial sums of decay, in_weight, out_weight
    int64_t b, L, h, d;
    int64_t x_sb, x_sl, x_sh;
    int64_t o_sb, o_sl, o_sh;
    int64_t g_sb, g_sl, g_sh;
    int64_t a_sb, a_sl, a_sh;
    int decay_mode, convention, chunk;
    int n_tiles, n_dtiles;
    int64_t n_chunks;
    float stop_below;
    // scratch for carries handed between CTAs of the tensor-core kernels (optional; see tc_sync_bytes)
    void *sync_ws;
    size_t sync_ws_bytes;
    // bounds-checking build: the table of this call's buffers (null in the normal build)
    BoundsTable *bounds;
};

// ---- raw vector types: VEC elements of T moved by one load/store instruction ----------------
template <int BYTES> struct RawT;
template <> struct RawT<16> { using type = uint4; };
template <> struct RawT<8> { using type = uint2; };
template <> struct RawT<4> { using type = uint32_t; };
template <> struct RawT<2> { using type = unsigned short; };

template <typename T, int VEC> using raw_t = typename RawT<sizeof(T) * VEC>::type;

template <typename T, int VEC>
__device__ __forceinline__ raw_t<T, VEC> raw_zero() {
    raw_t<T, VEC> r;
    if constexpr (sizeof(T) * VEC == 16) r = make_uint4(0u, 0u, 0u, 0u);
    else if constexpr (sizeof(T) * VEC == 8) r = make_uint2(0u, 0u);
    else r = 0;
    return r;
}

// streaming (evict-first) load/store: every big tensor is touched exactly once per pass
template <typename T, int VEC>
__device__ __forceinline__ raw_t<T, VEC> ld_stream(const T *p) {
    return __ldcs(reinterpret_cast<const raw_t<T, VEC> *>(p));
}
template <typename T, int VEC>
__device__ __forceinline__ void st_stream(T *p, const raw_t<T, VEC> &r) {
    __stcs(reinterpret_cast<raw_t<T, VEC> *>(p), r);
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

template <typename T, int VEC>
__device__ __forceinline__ void unpack(const raw_t<T, VEC> &r, float (&f)[VEC]) {
    if constexpr (sizeof(T) == 4) {
        if constexpr (VEC == 4) {
            f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y);
            f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
        } else {
            static_assert(VEC == 1, "fp32 vectors are 1 or 4 wide");
            f[0] = __uint_as_float(r);
        }
    } else {
        if constexpr (VEC == 8) {
            f[0] = bf16lo(r.x); f[1] = bf16hi(r.x); f[2] = bf16lo(r.y); f[3] = bf16hi(r.y);
            f[4] = bf16lo(r.z); f[5] = bf16hi(r.z); f[6] = bf16lo(r.w); f[7] = bf16hi(r.w);
        } else if constexpr (VEC == 4) {
            f[0] = bf16lo(r.x); f[1] = bf16hi(r.x); f[2] = bf16lo(r.y); f[3] = bf16hi(r.y);
        } else {
            static_assert(VEC == 1, "bf16 vectors are 1, 4 or 8 wide");
            f[0] = __uint_as_float(static_cast<uint32_t>(r) << 16);
        }
    }
}

template <typename T, int VEC>
__device__ __forceinline__ raw_t<T, VEC> pack(const float (&f)[VEC]) {
    raw_t<T, VEC> r;
    if constexpr (sizeof(T) == 4) {
        if constexpr (VEC == 4) {
            r = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                           __float_as_uint(f[3]));
        } else {
            r = __float_as_uint(f[0]);
        }
    } else {
        if constexpr (VEC == 8) {
            r = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                           pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        } else if constexpr (VEC == 4) {
            r = make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
        } else {
            __nv_bfloat16 v = __float2bfloat16_rn(f[0]);
            r = *reinterpret_cast<unsigned short *>(&v);
        }
    }
    return r;
}

// scalar element access for the stage kernels
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// decay value -> multiplicative decay a, for either convention; steps past L use a = 1
__device__ __forceinline__ float decay_to_a(float v, int convention) {
    return convention == EMA_CONV_PRESCALED_LOG ? __expf(v) : v;
}

// ---- programmatic dependent launch ----------------------------------------------------------
// The scan, aggregate and reduction kernels are launched so that a kernel may be scheduled while the kernel before it
// on the stream is still running (launch_overlapped below).  Such a kernel does its own set-up - barriers, tensor
// memory, zero-filled shared memory - and then calls grid_dependency_wait() before it touches global memory: the wait
// returns once the preceding kernel has finished and its writes are visible.  grid_dependents_launch() tells the
// scheduler that the kernel after this one may be brought in as soon as SMs are free.  Launched the ordinary way both
// calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- host side ------------------------------------------------------------------------------
void set_last_cuda_error(cudaError_t e);
bool overlapped_launches();   // EMA_B200_PDL=0 turns the overlap off (ema_api.cu)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = overlapped_launches() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
inline int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return EMA_ERR_CUDA;
    }
    return EMA_OK;
}

// geometry of the FMA kernels: 256 threads = NS sub-blocks x CT channel threads
constexpr int kFmaThreads = 256;
constexpr int kFmaCT = 16;
constexpr int kFmaSB = 8;
constexpr int kFmaNS = kFmaThreads / kFmaCT;
constexpr int kFmaTile = kFmaNS * kFmaSB;  // 128 time steps per tile, like the tensor-core path

// per-head decay gradient workspace: [rows * kHeadRowSplit doubles of partial row sums][arrival counter, 3 floats of
// padding][partials]: float index of the counter, and of the first partial (16-byte aligned).  The backward scan
// kernels clear the counter (one thread, at their start), so that the caller's workspace needs no preparation.
constexpr int kHeadRowSplit = 8;
__host__ __device__ inline int64_t kHeadCounterIndex(int64_t rows) { return rows * 2 * kHeadRowSplit; }
__host__ __device__ inline int64_t kHeadPartialOffset(int64_t rows) { return kHeadCounterIndex(rows) + 4; }

int launch_fused_fwd_fma(const FusedParams &p, int dtype, int vec, cudaStream_t stream);
int launch_fused_bwd_fma(const FusedParams &p, int dtype, int vec, cudaStream_t stream);
int launch_fused_bwd_fma_weighted(const FusedParams &p, int dtype, int vec, cudaStream_t stream);
int launch_da_reduce(const FusedParams &p, float *ddecay, int tile_steps, cudaStream_t stream);

// tensor-core path (bf16): eligibility of one [b,L,h,d] tensor for TMA, launches, device status word
bool tc_tensor_ok(const void *base, int64_t d, int64_t sb, int64_t sl, int64_t sh, int64_t b, int64_t L, int64_t h);
int launch_fused_fwd_tc(const FusedParams &p, cudaStream_t stream);
int launch_fused_bwd_tc(const FusedParams &p, cudaStream_t stream);
// fp32 forward on the CUDA cores with x brought in by TMA; p.n_dtiles must count 64-channel tiles (vec 4)
int launch_fused_fwd_fma_tma(const FusedParams &p, cudaStream_t stream);
int launch_fused_bwd_fma_tma(const FusedParams &p, cudaStream_t stream);
int read_tc_status(int clear);
int launch_selftest_wait(int mode, unsigned polls, const unsigned *scratch, cudaStream_t stream);
// bytes of scratch that let the tensor-core kernels cut work items across CTAs: carries handed between thread
// blocks, plus per-tile aggregates for problems with few work items (rows = b * h scan rows)
size_t tc_sync_bytes(int64_t rows, int64_t L, int64_t d);
bool tc_wants_aggregates(int64_t rows, int64_t L, int64_t d);
int tc_set_split(int on);   // returns the previous setting
int tc_last_schedule();     // schedule of this thread's last tensor-core launch: 0 whole items, 1 carries, 2 aggregates
// per-tile aggregates (ema_tile_agg.cu): one buffer's size, and the pass that fills it from x (adjoint = 0) or dy
size_t tile_aggregate_bytes(int64_t rows, int64_t L, int64_t d);
int launch_tile_aggregates(const FusedParams &fp, int adjoint, float *buf, cudaStream_t stream);

}  // namespace ema
