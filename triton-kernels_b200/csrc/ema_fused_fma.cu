// Fused EMA scan on the CUDA cores: one pass over HBM per direction, fp32 state.
//
// This is the exact path: fp32 inputs (which must meet a 1e-4 absolute tolerance, out of reach of
// a bf16/tf32 tensor-core contraction) and every shape or alignment the tensor-core path does not
// take.  A CTA owns one scan row (b,h) and DT = 16*VEC channels and walks the sequence in tiles of
// 128 steps.  Inside a tile the 256 threads form 16 sub-blocks of 8 steps x 16 channel threads:
//   phase 1  every sub-block scans its 8 steps from a zero state (local state S, decay product P)
//   carry    state entering sub-block j = fold of (P_i, S_i), i < j, onto the state entering the tile
//   phase 2  every sub-block re-runs its 8 steps from its true entering state and writes the result
// so the sequential dependence costs one __syncthreads per tile.  x is held in registers between
// the phases and the next tile is already in flight (register prefetch) while this one computes.
#include "ema_common.cuh"
#include "ema_fwd_fma_kernel.cuh"
#include "ema_bwd_fma_kernel.cuh"

namespace ema {

namespace {

// ------------------------------------------------------------------------------------------------
// forward (body in ema_fwd_fma_kernel.cuh)
// ------------------------------------------------------------------------------------------------
template <typename T, int VEC, bool WEIGHTED>
__global__ void __launch_bounds__(kFmaThreads) ema_fwd_fma_kernel(const FusedParams p) {
    RegisterFeed<T, VEC> feed;
    ema_fwd_fma_body<T, VEC, WEIGHTED>(p, feed);
}

// ------------------------------------------------------------------------------------------------
// backward (body in ema_bwd_fma_kernel.cuh)
// ------------------------------------------------------------------------------------------------
template <typename T, int VEC, bool PREFETCH>
__global__ void __launch_bounds__(kFmaThreads) ema_bwd_fma_kernel(const FusedParams p) {
    RegisterFeedBwd<T, VEC, PREFETCH> feed;
    ema_bwd_fma_body<T, VEC>(p, feed);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kFmaThreads) ema_bwd_fma_weighted_kernel(const FusedParams p) {
    RegisterFeedBwd<T, VEC, false> feed;
    ema_bwd_fma_body<T, VEC, RegisterFeedBwd<T, VEC, false>, true>(p, feed);
}

// ------------------------------------------------------------------------------------------------
// decay-gradient reductions (fixed order, no atomics)
// ------------------------------------------------------------------------------------------------
struct BoundsRef {   // what EMA_AT needs from a parameter block
    BoundsTable *bounds;
};
// per-step decay: ddecay[b,t,h] = sum over channel tiles of da_partial[row][dtile][t]
__global__ void da_reduce_steps_kernel(const float *__restrict__ part, float *__restrict__ ddecay,
                                       int64_t rows, int64_t h, int64_t L, int64_t L_pad,
                                       int n_dtiles, int64_t a_sb, int64_t a_sl, int64_t a_sh, BoundsRef br) {
    grid_dependents_launch();   // (see ema_common.cuh)
    grid_dependency_wait();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * L) return;
    const int64_t row = idx / L, t = idx % L;
    const float *src = part + row * n_dtiles * L_pad + t;
    float s = 0.f;
    for (int j = 0; j < n_dtiles; ++j) s += *EMA_AT(br, src + static_cast<int64_t>(j) * L_pad, 220);
    *EMA_AT(br, ddecay + (row / h) * a_sb + t * a_sl + (row % h) * a_sh, 221) = s;
}

// Per-head decay, one launch.  Thread block (row, s) sums the s-th of `split` equal parts of that scan row's partials
// (channel tiles x time tiles x warps) in a fixed order and leaves the sum in sub_sum[row * split + s]; the block that
// arrives last (a counter the backward scan kernel cleared) then adds the sub-sums of every head over the batch, again
// in a fixed order, so that the result does not depend on which block that was.
__global__ void da_reduce_head_kernel(const float *__restrict__ part, double *sub_sum, unsigned *counter,
                                      float *__restrict__ ddecay, int64_t per_row, int split, int64_t b, int64_t h,
                                      int64_t a_sh, BoundsRef br) {
    __shared__ double red[256];
    __shared__ bool last;
    grid_dependents_launch();   // (see ema_common.cuh)
    grid_dependency_wait();
    const int64_t row = blockIdx.x / split;
    const int s = static_cast<int>(blockIdx.x % split);
    const int64_t part_len = (per_row + split - 1) / split;
    const int64_t i0 = s * part_len, i1 = i0 + part_len < per_row ? i0 + part_len : per_row;
    const float *src = part + row * per_row;
    double acc = 0.0;
    for (int64_t i = i0 + threadIdx.x; i < i1; i += blockDim.x) acc += static_cast<double>(*EMA_AT(br, src + i, 222));
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *EMA_AT(br, sub_sum + blockIdx.x, 223) = red[0];
        __threadfence();   // the sub-sum is visible before the arrival is
        last = atomicAdd(EMA_AT(br, counter, 226), 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    const int64_t per_head = b * split;   // sub-sums per head
    if (h >= 64) {
        // many heads: a thread per head, its sub-sums in order (the threads' loads overlap one another)
        for (int64_t hi = threadIdx.x; hi < h; hi += blockDim.x) {
            double sum = 0.0;
            for (int64_t i = 0; i < per_head; ++i)
                sum += __ldcg(EMA_AT(br, sub_sum + ((i / split) * h + hi) * split + i % split, 224));
            *EMA_AT(br, ddecay + hi * a_sh, 225) = static_cast<float>(sum);
        }
        return;
    }
    // few heads: the whole block on one head at a time - thread t takes the sub-sums t, t + 256, ... in order, then the
    // same tree as above; a single thread walking the list would pay an L2 round trip per element
    for (int64_t hi = 0; hi < h; ++hi) {
        double sum = 0.0;
        for (int64_t i = threadIdx.x; i < per_head; i += blockDim.x)
            sum += __ldcg(EMA_AT(br, sub_sum + ((i / split) * h + hi) * split + i % split, 227));
        __syncthreads();   // the previous head's tree has been read
        red[threadIdx.x] = sum;
        __syncthreads();
        for (int o = 128; o > 0; o >>= 1) {
            if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
            __syncthreads();
        }
        if (threadIdx.x == 0) *EMA_AT(br, ddecay + hi * a_sh, 228) = static_cast<float>(red[0]);
    }
}

template <typename T, int VEC>
int launch_fwd(const FusedParams &p, cudaStream_t stream) {
    const int64_t blocks = p.b * p.h * p.n_dtiles;
    if (p.in_weight || p.out_weight)
        ema_fwd_fma_kernel<T, VEC, true><<<static_cast<unsigned>(blocks), kFmaThreads, 0, stream>>>(p);
    else
        ema_fwd_fma_kernel<T, VEC, false><<<static_cast<unsigned>(blocks), kFmaThreads, 0, stream>>>(p);
    return check_launch();
}
template <typename T, int VEC, bool PF>
int launch_bwd(const FusedParams &p, cudaStream_t stream) {
    const int64_t blocks = p.b * p.h * p.n_dtiles;
    ema_bwd_fma_kernel<T, VEC, PF><<<static_cast<unsigned>(blocks), kFmaThreads, 0, stream>>>(p);
    return check_launch();
}

}  // namespace

int launch_fused_fwd_fma(const FusedParams &p, int dtype, int vec, cudaStream_t stream) {
    if (dtype == EMA_F32) return vec == 4 ? launch_fwd<float, 4>(p, stream) : launch_fwd<float, 1>(p, stream);
    return vec == 4 ? launch_fwd<__nv_bfloat16, 4>(p, stream) : launch_fwd<__nv_bfloat16, 1>(p, stream);
}

int launch_fused_bwd_fma(const FusedParams &p, int dtype, int vec, cudaStream_t stream) {
    if (dtype == EMA_F32)
        return vec == 4 ? launch_bwd<float, 4, false>(p, stream) : launch_bwd<float, 1, true>(p, stream);
    return vec == 4 ? launch_bwd<__nv_bfloat16, 4, true>(p, stream)
                    : launch_bwd<__nv_bfloat16, 1, true>(p, stream);
}

int launch_fused_bwd_fma_weighted(const FusedParams &p, int dtype, int vec, cudaStream_t stream) {
    const unsigned blocks = static_cast<unsigned>(p.b * p.h * p.n_dtiles);
    if (dtype == EMA_F32) {
        if (vec == 4) ema_bwd_fma_weighted_kernel<float, 4><<<blocks, kFmaThreads, 0, stream>>>(p);
        else ema_bwd_fma_weighted_kernel<float, 1><<<blocks, kFmaThreads, 0, stream>>>(p);
    } else {
        if (vec == 4) ema_bwd_fma_weighted_kernel<__nv_bfloat16, 4><<<blocks, kFmaThreads, 0, stream>>>(p);
        else ema_bwd_fma_weighted_kernel<__nv_bfloat16, 1><<<blocks, kFmaThreads, 0, stream>>>(p);
    }
    return check_launch();
}

int launch_da_reduce(const FusedParams &p, float *ddecay, int tile_steps, cudaStream_t stream) {
    const int64_t rows = p.b * p.h;
    if (p.decay_mode == EMA_DECAY_PER_STEP) {
        const int64_t n = rows * p.L;
        const int64_t L_pad = static_cast<int64_t>(p.n_tiles) * tile_steps;
        if ((n + 255) / 256 >= (1ll << 31)) return EMA_ERR_UNSUPPORTED;   // beyond one grid dimension
        const cudaError_t e = launch_overlapped(da_reduce_steps_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
                                                stream, p.da_partial, ddecay, rows, p.h, p.L, L_pad, p.n_dtiles, p.a_sb, p.a_sl,
                                                p.a_sh, BoundsRef{p.bounds});
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    } else {
        const int64_t per_row = static_cast<int64_t>(p.n_dtiles) * p.n_tiles * (kFmaThreads / 32);
        // enough thread blocks to have the partials' loads in flight at once, at least 2048 floats each
        int64_t split = per_row / 2048;
        split = split < 1 ? 1 : (split > kHeadRowSplit ? kHeadRowSplit : split);
        double *sub_sum = reinterpret_cast<double *>(p.da_partial);
        unsigned *counter = reinterpret_cast<unsigned *>(p.da_partial + kHeadCounterIndex(rows));
        const cudaError_t e = launch_overlapped(da_reduce_head_kernel, dim3(static_cast<unsigned>(rows * split)), dim3(256), 0,
                                                stream, p.da_partial + kHeadPartialOffset(rows), sub_sum, counter, ddecay, per_row,
                                                static_cast<int>(split), p.b, p.h, p.a_sh, BoundsRef{p.bounds});
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    }
    return check_launch();
}

}  // namespace ema
