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
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * L) return;
    const int64_t row = idx / L, t = idx % L;
    const float *src = part + row * n_dtiles * L_pad + t;
    float s = 0.f;
    for (int j = 0; j < n_dtiles; ++j) s += *EMA_AT(br, src + static_cast<int64_t>(j) * L_pad, 220);
    *EMA_AT(br, ddecay + (row / h) * a_sb + t * a_sl + (row % h) * a_sh, 221) = s;
}

// per-head decay, level 1: one CTA per scan row sums that row's partials (channel tiles x time
// tiles x warps) in a fixed order
__global__ void da_reduce_rows_kernel(const float *__restrict__ part, double *__restrict__ row_sum,
                                      int64_t per_row, BoundsRef br) {
    __shared__ double red[256];
    const float *src = part + static_cast<int64_t>(blockIdx.x) * per_row;
    double s = 0.0;
    for (int64_t i = threadIdx.x; i < per_row; i += blockDim.x) s += static_cast<double>(*EMA_AT(br, src + i, 222));
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *EMA_AT(br, row_sum + blockIdx.x, 223) = red[0];
}

// level 2: ddecay[h] = sum over the batch of the row sums
__global__ void da_reduce_head_kernel(const double *__restrict__ row_sum, float *__restrict__ ddecay,
                                      int64_t b, int64_t h, int64_t a_sh, BoundsRef br) {
    const int64_t hi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (hi >= h) return;
    double s = 0.0;
    for (int64_t bi = 0; bi < b; ++bi) s += *EMA_AT(br, row_sum + bi * h + hi, 224);
    *EMA_AT(br, ddecay + hi * a_sh, 225) = static_cast<float>(s);
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
        da_reduce_steps_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
            p.da_partial, ddecay, rows, p.h, p.L, L_pad, p.n_dtiles, p.a_sb, p.a_sl, p.a_sh, BoundsRef{p.bounds});
    } else {
        const int64_t per_row = static_cast<int64_t>(p.n_dtiles) * p.n_tiles * (kFmaThreads / 32);
        double *row_sum = reinterpret_cast<double *>(p.da_partial);
        da_reduce_rows_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
            p.da_partial + kHeadPartialOffset(rows), row_sum, per_row, BoundsRef{p.bounds});
        da_reduce_head_kernel<<<static_cast<unsigned>((p.h + 127) / 128), 128, 0, stream>>>(
            row_sum, ddecay, p.b, p.h, p.a_sh, BoundsRef{p.bounds});
    }
    return check_launch();
}

}  // namespace ema
