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

namespace ema {

namespace {

constexpr unsigned kFull = 0xffffffffu;

// ------------------------------------------------------------------------------------------------
// forward (body in ema_fwd_fma_kernel.cuh)
// ------------------------------------------------------------------------------------------------
template <typename T, int VEC, bool WEIGHTED>
__global__ void __launch_bounds__(kFmaThreads) ema_fwd_fma_kernel(const FusedParams p) {
    RegisterFeed<T, VEC> feed;
    ema_fwd_fma_body<T, VEC, WEIGHTED>(p, feed);
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
// Sum acc[0..7] over the 16 lanes that share a sub-block; afterwards lane lc (even) holds the total
// for step lc/2.  Halving exchange: 8 shuffles instead of 32.
__device__ __forceinline__ float reduce8_over16(const float (&acc)[8], int lc) {
    float v4[4], v2[2];
    const bool b3 = lc & 8, b2 = lc & 4, b1 = lc & 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = b3 ? acc[i] : acc[i + 4];
        const float keep = b3 ? acc[i + 4] : acc[i];
        v4[i] = keep + __shfl_xor_sync(kFull, send, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = b2 ? v4[i] : v4[i + 2];
        const float keep = b2 ? v4[i + 2] : v4[i];
        v2[i] = keep + __shfl_xor_sync(kFull, send, 4);
    }
    const float send = b1 ? v2[0] : v2[1];
    const float keep = b1 ? v2[1] : v2[0];
    float v1 = keep + __shfl_xor_sync(kFull, send, 2);
    v1 += __shfl_xor_sync(kFull, v1, 1);
    return v1;
}

template <typename T, int VEC, bool PREFETCH>
__global__ void __launch_bounds__(kFmaThreads) ema_bwd_fma_kernel(const FusedParams p) {
    constexpr int CT = kFmaCT, SB = kFmaSB, NS = kFmaNS, QT = kFmaTile, DT = CT * VEC;
    static_assert(SB == 8 && CT == 16, "reduce8_over16 assumes 8 steps x 16 lanes");
    using R = raw_t<T, VEC>;
    __shared__ float a_sm[2][QT + 1];
    __shared__ float Sf_sm[2][NS][DT];
    __shared__ float Rr_sm[2][NS][DT];
    __shared__ float Pf_sm[2][NS];
    __shared__ float Pr_sm[2][NS];
    __shared__ float g_sm[2][DT];

    const int tid = threadIdx.x, lc = tid % CT, sub = tid / CT;
    const int64_t blk = blockIdx.x;
    const int dtile = static_cast<int>(blk % p.n_dtiles);
    const int64_t row = blk / p.n_dtiles;
    const int64_t bi = row / p.h, hi = row % p.h;
    const int64_t c0 = static_cast<int64_t>(dtile) * DT + lc * VEC;
    const bool c_ok = c0 < p.d;
    const int L = static_cast<int>(p.L);
    const int conv = p.convention;
    const bool per_step = p.decay_mode == EMA_DECAY_PER_STEP;
    const int n_tiles = p.n_tiles;

    const T *xrow = static_cast<const T *>(p.x) + bi * p.x_sb + hi * p.x_sh + c0;
    const T *grow = static_cast<const T *>(p.dy) + bi * p.g_sb + hi * p.g_sh + c0;
    T *orow = static_cast<T *>(p.out) + bi * p.o_sb + hi * p.o_sh + c0;
    const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
    const float a_head = per_step ? 1.f : (conv ? expf(arow[0]) : arow[0]);

    auto load_a = [&](int t) -> float {
        if (t >= L) return 1.f;
        if (!per_step) return a_head;
        const float v = arow[static_cast<int64_t>(t) * p.a_sl];
        return conv ? expf(v) : v;
    };
    auto load_state = [&](int k, float (&hs)[VEC]) {
        const float *ts = p.tile_states + (row * n_tiles + k) * p.d + c0;
#pragma unroll
        for (int v = 0; v < VEC; ++v) hs[v] = c_ok ? ts[v] : 0.f;
    };

    float dfin[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v)
        dfin[v] = (p.dfinal_state && c_ok) ? p.dfinal_state[row * p.d + c0 + v] : 0.f;

    if (sub == 0) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) g_sm[0][lc * VEC + v] = 0.f;
    }
    {
        const int k = n_tiles - 1;
        if (tid <= QT) a_sm[0][tid] = load_a(k * QT + tid);
    }
    R xc[SB], gc[SB], xn[SB], gn[SB];
    float hs[VEC], hs_next[VEC];
    {
        const int k = n_tiles - 1;
#pragma unroll
        for (int s = 0; s < SB; ++s) {
            const int t = k * QT + sub * SB + s;
            const bool ok = c_ok && t < L;
            xc[s] = load_or_zero<T, VEC>(xrow + static_cast<int64_t>(t) * p.x_sl, ok);
            gc[s] = load_or_zero<T, VEC>(grow + static_cast<int64_t>(t) * p.g_sl, ok);
        }
        load_state(k, hs);
    }
    __syncthreads();

    float run = 1.f;
    for (int kk = 0; kk < n_tiles; ++kk) {
        const int k = n_tiles - 1 - kk;
        const int par = kk & 1;
        const int t0 = k * QT + sub * SB;
        const bool more = k > 0;
        float a_pref = 1.f;
        if (more) {
            if (PREFETCH) {
#pragma unroll
                for (int s = 0; s < SB; ++s) {
                    const int t = t0 - QT + s;  // never past L: tile k-1 is a full tile
                    xn[s] = load_or_zero<T, VEC>(xrow + static_cast<int64_t>(t) * p.x_sl, c_ok);
                    gn[s] = load_or_zero<T, VEC>(grow + static_cast<int64_t>(t) * p.g_sl, c_ok);
                }
            }
            if (tid < QT) a_pref = load_a((k - 1) * QT + tid);
            load_state(k - 1, hs_next);
        }

        float a_r[SB + 1];
#pragma unroll
        for (int s = 0; s <= SB; ++s) a_r[s] = a_sm[par][sub * SB + s];
        // the gradient entering the state after step L-1 rides on dy_{L-1}
        const int s_last = (L - 1) - t0;

        // phase 1: local forward scan and local reverse scan, both from zero
        float st[VEC], lam[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { st[v] = 0.f; lam[v] = 0.f; }
        float Pf = 1.f, Pr = 1.f;
#pragma unroll
        for (int s = 0; s < SB; ++s) {
            float xf[VEC];
            unpack<T, VEC>(xc[s], xf);
            const float pw = conv ? 1.f : 1.f - a_r[s];
#pragma unroll
            for (int v = 0; v < VEC; ++v) st[v] = fmaf(a_r[s], st[v], pw * xf[v]);
            Pf *= a_r[s];
        }
#pragma unroll
        for (int s = SB - 1; s >= 0; --s) {
            float gf[VEC];
            unpack<T, VEC>(gc[s], gf);
            if (s == s_last) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) gf[v] += dfin[v];
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) lam[v] = fmaf(a_r[s + 1], lam[v], gf[v]);
            Pr *= a_r[s + 1];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            Sf_sm[par][sub][lc * VEC + v] = st[v];
            Rr_sm[par][sub][lc * VEC + v] = lam[v];
        }
        if (lc == 0) { Pf_sm[par][sub] = Pf; Pr_sm[par][sub] = Pr; }
        if (more) {
            if (tid < QT) a_sm[par ^ 1][tid] = a_pref;
            if (tid == QT) a_sm[par ^ 1][QT] = a_sm[par][0];  // a of the first step of this tile
        }
        __syncthreads();

        // carries: forward state entering the sub-block, adjoint entering it from the right
        float h[VEC], g[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) { h[v] = hs[v]; g[v] = g_sm[par][lc * VEC + v]; }
        for (int i = 0; i < sub; ++i) {
            const float Pi = Pf_sm[par][i];
#pragma unroll
            for (int v = 0; v < VEC; ++v) h[v] = fmaf(Pi, h[v], Sf_sm[par][i][lc * VEC + v]);
        }
        for (int i = NS - 1; i > sub; --i) {
            const float Pi = Pr_sm[par][i];
#pragma unroll
            for (int v = 0; v < VEC; ++v) g[v] = fmaf(Pi, g[v], Rr_sm[par][i][lc * VEC + v]);
        }

        // phase 2: y_{t-1} for every step of the sub-block, then the adjoint right to left
        float yprev[SB][VEC];
#pragma unroll
        for (int s = 0; s < SB; ++s) {
            float xf[VEC];
            unpack<T, VEC>(xc[s], xf);
            const float pw = conv ? 1.f : 1.f - a_r[s];
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                yprev[s][v] = h[v];
                h[v] = fmaf(a_r[s], h[v], pw * xf[v]);
            }
        }
        float acc[SB];
#pragma unroll
        for (int s = SB - 1; s >= 0; --s) {
            float gf[VEC], xf[VEC], dxf[VEC];
            unpack<T, VEC>(gc[s], gf);
            unpack<T, VEC>(xc[s], xf);
            if (s == s_last) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) gf[v] += dfin[v];
            }
            const float pw = conv ? 1.f : 1.f - a_r[s];
            float a_acc = 0.f;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                g[v] = fmaf(a_r[s + 1], g[v], gf[v]);  // lambda_t
                dxf[v] = pw * g[v];
                a_acc = conv ? fmaf(g[v], yprev[s][v], a_acc)
                             : fmaf(g[v], yprev[s][v] - xf[v], a_acc);
            }
            const int t = t0 + s;
            acc[s] = (t < L) ? (conv ? a_r[s] * a_acc : a_acc) : 0.f;
            if (c_ok && t < L)
                st_stream<T, VEC>(orow + static_cast<int64_t>(t) * p.o_sl, pack<T, VEC>(dxf));
        }
        if (sub == 0) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) g_sm[par ^ 1][lc * VEC + v] = g[v];
            if (k == 0 && p.dinit_state && c_ok) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) p.dinit_state[row * p.d + c0 + v] = a_r[0] * g[v];
            }
        }

        // decay gradient: partial over this CTA's channels
        if (per_step) {
            const float tot = reduce8_over16(acc, lc);
            if ((lc & 1) == 0)
                p.da_partial[blk * (static_cast<int64_t>(n_tiles) * QT) + t0 + (lc >> 1)] = tot;
        } else {
            float tot = 0.f;
#pragma unroll
            for (int s = 0; s < SB; ++s) tot += acc[s];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(kFull, tot, o);
            if ((tid & 31) == 0)
                p.da_partial[kHeadPartialOffset(p.b * p.h) + (blk * n_tiles + k) * (kFmaThreads / 32) + (tid >> 5)] = tot;
        }

        if (p.stop_below > 0.f) {
            float tp = 1.f;
#pragma unroll
            for (int i = 0; i < NS; ++i) tp *= Pr_sm[par][i];
            run *= tp;
            if (run < p.stop_below) break;
        }
        if (more) {
            if (PREFETCH) {
#pragma unroll
                for (int s = 0; s < SB; ++s) { xc[s] = xn[s]; gc[s] = gn[s]; }
            } else {
#pragma unroll
                for (int s = 0; s < SB; ++s) {
                    const int t = t0 - QT + s;
                    xc[s] = load_or_zero<T, VEC>(xrow + static_cast<int64_t>(t) * p.x_sl, c_ok);
                    gc[s] = load_or_zero<T, VEC>(grow + static_cast<int64_t>(t) * p.g_sl, c_ok);
                }
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) hs[v] = hs_next[v];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// decay-gradient reductions (fixed order, no atomics)
// ------------------------------------------------------------------------------------------------
// per-step decay: ddecay[b,t,h] = sum over channel tiles of da_partial[row][dtile][t]
__global__ void da_reduce_steps_kernel(const float *__restrict__ part, float *__restrict__ ddecay,
                                       int64_t rows, int64_t h, int64_t L, int64_t L_pad,
                                       int n_dtiles, int64_t a_sb, int64_t a_sl, int64_t a_sh) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * L) return;
    const int64_t row = idx / L, t = idx % L;
    const float *src = part + row * n_dtiles * L_pad + t;
    float s = 0.f;
    for (int j = 0; j < n_dtiles; ++j) s += src[static_cast<int64_t>(j) * L_pad];
    ddecay[(row / h) * a_sb + t * a_sl + (row % h) * a_sh] = s;
}

// per-head decay, level 1: one CTA per scan row sums that row's partials (channel tiles x time
// tiles x warps) in a fixed order
__global__ void da_reduce_rows_kernel(const float *__restrict__ part, double *__restrict__ row_sum,
                                      int64_t per_row) {
    __shared__ double red[256];
    const float *src = part + static_cast<int64_t>(blockIdx.x) * per_row;
    double s = 0.0;
    for (int64_t i = threadIdx.x; i < per_row; i += blockDim.x) s += static_cast<double>(src[i]);
    red[threadIdx.x] = s;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (static_cast<int>(threadIdx.x) < o) red[threadIdx.x] += red[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) row_sum[blockIdx.x] = red[0];
}

// level 2: ddecay[h] = sum over the batch of the row sums
__global__ void da_reduce_head_kernel(const double *__restrict__ row_sum, float *__restrict__ ddecay,
                                      int64_t b, int64_t h, int64_t a_sh) {
    const int64_t hi = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (hi >= h) return;
    double s = 0.0;
    for (int64_t bi = 0; bi < b; ++bi) s += row_sum[bi * h + hi];
    ddecay[hi * a_sh] = static_cast<float>(s);
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

int launch_da_reduce(const FusedParams &p, float *ddecay, int tile_steps, cudaStream_t stream) {
    const int64_t rows = p.b * p.h;
    if (p.decay_mode == EMA_DECAY_PER_STEP) {
        const int64_t n = rows * p.L;
        const int64_t L_pad = static_cast<int64_t>(p.n_tiles) * tile_steps;
        da_reduce_steps_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
            p.da_partial, ddecay, rows, p.h, p.L, L_pad, p.n_dtiles, p.a_sb, p.a_sl, p.a_sh);
    } else {
        const int64_t per_row = static_cast<int64_t>(p.n_dtiles) * p.n_tiles * (kFmaThreads / 32);
        double *row_sum = reinterpret_cast<double *>(p.da_partial);
        da_reduce_rows_kernel<<<static_cast<unsigned>(rows), 256, 0, stream>>>(
            p.da_partial + kHeadPartialOffset(rows), row_sum, per_row);
        da_reduce_head_kernel<<<static_cast<unsigned>((p.h + 127) / 128), 128, 0, stream>>>(row_sum, ddecay, p.b,
                                                                                           p.h, p.a_sh);
    }
    return check_launch();
}

}  // namespace ema
