// The backward scan of the CUDA-core family as a function template (see ema_fwd_fma_kernel.cuh): the same arithmetic
// fed either by plain global loads or by a TMA ring in shared memory.
#pragma once

#include "ema_common.cuh"
#include "ema_fwd_fma_kernel.cuh"

namespace ema {

// x and dy tiles through registers.  PREFETCH: tile k - 1 is loaded while tile k computes (twice the registers);
// otherwise it is loaded at the bottom of the iteration.
template <typename T, int VEC, bool PREFETCH>
struct RegisterFeedBwd {
    using R = raw_t<T, VEC>;
    R xc[kFmaSB], gc[kFmaSB], xn[PREFETCH ? kFmaSB : 1], gn[PREFETCH ? kFmaSB : 1];
    const T *xrow, *grow;
    int64_t x_sl, g_sl;
    int sub;
    bool c_ok;
    BoundsTable *bounds;
    // VEC elements at q (bounds-checked in the checking build), or zeros
    __device__ __forceinline__ R fetch(const T *q, bool ok, unsigned site) {
        return ok ? ld_stream<T, VEC>(EMA_ATN(*this, q, site, sizeof(T) * VEC)) : raw_zero<T, VEC>();
    }
    __device__ __forceinline__ void init(const FusedParams &p, const T *xrow_, const T *grow_, bool c_ok_, int sub_, int L,
                                         int n_tiles) {
        xrow = xrow_; grow = grow_; x_sl = p.x_sl; g_sl = p.g_sl; sub = sub_; c_ok = c_ok_; bounds = p.bounds;
#pragma unroll
        for (int s = 0; s < kFmaSB; ++s) {   // the last tile may be ragged
            const int t = (n_tiles - 1) * kFmaTile + sub * kFmaSB + s;
            const bool ok = c_ok && t < L;
            xc[s] = fetch(xrow + static_cast<int64_t>(t) * x_sl, ok, 50);
            gc[s] = fetch(grow + static_cast<int64_t>(t) * g_sl, ok, 51);
        }
    }
    // tile k (never the last one: it is a full tile)
    __device__ __forceinline__ void load(R (&xd)[kFmaSB], R (&gd)[kFmaSB], int k) {
#pragma unroll
        for (int s = 0; s < kFmaSB; ++s) {
            const int t = k * kFmaTile + sub * kFmaSB + s;
            xd[s] = fetch(xrow + static_cast<int64_t>(t) * x_sl, c_ok, 52);
            gd[s] = fetch(grow + static_cast<int64_t>(t) * g_sl, c_ok, 53);
        }
    }
    __device__ __forceinline__ void begin(int, int k, bool more) {
        if constexpr (PREFETCH) {
            if (more) load(xn, gn, k - 1);
        }
    }
    __device__ __forceinline__ void after_barrier(int) {}
    __device__ __forceinline__ void end(int k, bool more) {
        if (!more) return;
        if constexpr (PREFETCH) {
#pragma unroll
            for (int s = 0; s < kFmaSB; ++s) { xc[s] = xn[s]; gc[s] = gn[s]; }
        } else {
            load(xc, gc, k - 1);
        }
    }
    __device__ __forceinline__ void finish() {}
};

// Sum acc[0..7] over the 16 lanes that share a sub-block; afterwards lane lc (even) holds the total
// for step lc/2.  Halving exchange: 8 shuffles instead of 32.
__device__ __forceinline__ float reduce8_over16(const float (&acc)[8], int lc) {
    float v4[4], v2[2];
    const bool b3 = lc & 8, b2 = lc & 4, b1 = lc & 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = b3 ? acc[i] : acc[i + 4];
        const float keep = b3 ? acc[i + 4] : acc[i];
        v4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = b2 ? v4[i] : v4[i + 2];
        const float keep = b2 ? v4[i + 2] : v4[i];
        v2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    const float send = b1 ? v2[0] : v2[1];
    const float keep = b1 ? v2[1] : v2[0];
    float v1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
    v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
    return v1;
}

// FEED supplies the x and dy tiles, walked from the last tile to the first: `xc[s]`, `gc[s]` hold this thread's VEC
// channels of step s of its sub-block.
//   init(...)          before the first (= last in time) tile, ends before the block-wide barrier of the prologue
//   begin(kk, k, more) top of iteration kk (tile k): make xc/gc valid / start fetching tile k - 1
//   after_barrier(kk)  after the tile's block-wide barrier: every thread has consumed the tile's staging, if any
//   end(k, more)       bottom of the iteration
//   finish()           after the loop
//
// WEIGHTED (per-step decay only): the forward was  s_t = a_t s_{t-1} + w_t x_t,  y_t = c_t s_t  with per-step weights
// w = in_weight (or the convention's 1 - a | 1 when null) and c = out_weight (or 1).  Then
//     lambda_t = c_t dy_t + a_{t+1} lambda_{t+1},   dx_t = w_t lambda_t,
//     d decay_t = sum_d lambda_t s_{t-1}  (times a_t for a log decay; minus sum_d lambda_t x_t when w is the convention's 1 - a),
//     d in_weight_t = sum_d lambda_t x_t,   d out_weight_t = sum_d dy_t s_t,
// all in the one pass: three partial sums per step instead of one (partial regions p.weighted_partial_stride apart).
template <typename T, int VEC, typename FEED, bool WEIGHTED = false>
__device__ __forceinline__ void ema_bwd_fma_body(const FusedParams &p, FEED &feed) {
    constexpr int CT = kFmaCT, SB = kFmaSB, NS = kFmaNS, QT = kFmaTile, DT = CT * VEC;
    static_assert(SB == 8 && CT == 16, "reduce8_over16 assumes 8 steps x 16 lanes");
    using R = raw_t<T, VEC>;
    constexpr int WQ = WEIGHTED ? QT : 1;   // the weight tables exist only in the weighted kernel
    __shared__ float a_sm[2][QT + 1];
    __shared__ float w_sm[2][WQ];   // input weights of the tile
    __shared__ float c_sm[2][WQ];   // output weights of the tile
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

    // arrival counter of the per-head reduction that follows this kernel (see kHeadCounterIndex)
    if (!per_step && blk == 0 && tid == 0)
        *reinterpret_cast<unsigned *>(EMA_AT(p, p.da_partial + kHeadCounterIndex(p.b * p.h), 67)) = 0u;

    const T *xrow = static_cast<const T *>(p.x) + bi * p.x_sb + hi * p.x_sh + c0;
    const T *grow = static_cast<const T *>(p.dy) + bi * p.g_sb + hi * p.g_sh + c0;
    T *orow = static_cast<T *>(p.out) + bi * p.o_sb + hi * p.o_sh + c0;
    const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
    const float a_head_raw = per_step ? 0.f : *EMA_AT(p, arow, 54);
    const float a_head = per_step ? 1.f : (conv ? expf(a_head_raw) : a_head_raw);

    auto load_a = [&](int t) -> float {
        if (t >= L) return 1.f;
        if (!per_step) return a_head;
        const float v = *EMA_AT(p, arow + static_cast<int64_t>(t) * p.a_sl, 55);
        return conv ? expf(v) : v;
    };
    // per-step weights share the decay's strides; a missing output weight is 1, a missing input weight the convention's
    const int64_t w_off = bi * p.a_sb + hi * p.a_sh;
    const bool explicit_w = WEIGHTED && p.in_weight != nullptr;
    auto load_in_w = [&](int t) -> float {
        if (t >= L) return 0.f;
        if (p.in_weight) return *EMA_AT(p, p.in_weight + w_off + static_cast<int64_t>(t) * p.a_sl, 56);
        return conv ? 1.f : 1.f - *EMA_AT(p, arow + static_cast<int64_t>(t) * p.a_sl, 57);
    };
    auto load_out_w = [&](int t) -> float {
        if (!p.out_weight) return 1.f;
        return t < L ? *EMA_AT(p, p.out_weight + w_off + static_cast<int64_t>(t) * p.a_sl, 58) : 0.f;
    };
    auto load_state = [&](int k, float (&hs)[VEC]) {
        const float *ts = p.tile_states + (row * n_tiles + k) * p.d + c0;
#pragma unroll
        for (int v = 0; v < VEC; ++v) hs[v] = c_ok ? *EMA_AT(p, ts + v, 59) : 0.f;
    };

    float dfin[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v)
        dfin[v] = (p.dfinal_state && c_ok) ? *EMA_AT(p, p.dfinal_state + row * p.d + c0 + v, 60) : 0.f;

    if (sub == 0) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) g_sm[0][lc * VEC + v] = 0.f;
    }
    {
        const int k = n_tiles - 1;
        if (tid <= QT) a_sm[0][tid] = load_a(k * QT + tid);
        if constexpr (WEIGHTED) {
            if (tid < QT) { w_sm[0][tid] = load_in_w(k * QT + tid); c_sm[0][tid] = load_out_w(k * QT + tid); }
        }
    }
    feed.init(p, xrow, grow, c_ok, sub, L, n_tiles);
    R (&xc)[SB] = feed.xc;
    R (&gc)[SB] = feed.gc;
    float hs[VEC], hs_next[VEC];
    load_state(n_tiles - 1, hs);
    __syncthreads();

    float run = 1.f;
    for (int kk = 0; kk < n_tiles; ++kk) {
        const int k = n_tiles - 1 - kk;
        const int par = kk & 1;
        const int t0 = k * QT + sub * SB;
        const bool more = k > 0;
        float a_pref = 1.f, w_pref = 0.f, c_pref = 0.f;
        feed.begin(kk, k, more);
        if (more) {
            if (tid < QT) a_pref = load_a((k - 1) * QT + tid);
            if constexpr (WEIGHTED) {
                if (tid < QT) { w_pref = load_in_w((k - 1) * QT + tid); c_pref = load_out_w((k - 1) * QT + tid); }
            }
            load_state(k - 1, hs_next);
        }

        float a_r[SB + 1];
#pragma unroll
        for (int s = 0; s <= SB; ++s) a_r[s] = a_sm[par][sub * SB + s];
        // the tile's weights go to registers before the barrier: the table of the other parity is rewritten after it
        float w_r[WEIGHTED ? SB : 1], c_r[WEIGHTED ? SB : 1];
        if constexpr (WEIGHTED) {
#pragma unroll
            for (int s = 0; s < SB; ++s) { w_r[s] = w_sm[par][sub * SB + s]; c_r[s] = c_sm[par][sub * SB + s]; }
        }
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
            const float pw = WEIGHTED ? w_r[s] : (conv ? 1.f : 1.f - a_r[s]);
#pragma unroll
            for (int v = 0; v < VEC; ++v) st[v] = fmaf(a_r[s], st[v], pw * xf[v]);
            Pf *= a_r[s];
        }
#pragma unroll
        for (int s = SB - 1; s >= 0; --s) {
            float gf[VEC];
            unpack<T, VEC>(gc[s], gf);
            if constexpr (WEIGHTED) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) gf[v] *= c_r[s];
            }
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
            if constexpr (WEIGHTED) {
                if (tid < QT) { w_sm[par ^ 1][tid] = w_pref; c_sm[par ^ 1][tid] = c_pref; }
            }
        }
        __syncthreads();
        feed.after_barrier(kk);

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
            const float pw = WEIGHTED ? w_r[s] : (conv ? 1.f : 1.f - a_r[s]);
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                yprev[s][v] = h[v];
                h[v] = fmaf(a_r[s], h[v], pw * xf[v]);
            }
        }
        float acc[SB];
        float acc_w[WEIGHTED ? SB : 1], acc_c[WEIGHTED ? SB : 1];
#pragma unroll
        for (int s = SB - 1; s >= 0; --s) {
            float gf[VEC], xf[VEC], dxf[VEC];
            unpack<T, VEC>(gc[s], gf);
            unpack<T, VEC>(xc[s], xf);
            const float pw = WEIGHTED ? w_r[s] : (conv ? 1.f : 1.f - a_r[s]);
            float c_acc = 0.f, w_acc = 0.f;
            if constexpr (WEIGHTED) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    c_acc = fmaf(gf[v], fmaf(a_r[s], yprev[s][v], pw * xf[v]), c_acc);   // dy_t . s_t
                    gf[v] *= c_r[s];
                }
            }
            if (s == s_last) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) gf[v] += dfin[v];
            }
            float a_acc = 0.f;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                g[v] = fmaf(a_r[s + 1], g[v], gf[v]);  // lambda_t
                dxf[v] = pw * g[v];
                a_acc = (conv || explicit_w) ? fmaf(g[v], yprev[s][v], a_acc)
                                             : fmaf(g[v], yprev[s][v] - xf[v], a_acc);
                if constexpr (WEIGHTED) w_acc = fmaf(g[v], xf[v], w_acc);
            }
            const int t = t0 + s;
            acc[s] = (t < L) ? (conv ? a_r[s] * a_acc : a_acc) : 0.f;
            if constexpr (WEIGHTED) {
                acc_w[s] = (t < L) ? w_acc : 0.f;
                acc_c[s] = (t < L) ? c_acc : 0.f;
            }
            if (c_ok && t < L)
                st_stream<T, VEC>(EMA_ATN(p, orow + static_cast<int64_t>(t) * p.o_sl, 61, sizeof(T) * VEC),
                                  pack<T, VEC>(dxf));
        }
        if (sub == 0) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) g_sm[par ^ 1][lc * VEC + v] = g[v];
            if (k == 0 && p.dinit_state && c_ok) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) *EMA_AT(p, p.dinit_state + row * p.d + c0 + v, 62) = a_r[0] * g[v];
            }
        }

        // decay gradient: partial over this CTA's channels
        if (per_step) {
            const float tot = reduce8_over16(acc, lc);
            const int64_t slot = blk * (static_cast<int64_t>(n_tiles) * QT) + t0 + (lc >> 1);
            if ((lc & 1) == 0) *EMA_AT(p, p.da_partial + slot, 63) = tot;
            if constexpr (WEIGHTED) {
                const float tot_w = reduce8_over16(acc_w, lc);
                const float tot_c = reduce8_over16(acc_c, lc);
                if ((lc & 1) == 0) {
                    *EMA_AT(p, p.da_partial + p.weighted_partial_stride + slot, 64) = tot_w;
                    *EMA_AT(p, p.da_partial + 2 * p.weighted_partial_stride + slot, 65) = tot_c;
                }
            }
        } else {
            float tot = 0.f;
#pragma unroll
            for (int s = 0; s < SB; ++s) tot += acc[s];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
            if ((tid & 31) == 0)
                *EMA_AT(p, p.da_partial + kHeadPartialOffset(p.b * p.h) + (blk * n_tiles + k) * (kFmaThreads / 32) + (tid >> 5),
                        66) = tot;
        }

        if (p.stop_below > 0.f) {
            float tp = 1.f;
#pragma unroll
            for (int i = 0; i < NS; ++i) tp *= Pr_sm[par][i];
            run *= tp;
            if (run < p.stop_below) break;
        }
        feed.end(k, more);
        if (more) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) hs[v] = hs_next[v];
        }
    }
    feed.finish();
}

}  // namespace ema
