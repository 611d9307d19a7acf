// The forward scan of the CUDA-core family as a function template, so that the same arithmetic can be fed either by
// plain global loads with a register prefetch (any dtype, stride or alignment) or by a TMA ring in shared memory.
#pragma once

#include "ema_common.cuh"

namespace ema {

// x tiles through registers: tile k + 1 is loaded while tile k computes
template <typename T, int VEC>
struct RegisterFeed {
    using R = raw_t<T, VEC>;
    R cur[kFmaSB], nxt[kFmaSB];
    const T *xrow;
    int64_t x_sl;
    int sub, L;
    bool c_ok;
    BoundsTable *bounds;
    __device__ __forceinline__ void load(R (&dst)[kFmaSB], int t0) {
#pragma unroll
        for (int s = 0; s < kFmaSB; ++s) {
            const int t = t0 + s;
            const bool ok = c_ok && t < L;
            dst[s] = ok ? ld_stream<T, VEC>(EMA_ATN(*this, xrow + static_cast<int64_t>(t) * x_sl, 1, sizeof(T) * VEC))
                        : raw_zero<T, VEC>();
        }
    }
    __device__ __forceinline__ void init(const FusedParams &p, const T *xrow_, bool c_ok_, int sub_, int L_) {
        xrow = xrow_; x_sl = p.x_sl; sub = sub_; L = L_; c_ok = c_ok_; bounds = p.bounds;
        load(cur, sub * kFmaSB);
    }
    __device__ __forceinline__ void begin(int k, bool more) {
        if (more) load(nxt, (k + 1) * kFmaTile + sub * kFmaSB);
    }
    __device__ __forceinline__ void after_barrier(int) {}
    __device__ __forceinline__ void end() {
#pragma unroll
        for (int s = 0; s < kFmaSB; ++s) cur[s] = nxt[s];
    }
    __device__ __forceinline__ void finish() {}
};

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
// WEIGHTED: the input weight of step t is in_weight[b,t,h] instead of the convention's (1 - a_t or 1), and what is
// written is out_weight[b,t,h] * state (when given); the saved, chunk and final states are the states themselves.
//
// FEED supplies the x tile: `cur[s]` holds this thread's VEC channels of step s of its sub-block.
//   init(...)         before the first tile (ends before the block-wide barrier of the prologue)
//   begin(k, more)    top of tile k: make cur valid / start fetching tile k + 1
//   after_barrier(k)  after the tile's block-wide barrier: every thread has consumed tile k's staging, if any
//   end()             bottom of tile k
//   finish()          after the last tile
template <typename T, int VEC, bool WEIGHTED, typename FEED>
__device__ __forceinline__ void ema_fwd_fma_body(const FusedParams &p, FEED &feed) {
    constexpr int CT = kFmaCT, SB = kFmaSB, NS = kFmaNS, QT = kFmaTile, DT = CT * VEC;
    using R = raw_t<T, VEC>;
    constexpr int WQ = WEIGHTED ? QT : 1;   // the weight tables exist only in the weighted kernel
    __shared__ float a_sm[2][QT];
    // Weight tables of a tile.  Unlike the decays they are read after the tile's block-wide barrier too, while a faster
    // thread may already be writing the next tile's entries: three buffers (tile k in buffer k % 3) keep the two apart.
    __shared__ float w_sm[3][WQ];   // input weights
    __shared__ float c_sm[3][WQ];   // output weights
    __shared__ float S_sm[2][NS][DT];
    __shared__ float P_sm[2][NS];
    __shared__ float h_sm[2][DT];

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

    const T *xrow = static_cast<const T *>(p.x) + bi * p.x_sb + hi * p.x_sh + c0;
    T *yrow = static_cast<T *>(p.out) + bi * p.o_sb + hi * p.o_sh + c0;
    const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
    const float a_head_raw = per_step ? 0.f : *EMA_AT(p, arow, 2);
    const float a_head = per_step ? 1.f : (conv ? expf(a_head_raw) : a_head_raw);

    auto load_a = [&](int t) -> float {  // multiplicative decay of step t (identity past the end)
        if (t >= L) return 1.f;
        if (!per_step) return a_head;
        const float v = *EMA_AT(p, arow + static_cast<int64_t>(t) * p.a_sl, 3);
        return conv ? expf(v) : v;
    };
    // per-step weights share the decay's strides (weighted calls always have a per-step decay); a missing output
    // weight is 1, a missing input weight the convention's (1 - a, or 1)
    const int64_t w_off = bi * p.a_sb + hi * p.a_sh;
    auto load_w = [&](const float *w, int t) -> float {
        if (!w) return 1.f;
        return t < L ? *EMA_AT(p, w + w_off + static_cast<int64_t>(t) * p.a_sl, 4) : 0.f;
    };
    auto load_in_w = [&](int t) -> float {
        if (p.in_weight) return load_w(p.in_weight, t);
        if (t >= L) return 0.f;
        return conv ? 1.f : 1.f - *EMA_AT(p, arow + static_cast<int64_t>(t) * p.a_sl, 5);
    };

    float h[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v)
        h[v] = (p.init_state && c_ok) ? *EMA_AT(p, p.init_state + row * p.d + c0 + v, 6) : 0.f;
    if (sub == 0) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) h_sm[0][lc * VEC + v] = h[v];
    }
    if (tid < QT) a_sm[0][tid] = load_a(tid);
    if constexpr (WEIGHTED) {
        if (tid < QT) {
            w_sm[0][tid] = load_in_w(tid);
            c_sm[0][tid] = load_w(p.out_weight, tid);
        }
    }

    feed.init(p, xrow, c_ok, sub, L);
    R (&cur)[SB] = feed.cur;
    __syncthreads();

    float run = 1.f, logsum = 0.f;
    for (int k = 0; k < p.n_tiles; ++k) {
        const int par = k & 1;
        const int wb = WEIGHTED ? k % 3 : 0;   // buffer of the weight tables
        const int t0 = k * QT + sub * SB;
        const bool more = k + 1 < p.n_tiles;
        float a_pref = 1.f, w_pref = 0.f, c_pref = 0.f;
        feed.begin(k, more);
        if (more) {
            if (tid < QT) a_pref = load_a((k + 1) * QT + tid);
            if constexpr (WEIGHTED) {
                if (tid < QT) {
                    w_pref = load_in_w((k + 1) * QT + tid);
                    c_pref = load_w(p.out_weight, (k + 1) * QT + tid);
                }
            }
        }

        // phase 1: local scan from a zero state
        float a_r[SB];
#pragma unroll
        for (int s = 0; s < SB; ++s) a_r[s] = a_sm[par][sub * SB + s];
        float st[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) st[v] = 0.f;
        float Pl = 1.f;
#pragma unroll
        for (int s = 0; s < SB; ++s) {
            float xf[VEC];
            unpack<T, VEC>(cur[s], xf);
            const float pw = WEIGHTED ? w_sm[wb][(sub * SB + s) % WQ] : (conv ? 1.f : 1.f - a_r[s]);
#pragma unroll
            for (int v = 0; v < VEC; ++v) st[v] = fmaf(a_r[s], st[v], pw * xf[v]);
            Pl *= a_r[s];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) S_sm[par][sub][lc * VEC + v] = st[v];
        if (lc == 0) P_sm[par][sub] = Pl;
        if (more && tid < QT) a_sm[par ^ 1][tid] = a_pref;
        if constexpr (WEIGHTED) {
            if (more && tid < QT) {
                w_sm[(k + 1) % 3][tid] = w_pref;
                c_sm[(k + 1) % 3][tid] = c_pref;
            }
        }
        __syncthreads();
        feed.after_barrier(k);

        // carry: state entering this sub-block
#pragma unroll
        for (int v = 0; v < VEC; ++v) h[v] = h_sm[par][lc * VEC + v];
        if (sub == 0 && c_ok) {
            if (p.tile_states) {
                float *ts = p.tile_states + (row * p.n_tiles + k) * p.d + c0;
#pragma unroll
                for (int v = 0; v < VEC; ++v) *EMA_AT(p, ts + v, 7) = h[v];
            }
            if (k == 0 && p.chunk_states) {
                float *cs = p.chunk_states + (row * p.n_chunks) * p.d + c0;
#pragma unroll
                for (int v = 0; v < VEC; ++v) *EMA_AT(p, cs + v, 8) = h[v];
            }
        }
        for (int i = 0; i < sub; ++i) {
            const float Pi = P_sm[par][i];
#pragma unroll
            for (int v = 0; v < VEC; ++v) h[v] = fmaf(Pi, h[v], S_sm[par][i][lc * VEC + v]);
        }

        // phase 2: re-run from the true state and emit
        int c_idx = 0, c_rem = 1;
        if (p.chunk_states) {
            c_idx = (t0 + 1) / p.chunk;
            c_rem = (t0 + 1) % p.chunk;
        }
#pragma unroll
        for (int s = 0; s < SB; ++s) {
            float xf[VEC];
            unpack<T, VEC>(cur[s], xf);
            const float pw = WEIGHTED ? w_sm[wb][(sub * SB + s) % WQ] : (conv ? 1.f : 1.f - a_r[s]);
#pragma unroll
            for (int v = 0; v < VEC; ++v) h[v] = fmaf(a_r[s], h[v], pw * xf[v]);
            const int t = t0 + s;
            if (c_ok && t < L) {
                if constexpr (WEIGHTED) {
                    if (p.out) {
                        const float cw = c_sm[wb][(sub * SB + s) % WQ];
                        float ys[VEC];
#pragma unroll
                        for (int v = 0; v < VEC; ++v) ys[v] = cw * h[v];
                        st_stream<T, VEC>(EMA_ATN(p, yrow + static_cast<int64_t>(t) * p.o_sl, 9, sizeof(T) * VEC),
                                          pack<T, VEC>(ys));
                    }
                } else {
                    if (p.out)
                        st_stream<T, VEC>(EMA_ATN(p, yrow + static_cast<int64_t>(t) * p.o_sl, 10, sizeof(T) * VEC),
                                          pack<T, VEC>(h));
                }
                if (p.chunk_states) {
                    // y_t is the state at the start of chunk (t+1)/chunk when t+1 is a boundary
                    if (c_rem == 0 && t + 1 < L) {
                        float *cs = p.chunk_states + (row * p.n_chunks + c_idx) * p.d + c0;
#pragma unroll
                        for (int v = 0; v < VEC; ++v) *EMA_AT(p, cs + v, 11) = h[v];
                    }
                }
            }
            if (p.chunk_states) {
                if (++c_rem == p.chunk) { c_rem = 0; ++c_idx; }
            }
        }
        if (sub == NS - 1) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) h_sm[par ^ 1][lc * VEC + v] = h[v];
        }

        if (p.stop_below > 0.f || p.log_decay_sum) {
            float tp = 1.f;
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                const float Pi = P_sm[par][i];
                tp *= Pi;
                logsum += logf(Pi);
            }
            run *= tp;
            if (p.stop_below > 0.f && run < p.stop_below) break;
        }
        feed.end();
    }
    feed.finish();

    // h of the last sub-block is the state after the last processed step (steps past L are identity)
    if (sub == NS - 1 && c_ok && p.final_state) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) *EMA_AT(p, p.final_state + row * p.d + c0 + v, 12) = h[v];
    }
    if (p.log_decay_sum && tid == 0 && dtile == 0) *EMA_AT(p, p.log_decay_sum + row, 13) = logsum;
}

}  // namespace ema
