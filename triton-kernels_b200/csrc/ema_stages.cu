// Stage kernels: one CUDA kernel per stage of the reference's chunked EMA pipeline, on the
// reference's folded layouts (X[B,L,T], A[B,L], cs[B,C,Q], per-chunk states [B,C,T]).  They exist
// so that every per-stage entry point of the reference has a drop-in; the fused kernels are the
// fast path.  All are bandwidth-shaped: a thread owns a channel (coalesced across T) and walks the
// chunk with the O(Q) recurrence instead of the O(Q^2) decay matrix, which is the same sum.
#include "ema_common.cuh"

namespace ema {
namespace {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ int chunk_limit(int64_t L, int Q, int64_t c) {
    const int64_t rest = L - c * Q;
    return static_cast<int>(rest < Q ? rest : Q);
}

// cs[b,c,q] = inclusive cumsum over the chunk of A, zero padded past L.  One warp per (b,c).
__global__ void chunk_cumsum_kernel(Ptr<const float> A, int64_t A_sb, int64_t A_sl,
                                    Ptr<float> cs, int64_t B, int64_t L, int Q, int64_t C) {
    const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= B * C) return;
    const int64_t b = w / C, c = w % C;
    const int lim = chunk_limit(L, Q, c);
    float carry = 0.f;
    for (int q0 = 0; q0 < Q; q0 += 32) {
        const int q = q0 + lane;
        float v = (q < lim) ? A[b * A_sb + (c * Q + q) * A_sl] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(kFull, v, o);
            if (lane >= o) v += n;
        }
        v += carry;
        if (q < Q) cs[(b * C + c) * Q + q] = v;
        carry = __shfl_sync(kFull, v, 31);
    }
}

// S[b,c,t] = sum_q exp(min(cs_last - cs_q, 0)) u_q, cs_last read at the last valid step.
template <typename T>
__global__ void chunk_state_kernel(Ptr<const T> X, Ptr<const float> cs,
                                   Ptr<float> S, int64_t L, int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    const float last = csr[lim - 1];
    const auto xr = X + (b * L + c * Q) * Tn + t;
    float acc = 0.f;
    for (int q = 0; q < lim; ++q)
        acc = fmaf(expf(fminf(last - csr[q], 0.f)), to_f32<T>(xr[static_cast<int64_t>(q) * Tn]), acc);
    S[bc * Tn + t] = acc;
}

// out[b,c,:] = state at the start of chunk c; final[b,:] = state after the last chunk.
__global__ void state_passing_fwd_kernel(Ptr<const float> S, Ptr<const float> cl,
                                         int64_t cl_sb, int64_t cl_sc, Ptr<float> out,
                                         Ptr<float> fin, int64_t C, int64_t Tn) {
    const int64_t b = blockIdx.x;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    float acc = 0.f;
    for (int64_t c = 0; c < C; ++c) {
        out[(b * C + c) * Tn + t] = acc;
        acc = fmaf(expf(cl[b * cl_sb + c * cl_sc]), acc, S[(b * C + c) * Tn + t]);
    }
    fin[b * Tn + t] = acc;
}

// y_m = exp(min(cs_m,0)) h_c + sum_{k<=m} exp(min(cs_m-cs_k,0)) u_k, as the recurrence
// y_m = exp(min(cs_m - cs_{m-1},0)) y_{m-1} + u_m started from h_c.
template <typename T>
__global__ void chunk_scan_kernel(Ptr<const T> X, Ptr<const float> cs,
                                  Ptr<const float> h, Ptr<T> out, int64_t L,
                                  int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    const int64_t base = (b * L + c * Q) * Tn + t;
    float y = h[bc * Tn + t];
    float prev = 0.f;
    for (int m = 0; m < lim; ++m) {
        const float cur = csr[m];
        y = fmaf(expf(fminf(cur - prev, 0.f)), y, to_f32<T>(X[base + static_cast<int64_t>(m) * Tn]));
        out[base + static_cast<int64_t>(m) * Tn] = from_f32<T>(y);
        prev = cur;
    }
}

// dh[b,c,t] = sum_q exp(cs_q) dy_q
template <typename T>
__global__ void bwd_dstates_kernel(Ptr<const float> cs, Ptr<const T> dout,
                                   Ptr<float> dh, int64_t L, int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    const auto gr = dout + (b * L + c * Q) * Tn + t;
    float acc = 0.f;
    for (int q = 0; q < lim; ++q)
        acc = fmaf(expf(csr[q]), to_f32<T>(gr[static_cast<int64_t>(q) * Tn]), acc);
    dh[bc * Tn + t] = acc;
}

// Reverse carry of the adjoint over chunks.  One CTA per batch row; threads stride over T.
// dS[c] = adjoint of chunk c's local state; ddA_last[c] = exp(cs_last_c) <h_c, dS[c]>, 0 for c = 0.
__global__ void state_passing_bwd_kernel(Ptr<const float> h, Ptr<const float> cl,
                                         int64_t cl_sb, int64_t cl_sc, Ptr<const float> dh,
                                         Ptr<float> dS, Ptr<float> ddA, int64_t C,
                                         int64_t Tn) {
    constexpr int kMaxPerThread = 16;  // T <= 16 * blockDim.x is checked by the host
    __shared__ float red[32];
    const int64_t b = blockIdx.x;
    const int nthr = blockDim.x;
    float g[kMaxPerThread];
#pragma unroll
    for (int i = 0; i < kMaxPerThread; ++i) g[i] = 0.f;
    for (int64_t c = C - 1; c >= 0; --c) {
        const float scale = expf(cl[b * cl_sb + c * cl_sc]);
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxPerThread; ++i) {
            const int64_t t = static_cast<int64_t>(i) * nthr + threadIdx.x;
            if (t < Tn) {
                const int64_t o = (b * C + c) * Tn + t;
                dS[o] = g[i];
                if (c > 0) {
                    part = fmaf(h[o], g[i], part);
                    g[i] = fmaf(scale, g[i], dh[o]);
                }
            }
        }
        // block sum of part in a fixed order
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(kFull, part, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < (nthr + 31) / 32; ++w) s += red[w];
            ddA[b * C + c] = c > 0 ? s * scale : 0.f;
        }
        __syncthreads();
    }
}

// du_m = exp(min(cs_last - cs_m,0)) dS_c + sum_{k>=m} exp(min(cs_k - cs_m,0)) dy_k, as the reverse
// recurrence started from dS_c; cs_last is slot Q-1 (constant past a ragged end).
template <typename T>
__global__ void bwd_dx_kernel(Ptr<const float> cs, Ptr<const T> dout,
                              Ptr<const float> dS, Ptr<T> dx, int64_t L,
                              int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    const int64_t base = (b * L + c * Q) * Tn + t;
    float g = dS[bc * Tn + t];
    float next = csr[Q - 1];
    for (int m = lim - 1; m >= 0; --m) {
        const float cur = csr[m];
        g = fmaf(expf(fminf(next - cur, 0.f)), g, to_f32<T>(dout[base + static_cast<int64_t>(m) * Tn]));
        dx[base + static_cast<int64_t>(m) * Tn] = from_f32<T>(g);
        next = cur;
    }
}

// row-wise dot products: one warp per (b, c, m).
//   kind 0 (db): g_m = exp(min(cs_last - cs_m,0)) <dS_c, u_m>, written to slot m+1 for m < limit-1
//   kind 1 (dc): r_m = exp(cs_m) <dy_m, h_c>, zero for m >= limit
template <typename T, int KIND>
__global__ void row_dot_kernel(Ptr<const T> rows, Ptr<const float> cs,
                               Ptr<const float> vec, Ptr<float> out, int64_t L,
                               int64_t Tn, int Q, int64_t C, int64_t total) {
    const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= total) return;
    const int m = static_cast<int>(w % Q);
    const int64_t bc = w / Q;
    const int64_t b = bc / C, c = bc % C;
    const int lim = chunk_limit(L, Q, c);
    float acc = 0.f;
    if (m < lim) {
        const auto r = rows + (b * L + c * Q + m) * Tn;
        const auto v = vec + bc * Tn;
        for (int64_t t = lane; t < Tn; t += 32) acc = fmaf(to_f32<T>(r[t]), v[t], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
    if (lane != 0) return;
    const auto csr = cs + bc * Q;
    if (KIND == 0) {
        if (m == 0) out[bc * Q] = 0.f;
        if (m + 1 < Q)
            out[bc * Q + m + 1] = (m < lim - 1) ? acc * expf(fminf(csr[Q - 1] - csr[m], 0.f)) : 0.f;
    } else {
        out[bc * Q + m] = (m < lim) ? acc * expf(csr[m]) : 0.f;
    }
}

// in-place inclusive cumsum along the last axis of [rows, Q]; one warp per row
__global__ void row_cumsum_kernel(Ptr<float> v, int64_t rows, int Q) {
    const int64_t w = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= rows) return;
    float carry = 0.f;
    for (int q0 = 0; q0 < Q; q0 += 32) {
        const int q = q0 + lane;
        float x = (q < Q) ? v[w * Q + q] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(kFull, x, o);
            if (lane >= o) x += n;
        }
        x += carry;
        if (q < Q) v[w * Q + q] = x;
        carry = __shfl_sync(kFull, x, 31);
    }
}

// Intra-chunk decay gradient.  The reference builds G[m,k] = <dy_m,u_k> exp(min(cs_m-cs_k,0)) for
// m > k and returns out[j+1] = sum_{m>j} sum_{k<=j} G[m,k].  With the local scans
//   yl_j = sum_{k<=j} exp(cs_j-cs_k) u_k   and   ll_m = sum_{n>=m} exp(cs_n-cs_m) dy_n
// that double sum is out[j+1] = exp(min(cs_{j+1}-cs_j,0)) <ll_{j+1}, yl_j>: two O(Q) passes.
// One CTA per (b,c); each warp owns 32 channels at a time, keeps yl for the whole chunk in shared
// memory, runs the reverse pass, and adds its per-step sums into a shared accumulator in a fixed
// order (warps take turns), so the result is deterministic.
template <typename T>
__global__ void bwd_dacs_kernel(Ptr<const T> X, Ptr<const float> cs,
                                Ptr<const T> dout, Ptr<float> out, int64_t L,
                                int64_t Tn, int Q, int64_t C) {
    extern __shared__ float sm[];
    const int nwarps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float *acc = sm;                                // [Q]
    float *part = sm + Q;                           // [nwarps][Q]
    float *yl = sm + Q + static_cast<size_t>(nwarps) * Q + static_cast<size_t>(warp) * Q * 32;  // [Q][32]
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    for (int q = threadIdx.x; q < Q; q += blockDim.x) acc[q] = 0.f;
    __syncthreads();
    for (int64_t t0 = 0; t0 < Tn; t0 += static_cast<int64_t>(nwarps) * 32) {
        const int64_t t = t0 + warp * 32 + lane;
        const bool ok = t < Tn;
        const int64_t base = (b * L + c * Q) * Tn + t;
        float y = 0.f, prev = 0.f;
        for (int j = 0; j < lim; ++j) {
            const float cur = csr[j];
            const float xv = ok ? to_f32<T>(X[base + static_cast<int64_t>(j) * Tn]) : 0.f;
            y = fmaf(expf(fminf(cur - prev, 0.f)), y, xv);
            yl[j * 32 + lane] = y;
            prev = cur;
        }
        float ll = 0.f;
        float next = lim > 0 ? csr[lim - 1] : 0.f;
        for (int m = lim - 1; m >= 1; --m) {
            const float cur = csr[m];
            const float gv = ok ? to_f32<T>(dout[base + static_cast<int64_t>(m) * Tn]) : 0.f;
            ll = fmaf(expf(fminf(next - cur, 0.f)), ll, gv);  // ll_m
            float v = ll * yl[(m - 1) * 32 + lane] * expf(fminf(cur - csr[m - 1], 0.f));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
            if (lane == 0) part[warp * Q + m] = v;
            next = cur;
        }
        __syncthreads();
        for (int q = threadIdx.x; q < Q; q += blockDim.x) {
            if (q >= 1 && q < lim) {
                float s = acc[q];
                for (int w = 0; w < nwarps; ++w) s += part[w * Q + q];
                acc[q] = s;
            }
        }
        __syncthreads();
    }
    for (int q = threadIdx.x; q < Q; q += blockDim.x) out[bc * Q + q] = acc[q];
}

// ------------------------------------------------------------------------------------------------
// 128-bit variants.  Taken when T is a multiple of the vector width (4 fp32 or 8 bf16 channels) and the tensors are
// 16-byte aligned; the scalar kernels above remain for every other shape.  Same sums in a different order.
// ------------------------------------------------------------------------------------------------
template <typename T> struct Vec16 { static constexpr int n = 16 / static_cast<int>(sizeof(T)); };

template <typename T>
__device__ __forceinline__ void load16(Ptr<const T> p, float (&f)[Vec16<T>::n]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4 *>(chk_bytes(p, 16)));
    unpack<T, Vec16<T>::n>(r, f);
}
template <typename T>
__device__ __forceinline__ void store16(Ptr<T> p, const float (&f)[Vec16<T>::n]) {
    *reinterpret_cast<uint4 *>(chk_bytes(p, 16)) = pack<T, Vec16<T>::n>(f);
}

// Weighted column sums of one chunk: out[b,c,:] = sum_q w_q rows[b, cQ+q, :].
//   KIND 0 (chunk state)  w_q = exp(min(cs_last - cs_q, 0))      KIND 1 (dstates)  w_q = exp(cs_q)
// 256 threads: warp g takes steps g, g+8, ..., lane l takes VEC channels; four 16-byte loads in flight per thread,
// a fixed-order sum over the eight warps at the end.  Dynamic shared memory: w[Q] + red[8][32 VEC].
template <typename T, int KIND>
__global__ void __launch_bounds__(256) weighted_colsum_kernel(Ptr<const T> rows, Ptr<const float> cs,
                                                              Ptr<float> out, int64_t L, int64_t Tn, int Q,
                                                              int64_t C) {
    constexpr int VEC = Vec16<T>::n;
    constexpr int CH = 32 * VEC;
    extern __shared__ float sm[];
    float *w = sm;
    float *red = sm + Q;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    const float last = csr[lim - 1];
    for (int q = tid; q < Q; q += 256)
        w[q] = q < lim ? (KIND == 0 ? expf(fminf(last - csr[q], 0.f)) : expf(csr[q])) : 0.f;
    __syncthreads();
    const int64_t ch = static_cast<int64_t>(blockIdx.y) * CH + lane * VEC;
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    if (ch < Tn) {
        const auto base = rows + (b * L + c * Q) * Tn + ch;
        for (int q0 = warp; q0 < lim; q0 += 32) {
            float f[4][VEC];
            float wq[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int q = q0 + 8 * i;
                const bool ok = q < lim;
                load16<T>(base + static_cast<int64_t>(ok ? q : lim - 1) * Tn, f[i]);   // rows past the end count with weight 0
                wq[i] = ok ? w[q] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wq[i], f[i][e], acc[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) red[warp * CH + lane * VEC + e] = acc[e];
    __syncthreads();
    const int64_t co = static_cast<int64_t>(blockIdx.y) * CH + tid;
    if (tid < CH && co < Tn) {
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < 8; ++g) s += red[g * CH + tid];
        out[bc * Tn + co] = s;
    }
    if (CH > 256) {   // bf16: 256 channels per block, second half of the channels
        const int t2 = tid + 256;
        const int64_t co2 = static_cast<int64_t>(blockIdx.y) * CH + t2;
        if (t2 < CH && co2 < Tn) {
            float s = 0.f;
#pragma unroll
            for (int g = 0; g < 8; ++g) s += red[g * CH + t2];
            out[bc * Tn + co2] = s;
        }
    }
}

// The chunk scan and its mirror, a thread per VEC channels walking the chunk with the O(Q) recurrence; the per-step
// factors are worked out once per block into shared memory (dynamic, Q floats), four steps' loads are in flight.
//   REVERSE = false: y_m = f_m y_{m-1} + x_m from the chunk-start state,  f_m = exp(min(cs_m - cs_{m-1}, 0)), cs_{-1} = 0
//   REVERSE = true : g_m = f_m g_{m+1} + dy_m from dS_c,                  f_m = exp(min(cs_{m+1} - cs_m, 0)), cs past the end = cs[Q-1]
template <typename T, bool REVERSE>
__global__ void __launch_bounds__(128) chunk_recurrence_vec_kernel(Ptr<const T> in, Ptr<const float> cs,
                                                                   Ptr<const float> start, Ptr<T> out,
                                                                   int64_t L, int64_t Tn, int Q, int64_t C) {
    constexpr int VEC = Vec16<T>::n;
    extern __shared__ float fac[];
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int lim = chunk_limit(L, Q, c);
    const auto csr = cs + bc * Q;
    for (int m = threadIdx.x; m < lim; m += blockDim.x) {
        if (!REVERSE) fac[m] = expf(fminf(csr[m] - (m > 0 ? csr[m - 1] : 0.f), 0.f));
        else fac[m] = expf(fminf((m + 1 < lim ? csr[m + 1] : csr[Q - 1]) - csr[m], 0.f));
    }
    __syncthreads();
    const int64_t ch = (static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x) * VEC;
    if (ch >= Tn) return;
    float s[VEC];
#pragma unroll
    for (int e = 0; e < VEC; e += 4) {
        const float4 v = *reinterpret_cast<const float4 *>(chk_bytes(start + bc * Tn + ch + e, 16));
        s[e] = v.x; s[e + 1] = v.y; s[e + 2] = v.z; s[e + 3] = v.w;
    }
    const int64_t base = (b * L + c * Q) * Tn + ch;
    for (int j0 = 0; j0 < lim; j0 += 4) {
        float f[4][VEC];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = j0 + i < lim ? j0 + i : lim - 1;
            const int m = REVERSE ? lim - 1 - j : j;
            load16<T>(in + base + static_cast<int64_t>(m) * Tn, f[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (j0 + i < lim) {
                const int m = REVERSE ? lim - 1 - (j0 + i) : j0 + i;
                const float fm = fac[m];
#pragma unroll
                for (int e = 0; e < VEC; ++e) s[e] = fmaf(fm, s[e], f[i][e]);
                store16<T>(out + base + static_cast<int64_t>(m) * Tn, s);
            }
        }
    }
}

// Forward carry over the chunks, four channels per thread (128-bit loads and stores, coalesced across the warp) with
// the next kDepth chunk states already in flight: the chain itself is one FMA per chunk.
constexpr int kPassDepth = 16;
__global__ void __launch_bounds__(32) state_passing_fwd_vec_kernel(Ptr<const float4> S, Ptr<const float> cl,
                                                                   int64_t cl_sb, int64_t cl_sc, Ptr<float4> out,
                                                                   Ptr<float4> fin, int64_t C, int64_t T4) {
    const int64_t b = blockIdx.x;
    const int64_t t4 = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t4 >= T4) return;
    const auto src = S + b * C * T4 + t4;
    const auto dst = out + b * C * T4 + t4;
    const auto clb = cl + b * cl_sb;
    float4 buf[kPassDepth];
    float sc[kPassDepth];
#pragma unroll
    for (int i = 0; i < kPassDepth; ++i) {
        if (i < C) { buf[i] = __ldg(chk(src + i * T4)); sc[i] = expf(clb[i * cl_sc]); }
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t c0 = 0; c0 < C; c0 += kPassDepth) {
#pragma unroll
        for (int i = 0; i < kPassDepth; ++i) {
            const int64_t c = c0 + i;
            if (c < C) {
                dst[c * T4] = acc;
                acc.x = fmaf(sc[i], acc.x, buf[i].x); acc.y = fmaf(sc[i], acc.y, buf[i].y);
                acc.z = fmaf(sc[i], acc.z, buf[i].z); acc.w = fmaf(sc[i], acc.w, buf[i].w);
                if (c + kPassDepth < C) { buf[i] = __ldg(chk(src + (c + kPassDepth) * T4)); sc[i] = expf(clb[(c + kPassDepth) * cl_sc]); }
            }
        }
    }
    fin[b * T4 + t4] = acc;
}

// Reverse carry of the adjoint, one warp per 128 channels of a batch row (so a row is spread over T / 128 thread
// blocks).  Every warp writes the dot product <h_c, dS_c> over ITS channels to partial[b, c, warp]; a second kernel
// sums the partials in a fixed order and applies exp(cs_last).
constexpr int kPassBwdDepth = 8;
__global__ void __launch_bounds__(32) state_passing_bwd_vec_kernel(Ptr<const float4> h, Ptr<const float> cl,
                                                                   int64_t cl_sb, int64_t cl_sc, Ptr<const float4> dh,
                                                                   Ptr<float4> dS, Ptr<float> partial,
                                                                   int64_t C, int64_t T4, int n_warps) {
    const int64_t b = blockIdx.x;
    const int wi = blockIdx.y;
    const int lane = threadIdx.x;
    const int64_t t4 = static_cast<int64_t>(wi) * 32 + lane;
    const bool ok = t4 < T4;
    const int64_t off = b * C * T4 + (ok ? t4 : 0);
    const auto clb = cl + b * cl_sb;
    float4 hb[kPassBwdDepth], db[kPassBwdDepth];
    float sc[kPassBwdDepth];
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < kPassBwdDepth; ++i) {
        const int64_t c = C - 1 - i;
        if (c >= 0) {
            hb[i] = ok ? __ldg(chk(h + off + c * T4)) : zero;
            db[i] = ok ? __ldg(chk(dh + off + c * T4)) : zero;
            sc[i] = expf(clb[c * cl_sc]);
        }
    }
    float4 g = zero;
    for (int64_t c0 = C - 1; c0 >= 0; c0 -= kPassBwdDepth) {
#pragma unroll
        for (int i = 0; i < kPassBwdDepth; ++i) {
            const int64_t c = c0 - i;
            if (c >= 0) {
                if (ok) dS[off + c * T4] = g;
                float part = hb[i].x * g.x + hb[i].y * g.y + hb[i].z * g.z + hb[i].w * g.w;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(kFull, part, o);
                if (lane == 0) partial[(b * C + c) * n_warps + wi] = part;
                if (c > 0) {
                    g.x = fmaf(sc[i], g.x, db[i].x); g.y = fmaf(sc[i], g.y, db[i].y);
                    g.z = fmaf(sc[i], g.z, db[i].z); g.w = fmaf(sc[i], g.w, db[i].w);
                }
                const int64_t cn = c - kPassBwdDepth;
                if (cn >= 0) {
                    hb[i] = ok ? __ldg(chk(h + off + cn * T4)) : zero;
                    db[i] = ok ? __ldg(chk(dh + off + cn * T4)) : zero;
                    sc[i] = expf(clb[cn * cl_sc]);
                }
            }
        }
    }
}
// ddA_last[b, c] = exp(cs_last[b, c]) * sum_w partial[b, c, w] for c > 0, and 0 for the first chunk
__global__ void state_passing_bwd_sum_kernel(Ptr<const float> partial, Ptr<const float> cl, int64_t cl_sb,
                                             int64_t cl_sc, Ptr<float> ddA, int64_t B, int64_t C, int n_warps) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= B * C) return;
    const int64_t b = i / C, c = i % C;
    float s = 0.f;
    for (int w = 0; w < n_warps; ++w) s += partial[i * n_warps + w];
    ddA[i] = c > 0 ? s * expf(cl[b * cl_sb + c * cl_sc]) : 0.f;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline unsigned cdiv(int64_t a, int64_t b) { return static_cast<unsigned>((a + b - 1) / b); }

}  // namespace
}  // namespace ema

using namespace ema;

// ---- launchers of the 128-bit variants ------------------------------------------------------------------------
static bool colsum_vec_ok(const void *rows, int dtype, int64_t T, int Q) {
    const int vec = dtype == EMA_F32 ? 4 : 8;
    return (dtype == EMA_F32 || dtype == EMA_BF16) && T % vec == 0 && aligned16(rows) && Q <= 8192 &&
           (T + 32 * vec - 1) / (32 * vec) <= 65535;
}
template <int KIND>
static int launch_colsum_vec(const void *rows, const float *cs, float *out, int dtype, int64_t B, int64_t L, int64_t T,
                             int Q, int64_t C, cudaStream_t st, BoundsTable *tb) {
    const int vec = dtype == EMA_F32 ? 4 : 8;
    const size_t smem = (static_cast<size_t>(Q) + 8 * 32 * vec) * sizeof(float);
    dim3 grid(static_cast<unsigned>(B * C), static_cast<unsigned>((T + 32 * vec - 1) / (32 * vec)));
    if (dtype == EMA_F32)
        weighted_colsum_kernel<float, KIND><<<grid, 256, smem, st>>>(make_ptr(static_cast<const float *>(rows), tb, 300),
                                                                     make_ptr(cs, tb, 301), make_ptr(out, tb, 302), L, T, Q, C);
    else
        weighted_colsum_kernel<__nv_bfloat16, KIND><<<grid, 256, smem, st>>>(
            make_ptr(static_cast<const __nv_bfloat16 *>(rows), tb, 300), make_ptr(cs, tb, 301), make_ptr(out, tb, 302), L, T, Q, C);
    return check_launch();
}
static bool recurrence_vec_ok(const void *in, const void *out, const float *start, int dtype, int64_t T, int Q) {
    const int vec = dtype == EMA_F32 ? 4 : 8;
    return (dtype == EMA_F32 || dtype == EMA_BF16) && T % vec == 0 && aligned16(in) && aligned16(out) && aligned16(start) &&
           Q <= 8192 && (T / vec + 127) / 128 <= 65535;
}
template <bool REVERSE>
static int launch_recurrence_vec(const void *in, const float *cs, const float *start, void *out, int dtype, int64_t B,
                                 int64_t L, int64_t T, int Q, int64_t C, cudaStream_t st, BoundsTable *tb) {
    const int vec = dtype == EMA_F32 ? 4 : 8;
    const int64_t groups = T / vec;
    const int threads = groups >= 128 ? 128 : static_cast<int>((groups + 31) / 32 * 32);
    dim3 grid(static_cast<unsigned>(B * C), static_cast<unsigned>((groups + threads - 1) / threads));
    const size_t smem = static_cast<size_t>(Q) * sizeof(float);
    if (dtype == EMA_F32)
        chunk_recurrence_vec_kernel<float, REVERSE><<<grid, threads, smem, st>>>(
            make_ptr(static_cast<const float *>(in), tb, 310), make_ptr(cs, tb, 311), make_ptr(start, tb, 312),
            make_ptr(static_cast<float *>(out), tb, 313), L, T, Q, C);
    else
        chunk_recurrence_vec_kernel<__nv_bfloat16, REVERSE><<<grid, threads, smem, st>>>(
            make_ptr(static_cast<const __nv_bfloat16 *>(in), tb, 310), make_ptr(cs, tb, 311), make_ptr(start, tb, 312),
            make_ptr(static_cast<__nv_bfloat16 *>(out), tb, 313), L, T, Q, C);
    return check_launch();
}

#define EMA_REQUIRE(cond, code) \
    do {                        \
        if (!(cond)) return (code); \
    } while (0)

// Bounds-checking build: registers the buffers of a stage call (null otherwise, and the kernels' pointers are plain).
// Returns false when the table could not be written.
static bool stage_table(const BoundsRange *ranges, int n, cudaStream_t st, BoundsTable **tb) {
    *tb = nullptr;
    if (!ema_b200_bounds_checked()) return true;
    *tb = bounds_prepare(ranges, n, st);
    return *tb != nullptr;
}
static size_t esize(int dtype) { return dtype == EMA_F32 ? 4 : 2; }

static int stage_dims_ok(int64_t B, int64_t L, int64_t T, int Q) {
    if (B <= 0 || L <= 0 || T <= 0 || Q <= 0) return EMA_ERR_BADARG;
    if (L >= (1ll << 31) || (L + Q - 1) / Q * B > 2000000000ll || T > 65535ll * 128) return EMA_ERR_UNSUPPORTED;
    return EMA_OK;
}

extern "C" int ema_b200_chunk_cumsum(const float *A, int64_t A_sb, int64_t A_sl, float *cs, int64_t B,
                                     int64_t L, int Q, void *stream) {
    EMA_REQUIRE(A && cs, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, 1, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{cs, static_cast<size_t>(B * C * Q) * 4},
                                  {A, static_cast<size_t>((B - 1) * A_sb + (L - 1) * A_sl + 1) * 4}};
    if (!stage_table(ranges, 2, st, &tb)) return EMA_ERR_CUDA;
    chunk_cumsum_kernel<<<cdiv(B * C * 32, 128), 128, 0, st>>>(make_ptr(A, tb, 320), A_sb, A_sl, make_ptr(cs, tb, 321), B, L, Q,
                                                               C);
    return check_launch();
}

#define EMA_STAGE_DISPATCH(dtype, CALL_F32, CALL_BF16) \
    if ((dtype) == EMA_F32) { CALL_F32; }              \
    else if ((dtype) == EMA_BF16) { CALL_BF16; }       \
    else return EMA_ERR_UNSUPPORTED;

extern "C" int ema_b200_chunk_state(const void *X, const float *cs, float *S, int dtype, int64_t B,
                                    int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(X && cs && S, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{S, static_cast<size_t>(B * C * T) * 4}, {X, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {cs, static_cast<size_t>(B * C * Q) * 4}};
    if (!stage_table(ranges, 3, st, &tb)) return EMA_ERR_CUDA;
    if (colsum_vec_ok(X, dtype, T, Q)) return launch_colsum_vec<0>(X, cs, S, dtype, B, L, T, Q, C, st, tb);
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    EMA_STAGE_DISPATCH(dtype,
        (chunk_state_kernel<float><<<grid, 128, 0, st>>>(make_ptr(static_cast<const float *>(X), tb, 330), make_ptr(cs, tb, 331), make_ptr(S, tb, 332), L, T, Q, C)),
        (chunk_state_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(make_ptr(static_cast<const __nv_bfloat16 *>(X), tb, 330), make_ptr(cs, tb, 331), make_ptr(S, tb, 332), L, T, Q, C)))
    return check_launch();
}

extern "C" int ema_b200_state_passing_fwd(const float *S, const float *cs_last, int64_t cl_sb,
                                          int64_t cl_sc, float *out, float *final_states, int64_t B,
                                          int64_t C, int64_t T, void *stream) {
    EMA_REQUIRE(S && cs_last && out && final_states, EMA_ERR_BADARG);
    EMA_REQUIRE(B > 0 && C > 0 && T > 0, EMA_ERR_BADARG);
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{out, static_cast<size_t>(B * C * T) * 4}, {S, static_cast<size_t>(B * C * T) * 4},
                                  {final_states, static_cast<size_t>(B * T) * 4},
                                  {cs_last, static_cast<size_t>((B - 1) * cl_sb + (C - 1) * cl_sc + 1) * 4}};
    if (!stage_table(ranges, 4, st, &tb)) return EMA_ERR_CUDA;
    if (T % 4 == 0 && aligned16(S) && aligned16(out) && aligned16(final_states) && T / 4 <= 65535ll * 32) {
        dim3 grid(static_cast<unsigned>(B), cdiv(T / 4, 32));
        state_passing_fwd_vec_kernel<<<grid, 32, 0, st>>>(
            make_ptr(reinterpret_cast<const float4 *>(S), tb, 340), make_ptr(cs_last, tb, 341), cl_sb, cl_sc,
            make_ptr(reinterpret_cast<float4 *>(out), tb, 342), make_ptr(reinterpret_cast<float4 *>(final_states), tb, 343), C,
            T / 4);
        return check_launch();
    }
    dim3 grid(static_cast<unsigned>(B), cdiv(T, 128));
    state_passing_fwd_kernel<<<grid, 128, 0, st>>>(make_ptr(S, tb, 340), make_ptr(cs_last, tb, 341), cl_sb, cl_sc,
                                                   make_ptr(out, tb, 342), make_ptr(final_states, tb, 343), C, T);
    return check_launch();
}

extern "C" int ema_b200_chunk_scan(const void *X, const float *cs, const float *h, void *out, int dtype,
                                   int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(X && cs && h && out, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{out, static_cast<size_t>(B * L * T) * esize(dtype)}, {X, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {cs, static_cast<size_t>(B * C * Q) * 4}, {h, static_cast<size_t>(B * C * T) * 4}};
    if (!stage_table(ranges, 4, st, &tb)) return EMA_ERR_CUDA;
    if (recurrence_vec_ok(X, out, h, dtype, T, Q)) return launch_recurrence_vec<false>(X, cs, h, out, dtype, B, L, T, Q, C, st, tb);
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    EMA_STAGE_DISPATCH(dtype,
        (chunk_scan_kernel<float><<<grid, 128, 0, st>>>(make_ptr(static_cast<const float *>(X), tb, 350), make_ptr(cs, tb, 351), make_ptr(h, tb, 352), make_ptr(static_cast<float *>(out), tb, 353), L, T, Q, C)),
        (chunk_scan_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(make_ptr(static_cast<const __nv_bfloat16 *>(X), tb, 350), make_ptr(cs, tb, 351), make_ptr(h, tb, 352), make_ptr(static_cast<__nv_bfloat16 *>(out), tb, 353), L, T, Q, C)))
    return check_launch();
}

extern "C" int ema_b200_bwd_dstates(const float *cs, const void *dout, float *dh, int dtype, int64_t B,
                                    int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(cs && dout && dh, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{dh, static_cast<size_t>(B * C * T) * 4}, {dout, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {cs, static_cast<size_t>(B * C * Q) * 4}};
    if (!stage_table(ranges, 3, st, &tb)) return EMA_ERR_CUDA;
    if (colsum_vec_ok(dout, dtype, T, Q)) return launch_colsum_vec<1>(dout, cs, dh, dtype, B, L, T, Q, C, st, tb);
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    EMA_STAGE_DISPATCH(dtype,
        (bwd_dstates_kernel<float><<<grid, 128, 0, st>>>(make_ptr(cs, tb, 360), make_ptr(static_cast<const float *>(dout), tb, 361), make_ptr(dh, tb, 362), L, T, Q, C)),
        (bwd_dstates_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(make_ptr(cs, tb, 360), make_ptr(static_cast<const __nv_bfloat16 *>(dout), tb, 361), make_ptr(dh, tb, 362), L, T, Q, C)))
    return check_launch();
}

extern "C" size_t ema_b200_state_passing_bwd_workspace_bytes(int64_t B, int64_t C, int64_t T) {
    if (B <= 0 || C <= 0 || T <= 0 || T % 4 != 0) return 0;
    return static_cast<size_t>(B) * C * ((T / 4 + 31) / 32) * sizeof(float);
}

extern "C" int ema_b200_state_passing_bwd(const float *h, const float *cs_last, int64_t cl_sb,
                                          int64_t cl_sc, const float *dh, float *dS, float *ddA_last,
                                          int64_t B, int64_t C, int64_t T, void *workspace, size_t workspace_bytes,
                                          void *stream) {
    EMA_REQUIRE(h && cs_last && dh && dS && ddA_last, EMA_ERR_BADARG);
    EMA_REQUIRE(B > 0 && C > 0 && T > 0, EMA_ERR_BADARG);
    const size_t need = ema_b200_state_passing_bwd_workspace_bytes(B, C, T);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{dS, static_cast<size_t>(B * C * T) * 4}, {h, static_cast<size_t>(B * C * T) * 4},
                                  {dh, static_cast<size_t>(B * C * T) * 4}, {ddA_last, static_cast<size_t>(B * C) * 4},
                                  {cs_last, static_cast<size_t>((B - 1) * cl_sb + (C - 1) * cl_sc + 1) * 4},
                                  {workspace, workspace ? need : 0}};
    if (!stage_table(ranges, 6, static_cast<cudaStream_t>(stream), &tb)) return EMA_ERR_CUDA;
    if (workspace && need > 0 && workspace_bytes >= need && aligned16(h) && aligned16(dh) && aligned16(dS) &&
        (reinterpret_cast<uintptr_t>(workspace) & 3u) == 0 && (T / 4 + 31) / 32 <= 65535 && B * C < (1ll << 31) * 128) {
        const int n_warps = static_cast<int>((T / 4 + 31) / 32);
        auto st = static_cast<cudaStream_t>(stream);
        dim3 grid(static_cast<unsigned>(B), static_cast<unsigned>(n_warps));
        state_passing_bwd_vec_kernel<<<grid, 32, 0, st>>>(
            make_ptr(reinterpret_cast<const float4 *>(h), tb, 370), make_ptr(cs_last, tb, 371), cl_sb, cl_sc,
            make_ptr(reinterpret_cast<const float4 *>(dh), tb, 372), make_ptr(reinterpret_cast<float4 *>(dS), tb, 373),
            make_ptr(static_cast<float *>(workspace), tb, 374), C, T / 4, n_warps);
        state_passing_bwd_sum_kernel<<<cdiv(B * C, 128), 128, 0, st>>>(
            make_ptr(static_cast<const float *>(workspace), tb, 375), make_ptr(cs_last, tb, 371), cl_sb, cl_sc,
            make_ptr(ddA_last, tb, 376), B, C, n_warps);
        return check_launch();
    }
    EMA_REQUIRE(T <= 16 * 1024, EMA_ERR_UNSUPPORTED);
    int threads = static_cast<int>(((T + 15) / 16 + 31) / 32 * 32);
    if (threads < 32) threads = 32;
    state_passing_bwd_kernel<<<static_cast<unsigned>(B), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        make_ptr(h, tb, 370), make_ptr(cs_last, tb, 371), cl_sb, cl_sc, make_ptr(dh, tb, 372), make_ptr(dS, tb, 373),
        make_ptr(ddA_last, tb, 376), C, T);
    return check_launch();
}

extern "C" int ema_b200_bwd_dx(const float *cs, const void *dout, const float *dS, void *dx, int dtype,
                               int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(cs && dout && dS && dx, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{dx, static_cast<size_t>(B * L * T) * esize(dtype)}, {dout, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {cs, static_cast<size_t>(B * C * Q) * 4}, {dS, static_cast<size_t>(B * C * T) * 4}};
    if (!stage_table(ranges, 4, st, &tb)) return EMA_ERR_CUDA;
    if (recurrence_vec_ok(dout, dx, dS, dtype, T, Q)) return launch_recurrence_vec<true>(dout, cs, dS, dx, dtype, B, L, T, Q, C, st, tb);
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    EMA_STAGE_DISPATCH(dtype,
        (bwd_dx_kernel<float><<<grid, 128, 0, st>>>(make_ptr(cs, tb, 380), make_ptr(static_cast<const float *>(dout), tb, 381), make_ptr(dS, tb, 382), make_ptr(static_cast<float *>(dx), tb, 383), L, T, Q, C)),
        (bwd_dx_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(make_ptr(cs, tb, 380), make_ptr(static_cast<const __nv_bfloat16 *>(dout), tb, 381), make_ptr(dS, tb, 382), make_ptr(static_cast<__nv_bfloat16 *>(dx), tb, 383), L, T, Q, C)))
    return check_launch();
}

extern "C" int ema_b200_bwd_db(const void *X, const float *cs, const float *dS, float *ddA, int dtype,
                               int raw, int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(X && cs && dS && ddA, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    const int64_t total = B * C * Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{ddA, static_cast<size_t>(B * C * Q) * 4}, {X, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {cs, static_cast<size_t>(B * C * Q) * 4}, {dS, static_cast<size_t>(B * C * T) * 4}};
    if (!stage_table(ranges, 4, st, &tb)) return EMA_ERR_CUDA;
    EMA_STAGE_DISPATCH(dtype,
        (row_dot_kernel<float, 0><<<cdiv(total * 32, 256), 256, 0, st>>>(make_ptr(static_cast<const float *>(X), tb, 390), make_ptr(cs, tb, 391), make_ptr(dS, tb, 392), make_ptr(ddA, tb, 393), L, T, Q, C, total)),
        (row_dot_kernel<__nv_bfloat16, 0><<<cdiv(total * 32, 256), 256, 0, st>>>(make_ptr(static_cast<const __nv_bfloat16 *>(X), tb, 390), make_ptr(cs, tb, 391), make_ptr(dS, tb, 392), make_ptr(ddA, tb, 393), L, T, Q, C, total)))
    rc = check_launch();
    if (rc || raw) return rc;
    row_cumsum_kernel<<<cdiv(B * C * 32, 128), 128, 0, st>>>(make_ptr(ddA, tb, 394), B * C, Q);
    return check_launch();
}

extern "C" int ema_b200_bwd_dc(const float *h, const float *cs, const void *dout, float *ddA, int dtype,
                               int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(h && cs && dout && ddA, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    const int64_t total = B * C * Q;
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{ddA, static_cast<size_t>(B * C * Q) * 4}, {dout, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {cs, static_cast<size_t>(B * C * Q) * 4}, {h, static_cast<size_t>(B * C * T) * 4}};
    if (!stage_table(ranges, 4, st, &tb)) return EMA_ERR_CUDA;
    EMA_STAGE_DISPATCH(dtype,
        (row_dot_kernel<float, 1><<<cdiv(total * 32, 256), 256, 0, st>>>(make_ptr(static_cast<const float *>(dout), tb, 400), make_ptr(cs, tb, 401), make_ptr(h, tb, 402), make_ptr(ddA, tb, 403), L, T, Q, C, total)),
        (row_dot_kernel<__nv_bfloat16, 1><<<cdiv(total * 32, 256), 256, 0, st>>>(make_ptr(static_cast<const __nv_bfloat16 *>(dout), tb, 400), make_ptr(cs, tb, 401), make_ptr(h, tb, 402), make_ptr(ddA, tb, 403), L, T, Q, C, total)))
    return check_launch();
}

extern "C" int ema_b200_bwd_dacs(const void *X, const float *cs, const void *dout, float *ddA, int dtype,
                                 int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(X && cs && dout && ddA, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    // shared memory: acc[Q] + part[nwarps][Q] + yl[nwarps][Q][32]
    int nwarps = 4;
    while (nwarps > 1 && (static_cast<size_t>(Q) * (1 + nwarps + 32 * nwarps) * 4 > 200 * 1024 ||
                          static_cast<int64_t>(nwarps - 1) * 32 >= T))
        nwarps >>= 1;
    const size_t smem = static_cast<size_t>(Q) * (1 + nwarps + 32 * nwarps) * 4;
    EMA_REQUIRE(smem <= 200 * 1024, EMA_ERR_UNSUPPORTED);
    auto st = static_cast<cudaStream_t>(stream);
    BoundsTable *tb;
    const BoundsRange ranges[] = {{ddA, static_cast<size_t>(B * C * Q) * 4}, {X, static_cast<size_t>(B * L * T) * esize(dtype)},
                                  {dout, static_cast<size_t>(B * L * T) * esize(dtype)}, {cs, static_cast<size_t>(B * C * Q) * 4}};
    if (!stage_table(ranges, 4, st, &tb)) return EMA_ERR_CUDA;
    cudaError_t e;
    if (dtype == EMA_F32) {
        e = cudaFuncSetAttribute(bwd_dacs_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
        bwd_dacs_kernel<float><<<static_cast<unsigned>(B * C), nwarps * 32, smem, st>>>(
            make_ptr(static_cast<const float *>(X), tb, 410), make_ptr(cs, tb, 411), make_ptr(static_cast<const float *>(dout), tb, 412),
            make_ptr(ddA, tb, 413), L, T, Q, C);
    } else if (dtype == EMA_BF16) {
        e = cudaFuncSetAttribute(bwd_dacs_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
        bwd_dacs_kernel<__nv_bfloat16><<<static_cast<unsigned>(B * C), nwarps * 32, smem, st>>>(
            make_ptr(static_cast<const __nv_bfloat16 *>(X), tb, 410), make_ptr(cs, tb, 411),
            make_ptr(static_cast<const __nv_bfloat16 *>(dout), tb, 412), make_ptr(ddA, tb, 413), L, T, Q, C);
    } else {
        return EMA_ERR_UNSUPPORTED;
    }
    return check_launch();
}
