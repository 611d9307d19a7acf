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
__global__ void chunk_cumsum_kernel(const float *__restrict__ A, int64_t A_sb, int64_t A_sl,
                                    float *__restrict__ cs, int64_t B, int64_t L, int Q, int64_t C) {
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
__global__ void chunk_state_kernel(const T *__restrict__ X, const float *__restrict__ cs,
                                   float *__restrict__ S, int64_t L, int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const float *csr = cs + bc * Q;
    const float last = csr[lim - 1];
    const T *xr = X + (b * L + c * Q) * Tn + t;
    float acc = 0.f;
    for (int q = 0; q < lim; ++q)
        acc = fmaf(expf(fminf(last - csr[q], 0.f)), to_f32<T>(xr[static_cast<int64_t>(q) * Tn]), acc);
    S[bc * Tn + t] = acc;
}

// out[b,c,:] = state at the start of chunk c; final[b,:] = state after the last chunk.
__global__ void state_passing_fwd_kernel(const float *__restrict__ S, const float *__restrict__ cl,
                                         int64_t cl_sb, int64_t cl_sc, float *__restrict__ out,
                                         float *__restrict__ fin, int64_t C, int64_t Tn) {
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
__global__ void chunk_scan_kernel(const T *__restrict__ X, const float *__restrict__ cs,
                                  const float *__restrict__ h, T *__restrict__ out, int64_t L,
                                  int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const float *csr = cs + bc * Q;
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
__global__ void bwd_dstates_kernel(const float *__restrict__ cs, const T *__restrict__ dout,
                                   float *__restrict__ dh, int64_t L, int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const float *csr = cs + bc * Q;
    const T *gr = dout + (b * L + c * Q) * Tn + t;
    float acc = 0.f;
    for (int q = 0; q < lim; ++q)
        acc = fmaf(expf(csr[q]), to_f32<T>(gr[static_cast<int64_t>(q) * Tn]), acc);
    dh[bc * Tn + t] = acc;
}

// Reverse carry of the adjoint over chunks.  One CTA per batch row; threads stride over T.
// dS[c] = adjoint of chunk c's local state; ddA_last[c] = exp(cs_last_c) <h_c, dS[c]>, 0 for c = 0.
__global__ void state_passing_bwd_kernel(const float *__restrict__ h, const float *__restrict__ cl,
                                         int64_t cl_sb, int64_t cl_sc, const float *__restrict__ dh,
                                         float *__restrict__ dS, float *__restrict__ ddA, int64_t C,
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
__global__ void bwd_dx_kernel(const float *__restrict__ cs, const T *__restrict__ dout,
                              const float *__restrict__ dS, T *__restrict__ dx, int64_t L,
                              int64_t Tn, int Q, int64_t C) {
    const int64_t bc = blockIdx.x;
    const int64_t b = bc / C, c = bc % C;
    const int64_t t = static_cast<int64_t>(blockIdx.y) * blockDim.x + threadIdx.x;
    if (t >= Tn) return;
    const int lim = chunk_limit(L, Q, c);
    const float *csr = cs + bc * Q;
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
__global__ void row_dot_kernel(const T *__restrict__ rows, const float *__restrict__ cs,
                               const float *__restrict__ vec, float *__restrict__ out, int64_t L,
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
        const T *r = rows + (b * L + c * Q + m) * Tn;
        const float *v = vec + bc * Tn;
        for (int64_t t = lane; t < Tn; t += 32) acc = fmaf(to_f32<T>(r[t]), v[t], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
    if (lane != 0) return;
    const float *csr = cs + bc * Q;
    if (KIND == 0) {
        if (m == 0) out[bc * Q] = 0.f;
        if (m + 1 < Q)
            out[bc * Q + m + 1] = (m < lim - 1) ? acc * expf(fminf(csr[Q - 1] - csr[m], 0.f)) : 0.f;
    } else {
        out[bc * Q + m] = (m < lim) ? acc * expf(csr[m]) : 0.f;
    }
}

// in-place inclusive cumsum along the last axis of [rows, Q]; one warp per row
__global__ void row_cumsum_kernel(float *__restrict__ v, int64_t rows, int Q) {
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
__global__ void bwd_dacs_kernel(const T *__restrict__ X, const float *__restrict__ cs,
                                const T *__restrict__ dout, float *__restrict__ out, int64_t L,
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
    const float *csr = cs + bc * Q;
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

inline unsigned cdiv(int64_t a, int64_t b) { return static_cast<unsigned>((a + b - 1) / b); }

}  // namespace
}  // namespace ema

using namespace ema;

#define EMA_REQUIRE(cond, code) \
    do {                        \
        if (!(cond)) return (code); \
    } while (0)

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
    chunk_cumsum_kernel<<<cdiv(B * C * 32, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        A, A_sb, A_sl, cs, B, L, Q, C);
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
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    auto st = static_cast<cudaStream_t>(stream);
    EMA_STAGE_DISPATCH(dtype,
        (chunk_state_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float *>(X), cs, S, L, T, Q, C)),
        (chunk_state_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16 *>(X), cs, S, L, T, Q, C)))
    return check_launch();
}

extern "C" int ema_b200_state_passing_fwd(const float *S, const float *cs_last, int64_t cl_sb,
                                          int64_t cl_sc, float *out, float *final_states, int64_t B,
                                          int64_t C, int64_t T, void *stream) {
    EMA_REQUIRE(S && cs_last && out && final_states, EMA_ERR_BADARG);
    EMA_REQUIRE(B > 0 && C > 0 && T > 0, EMA_ERR_BADARG);
    dim3 grid(static_cast<unsigned>(B), cdiv(T, 128));
    state_passing_fwd_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        S, cs_last, cl_sb, cl_sc, out, final_states, C, T);
    return check_launch();
}

extern "C" int ema_b200_chunk_scan(const void *X, const float *cs, const float *h, void *out, int dtype,
                                   int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(X && cs && h && out, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    auto st = static_cast<cudaStream_t>(stream);
    EMA_STAGE_DISPATCH(dtype,
        (chunk_scan_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float *>(X), cs, h, static_cast<float *>(out), L, T, Q, C)),
        (chunk_scan_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16 *>(X), cs, h, static_cast<__nv_bfloat16 *>(out), L, T, Q, C)))
    return check_launch();
}

extern "C" int ema_b200_bwd_dstates(const float *cs, const void *dout, float *dh, int dtype, int64_t B,
                                    int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(cs && dout && dh, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    auto st = static_cast<cudaStream_t>(stream);
    EMA_STAGE_DISPATCH(dtype,
        (bwd_dstates_kernel<float><<<grid, 128, 0, st>>>(cs, static_cast<const float *>(dout), dh, L, T, Q, C)),
        (bwd_dstates_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(cs, static_cast<const __nv_bfloat16 *>(dout), dh, L, T, Q, C)))
    return check_launch();
}

extern "C" int ema_b200_state_passing_bwd(const float *h, const float *cs_last, int64_t cl_sb,
                                          int64_t cl_sc, const float *dh, float *dS, float *ddA_last,
                                          int64_t B, int64_t C, int64_t T, void *stream) {
    EMA_REQUIRE(h && cs_last && dh && dS && ddA_last, EMA_ERR_BADARG);
    EMA_REQUIRE(B > 0 && C > 0 && T > 0, EMA_ERR_BADARG);
    EMA_REQUIRE(T <= 16 * 1024, EMA_ERR_UNSUPPORTED);
    int threads = static_cast<int>(((T + 15) / 16 + 31) / 32 * 32);
    if (threads < 32) threads = 32;
    state_passing_bwd_kernel<<<static_cast<unsigned>(B), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        h, cs_last, cl_sb, cl_sc, dh, dS, ddA_last, C, T);
    return check_launch();
}

extern "C" int ema_b200_bwd_dx(const float *cs, const void *dout, const float *dS, void *dx, int dtype,
                               int64_t B, int64_t L, int64_t T, int Q, void *stream) {
    EMA_REQUIRE(cs && dout && dS && dx, EMA_ERR_BADARG);
    int rc = stage_dims_ok(B, L, T, Q);
    if (rc) return rc;
    const int64_t C = (L + Q - 1) / Q;
    dim3 grid(static_cast<unsigned>(B * C), cdiv(T, 128));
    auto st = static_cast<cudaStream_t>(stream);
    EMA_STAGE_DISPATCH(dtype,
        (bwd_dx_kernel<float><<<grid, 128, 0, st>>>(cs, static_cast<const float *>(dout), dS, static_cast<float *>(dx), L, T, Q, C)),
        (bwd_dx_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(cs, static_cast<const __nv_bfloat16 *>(dout), dS, static_cast<__nv_bfloat16 *>(dx), L, T, Q, C)))
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
    EMA_STAGE_DISPATCH(dtype,
        (row_dot_kernel<float, 0><<<cdiv(total * 32, 256), 256, 0, st>>>(static_cast<const float *>(X), cs, dS, ddA, L, T, Q, C, total)),
        (row_dot_kernel<__nv_bfloat16, 0><<<cdiv(total * 32, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(X), cs, dS, ddA, L, T, Q, C, total)))
    rc = check_launch();
    if (rc || raw) return rc;
    row_cumsum_kernel<<<cdiv(B * C * 32, 128), 128, 0, st>>>(ddA, B * C, Q);
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
    EMA_STAGE_DISPATCH(dtype,
        (row_dot_kernel<float, 1><<<cdiv(total * 32, 256), 256, 0, st>>>(static_cast<const float *>(dout), cs, h, ddA, L, T, Q, C, total)),
        (row_dot_kernel<__nv_bfloat16, 1><<<cdiv(total * 32, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(dout), cs, h, ddA, L, T, Q, C, total)))
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
    cudaError_t e;
    if (dtype == EMA_F32) {
        e = cudaFuncSetAttribute(bwd_dacs_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
        bwd_dacs_kernel<float><<<static_cast<unsigned>(B * C), nwarps * 32, smem, st>>>(
            static_cast<const float *>(X), cs, static_cast<const float *>(dout), ddA, L, T, Q, C);
    } else if (dtype == EMA_BF16) {
        e = cudaFuncSetAttribute(bwd_dacs_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
        bwd_dacs_kernel<__nv_bfloat16><<<static_cast<unsigned>(B * C), nwarps * 32, smem, st>>>(
            static_cast<const __nv_bfloat16 *>(X), cs, static_cast<const __nv_bfloat16 *>(dout), ddA, L, T, Q, C);
    } else {
        return EMA_ERR_UNSUPPORTED;
    }
    return check_launch();
}
