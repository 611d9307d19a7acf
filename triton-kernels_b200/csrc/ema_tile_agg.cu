// Per-tile aggregates of the scan, computed for all tiles at once (no dependence between tiles).
//
// The fused tensor-core kernels walk the 128-step tiles of a work item one after the other, which leaves SMs idle
// when a problem has fewer work items than the GPU has SMs.  The reference's own pipeline shows the way out: a
// chunk-state pass that is parallel over chunks (kernels/ema_kernels/ema_state_fwd.py:54-125,
// S_c = sum_q exp(cs_last - cs_q) u_q), a cheap serial carry over the chunk states
// (kernels/ema_kernels/ema_state_pass.py:100-120), and the chunk scan, again parallel over chunks
// (kernels/ema_kernels/ema_scan_fwd.py:169-170); the backward mirrors it with
// dh_c = sum_q exp(cs_q) dy_q (kernels/ema_kernels_bwd/ema_scan_bwd.py:39-110) and the reverse carry
// (kernels/ema_kernels_bwd/ema_state_passing_bwd_dstates.py:60-98).
//
// The kernel below is that first pass at the tile size of the fused kernels.  For every (scan row, tile k):
//   forward  (MODE 0)  S_k[c] = sum_q w_q x[q, c],   w_q = p_q prod_{j=q+1..end} a_j,   P_k = prod_{j in tile} a_j
//                      so that the state after the tile is  h_{k+1} = P_k h_k + S_k
//   adjoint  (MODE 1)  G_k[c] = sum_q v_q dy[q, c],  v_q = prod_{j=first+1..q} a_j,     F_k = prod_{j=first+1..first+128} a_j
//                      so that the adjoint at the tile's first step is  lambda_first(k) = G_k + F_k lambda_first(k+1)
// (steps past L are identity steps: a = 1, x = dy = 0).  The fused kernels then start any tile of an item from the fold
// of the aggregates before (after) it, which cuts an item into pieces that run on different SMs without waiting for
// one another.  One pass over x (or dy): HBM-bound, and the tensor it read is still in L2 for the scan when it fits.
#include "ema_common.cuh"

namespace ema {
namespace {

constexpr int kAggThreads = 256;
constexpr int kAggSteps = 128;                 // = the fused kernels' tile
constexpr int kAggChannels = 256;              // channels per thread block: 32 lanes x 8 bf16 (one 16-byte load)
constexpr int kAggGroups = kAggThreads / 32;   // step groups (warps): warp g handles steps g, g + 8, ...

struct AggParams {
    const __nv_bfloat16 *src;   // x (MODE 0) or dy (MODE 1), [b, L, h, d] with element strides sb, sl, sh
    const float *decay;
    float *vec;                 // [rows, n_tiles, d]
    float *fac;                 // [rows, n_tiles]
    int64_t b, L, h, d;
    int64_t sb, sl, sh;
    int64_t a_sb, a_sl, a_sh;
    int decay_mode, convention;
    int n_tiles, n_cgroups;
    BoundsTable *bounds;   // bounds-checking build only
};

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int MODE>
__global__ void __launch_bounds__(kAggThreads) tile_aggregate_kernel(const AggParams p) {
    __shared__ float w_sm[kAggSteps];
    __shared__ float cs_sm[kAggSteps];
    __shared__ float warp_tot[4];
    __shared__ float red[kAggGroups][kAggChannels];
    grid_dependents_launch();   // (see ema_common.cuh: this kernel may have been scheduled before its predecessor ended)
    grid_dependency_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t blk = blockIdx.x;
    const int cg = static_cast<int>(blk % p.n_cgroups);
    const int k = static_cast<int>((blk / p.n_cgroups) % p.n_tiles);
    const int64_t row = blk / p.n_cgroups / p.n_tiles;
    const int64_t bi = row / p.h, hi = row % p.h;
    const bool per_step = p.decay_mode == EMA_DECAY_PER_STEP;
    const int conv = p.convention;
    const int64_t t0 = static_cast<int64_t>(k) * kAggSteps;
    const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
    // log2 of a step's decay, clamped like the fused kernels' (a decay of exactly 0 stays finite)
    auto log2_decay = [&](float v) { return fmaxf(conv ? v * 1.4426950408889634f : __log2f(v), -160.f); };
    const float ident = conv ? 0.f : 1.f;

    // ---- this thread's 16 rows of the tile (lane -> 8 channels, warp -> every 8th step), requested before the weights
    // are worked out so that the memory round trip overlaps the scan below.  Rows past L re-read the last row and are
    // discarded: an unconditional load is what lets all of them be in flight at once.
    const int64_t c = static_cast<int64_t>(cg) * kAggChannels + lane * 8;
    const bool c_ok = c < p.d;   // d is a multiple of 8 on this path
    const __nv_bfloat16 *base = p.src + bi * p.sb + hi * p.sh + c;
    uint4 raw[16];
    if (c_ok) {
        const int64_t t_last = p.L - 1;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int64_t t = t0 + warp + kAggGroups * i;
            raw[i] = __ldg(reinterpret_cast<const uint4 *>(EMA_ATN(p, base + (t < p.L ? t : t_last) * p.sl, 200, 16)));
        }
    }

    // ---- the tile's weights: inclusive scan of log2 a over 128 steps (threads 0-127)
    float v = ident, cs = 0.f;
    if (tid < kAggSteps) {
        const int64_t t = t0 + tid;
        if (t < p.L) v = *EMA_AT(p, per_step ? arow + t * p.a_sl : arow, 201);
        cs = log2_decay(v);
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, cs, o);
            if (lane >= o) cs += n;
        }
        if (lane == 31) warp_tot[warp] = cs;
    }
    __syncthreads();
    if (tid < kAggSteps) {
#pragma unroll
        for (int i = 0; i < 3; ++i)
            if (i < warp) cs += warp_tot[i];
        cs_sm[tid] = cs;
    }
    __syncthreads();
    if (tid < kAggSteps) {
        const float total = cs_sm[kAggSteps - 1], first = cs_sm[0];
        const bool valid = t0 + tid < p.L;
        float w;
        if (MODE == 0) w = (conv ? 1.f : 1.f - v) * ex2f(total - cs);   // p_q prod_{j > q} a_j
        else w = ex2f(cs - first);                                       // prod_{first < j <= q} a_j
        w_sm[tid] = valid ? w : 0.f;
        if (tid == 0 && cg == 0) {
            float f = total;
            if (MODE == 1) {
                // the step after the tile (identity past L) closes the product handed to the tile on the left
                const int64_t te = t0 + kAggSteps;
                float ve = ident;
                if (te < p.L) ve = *EMA_AT(p, per_step ? arow + te * p.a_sl : arow, 202);
                f = total - first + log2_decay(ve);
            }
            *EMA_AT(p, p.fac + row * p.n_tiles + k, 203) = ex2f(f);
        }
    }
    __syncthreads();

    // ---- weighted column sums
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (c_ok) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int q = warp + kAggGroups * i;
            const float w = w_sm[q];   // 0 for steps past L
            float f[8];
            unpack<__nv_bfloat16, 8>(raw[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, f[e], acc[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) red[warp][lane * 8 + e] = acc[e];
    __syncthreads();
    // fixed-order sum over the step groups; thread -> channel (coalesced store)
    const int64_t cc = static_cast<int64_t>(cg) * kAggChannels + tid;
    if (cc < p.d) {
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < kAggGroups; ++g) s += red[g][tid];
        *EMA_AT(p, p.vec + (row * p.n_tiles + k) * p.d + cc, 204) = s;
    }
}

}  // namespace

// bytes of one aggregate buffer: [rows, n_tiles, d] vectors followed by [rows, n_tiles] factors (256-byte rounded)
size_t tile_aggregate_bytes(int64_t rows, int64_t L, int64_t d) {
    const int64_t n_tiles = (L + kAggSteps - 1) / kAggSteps;
    const size_t n = static_cast<size_t>(rows) * n_tiles * (d + 1) * sizeof(float);
    return (n + 255) / 256 * 256;
}

// adjoint == 0: aggregates of x for the forward scan; adjoint != 0: of dy for the reverse scan
int launch_tile_aggregates(const FusedParams &fp, int adjoint, float *buf, cudaStream_t stream) {
    AggParams p;
    const int64_t rows = fp.b * fp.h;
    p.n_tiles = static_cast<int>((fp.L + kAggSteps - 1) / kAggSteps);
    p.n_cgroups = static_cast<int>((fp.d + kAggChannels - 1) / kAggChannels);
    p.vec = buf;
    p.fac = buf + rows * p.n_tiles * fp.d;
    p.decay = fp.decay;
    p.b = fp.b; p.L = fp.L; p.h = fp.h; p.d = fp.d;
    p.a_sb = fp.a_sb; p.a_sl = fp.a_sl; p.a_sh = fp.a_sh;
    p.decay_mode = fp.decay_mode; p.convention = fp.convention;
    p.bounds = fp.bounds;
    const int64_t blocks = rows * p.n_tiles * p.n_cgroups;
    if (blocks <= 0) return EMA_OK;
    if (blocks >= (1ll << 31)) return EMA_ERR_UNSUPPORTED;
    if (!adjoint) {
        p.src = static_cast<const __nv_bfloat16 *>(fp.x);
        p.sb = fp.x_sb; p.sl = fp.x_sl; p.sh = fp.x_sh;
        const cudaError_t e = launch_overlapped(tile_aggregate_kernel<0>, dim3(static_cast<unsigned>(blocks)),
                                                dim3(kAggThreads), 0, stream, p);
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    } else {
        p.src = static_cast<const __nv_bfloat16 *>(fp.dy);
        p.sb = fp.g_sb; p.sl = fp.g_sl; p.sh = fp.g_sh;
        const cudaError_t e = launch_overlapped(tile_aggregate_kernel<1>, dim3(static_cast<unsigned>(blocks)),
                                                dim3(kAggThreads), 0, stream, p);
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    }
    return check_launch();
}

}  // namespace ema
