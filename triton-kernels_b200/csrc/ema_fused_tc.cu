// Fused EMA scan on the Blackwell tensor cores (bf16 in/out, fp32 accumulate and carries).
//
// Within a tile of 128 steps the scan is a dense contraction: with decays a_j and input weights p_k
//     y_m = sum_{k<=m} p_k (prod_{j=k+1..m} a_j) x_k  +  (prod_{j<=m} a_j) h
// i.e. Y = G X + E h^T with G a 128x128 lower-triangular matrix that depends on the decays only and is
// shared by all channels.  G is written to shared memory as bf16 (K-major, 128-byte swizzle), the x
// tile [128 steps x 64 channels] lands next to it by TMA exactly as the MMA wants its B operand
// (MN-major, 128-byte swizzle), tcgen05.mma accumulates Y in TMEM (fp32), and the epilogue warps add
// the carry term in fp32, hand the last row on as the next carry, and TMA-store bf16 y.
//
// One persistent CTA per SM walks its work items (scan row, 64-channel tile) and, inside an item, the
// tiles in sequence order.  Warp roles:  warp 0 TMA producer;  warp 1 MMA issuer (owns TMEM);
// warps 2-9 epilogue (a TMEM lane quadrant and one half of the 64 channels each);  warps 10-13 build G
// (once for a time-invariant decay, per tile otherwise, with running products: no exp, no division).
// Every wait on an mbarrier is bounded (ema_tc_common.cuh); after a timeout the roles run their
// loops to the end without waiting, the CTA tears down normally and the host sees EMA_ERR_TIMEOUT.
#include "ema_common.cuh"
#include "ema_tc_common.cuh"

namespace ema {
namespace tc {

constexpr int QT = 128;              // steps per tile = MMA M = MMA K extent
constexpr int DT = 64;               // channels per tile = MMA N
constexpr int kTileBytes = QT * DT * 2;
constexpr int kMatBytes = QT * QT * 2;
constexpr int kThreads = 448;      // 14 warps: TMA, MMA, 8 epilogue, 4 builders
constexpr int kEpiThread0 = 64;    // warps 2-9
constexpr int kEpiThreads = 256;
constexpr int kBuildThread0 = 320;  // warps 10-13
constexpr uint32_t kIdesc = make_idesc_bf16(QT, DT, 0, 1);

struct TcParams {
    const float *decay;
    float *chunk_states, *tile_states, *final_state, *log_decay_sum;
    const float *init_state;
    int64_t b, L, h, d;
    int64_t a_sb, a_sl, a_sh;
    int decay_mode, convention, chunk;
    int n_tiles;      // 128-step tiles
    int n_tiles64;    // saved states per row (64-step granularity, shared with the FMA path)
    int n_dtiles, n_items;
    int64_t n_chunks;
};

// named barriers (id 0 is __syncthreads)
__device__ __forceinline__ void bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Builder: thread r owns row r of a lower-triangular matrix.
//   a_sm[j], p_sm[j]: decay and input weight of step j of the tile (a = 1, p = 0 is never needed:
//   rows past the end multiply zero-filled x rows).
//   SHIFT = 0:  M[r,k] = p_k prod_{j=k+1..r} a_j,  k <= r          (forward matrix G)
//   SHIFT = 1:  M[r,k] = p_k prod_{j=k+1..r-1} a_j, k <= r-1;  M[r,r] = diag   (backward: y_{r-1} - x_r)
// Returns the product of a over all steps the row spans: prod_{j<=r} a_j (SHIFT 0) or prod_{j<r} a_j.
// The row is produced right to left in 8-element chunks, one 16-byte store per chunk.
// ---------------------------------------------------------------------------------------------
template <int SHIFT>
__device__ __forceinline__ float build_lower_row(uint8_t *mat, int r, const float *a_sm, const float *p_sm,
                                                 float diag) {
    const int top = r - SHIFT;  // highest k with a scan term
    float run = 1.f;
    // every thread visits the chunks in the same order, so a_sm / p_sm reads are warp broadcasts
    for (int c = QT / 8 - 1; c >= 0; --c) {
        if (c > (r >> 3)) continue;
        float v[8];
#pragma unroll
        for (int e = 7; e >= 0; --e) {
            const int k = c * 8 + e;
            float val = 0.f;
            if (k <= top) {
                val = p_sm[k] * run;
                run *= a_sm[k];
            } else if (SHIFT == 1 && k == r) {
                val = diag;
            }
            v[e] = val;
        }
        const uint4 q = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                   pack_bf16x2(v[6], v[7]));
        *reinterpret_cast<uint4 *>(mat + (c >> 3) * (QT * 128) + sw128_offset(r, c & 7)) = q;
    }
    return run;
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
constexpr int kFwdStages = 7;  // 7 x 16 KB of loads in flight per SM: HBM latency under load is ~3 us
constexpr int kFwdMatBufs = 2;
struct FwdSmem {
    static constexpr int mat = 0;
    static constexpr int x = mat + kFwdMatBufs * kMatBytes;
    static constexpr int ystage = x + kFwdStages * kTileBytes;
    static constexpr int h = ystage + 2 * kTileBytes;       // float[2][64]
    static constexpr int e = h + 2 * DT * 4;                 // float[4][128]
    static constexpr int a = e + 4 * QT * 4;                 // float[128]
    static constexpr int pw = a + QT * 4;                    // float[128]
    static constexpr int red = pw + QT * 4;                  // float[4]
    static constexpr int mid = red + 16;                     // float[2][64]: state after row 63
    static constexpr int bars = mid + 2 * DT * 4;            // uint64[...]
    static constexpr int n_bars = 2 * kFwdStages + 4 + 2 * kFwdMatBufs;
    static constexpr int tmem_slot = bars + n_bars * 8;
    static constexpr int abort_flag = tmem_slot + 4;
    static constexpr int total = abort_flag + 4;
};
constexpr int kFwdSmemBytes = FwdSmem::total + 1024;  // + slack for the manual 1024-byte alignment

__global__ void __launch_bounds__(kThreads, 1)
ema_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                  const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool per_step = p.decay_mode == EMA_DECAY_PER_STEP;
    const int conv = p.convention;
    const int L = static_cast<int>(p.L);

    float *h_sm = reinterpret_cast<float *>(smem + FwdSmem::h);
    float *e_sm = reinterpret_cast<float *>(smem + FwdSmem::e);
    float *a_sm = reinterpret_cast<float *>(smem + FwdSmem::a);
    float *p_sm = reinterpret_cast<float *>(smem + FwdSmem::pw);
    float *red_sm = reinterpret_cast<float *>(smem + FwdSmem::red);
    float *mid_sm = reinterpret_cast<float *>(smem + FwdSmem::mid);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + FwdSmem::abort_flag);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + FwdSmem::tmem_slot);
    auto bar = [&](int i) { return sbase + FwdSmem::bars + i * 8; };
    // barrier indices
    constexpr int B_FULL = 0, B_EMPTY = kFwdStages, B_ACC_FULL = 2 * kFwdStages, B_ACC_EMPTY = B_ACC_FULL + 2,
                  B_MAT_FULL = B_ACC_EMPTY + 2, B_MAT_EMPTY = B_MAT_FULL + kFwdMatBufs;

    if (tid == 0) {
        for (int i = 0; i < kFwdStages; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), kEpiThreads); }
        for (int i = 0; i < kFwdMatBufs; ++i) { mbar_init(bar(B_MAT_FULL + i), 128); mbar_init(bar(B_MAT_EMPTY + i), 1); }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_y);
    }
    // the matrices start as zeros; the builders only ever write the lower triangle
    for (int i = tid; i < kFwdMatBufs * kMatBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(smem + FwdSmem::mat)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 1) {
        tmem_alloc(sbase + FwdSmem::tmem_slot, 128);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t n_items = p.n_items;
    auto decay_a = [&](float v) { return conv ? expf(v) : v; };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x) {
                const int dtile = static_cast<int>(item % p.n_dtiles);
                const int64_t row = item / p.n_dtiles;
                const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
                for (int k = 0; k < p.n_tiles; ++k, ++it) {
                    const int s = it % kFwdStages;
                    const uint32_t ph = (it / kFwdStages) & 1;
                    if (!mbar_wait(bar(B_EMPTY + s), ph ^ 1, abort_flag, 1)) break;
                    mbar_expect_tx(bar(B_FULL + s), kTileBytes);
                    tma_load_4d(sbase + FwdSmem::x + s * kTileBytes, &tm_x, bar(B_FULL + s), dtile * DT, hi, k * QT, bi);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // A matrix is built per tile (per-step decay) or whenever the head changes (time-invariant
            // decay); the MMA issuer, the epilogue and the builders evaluate the same predicate, so they
            // agree on the build counter mt without talking to each other.
            uint32_t it = 0, mt = 0;
            int cur_head = -1, mb_cur = 0;
            for (int64_t item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x) {
                const int hi = static_cast<int>((item / p.n_dtiles) % p.h);
                for (int k = 0; k < p.n_tiles; ++k, ++it) {
                    const int s = it % kFwdStages;
                    const uint32_t ph = (it / kFwdStages) & 1;
                    const int acc = it & 1;
                    const uint32_t aph = (it >> 1) & 1;
                    if (per_step || hi != cur_head) {
                        // every MMA that read the previous head's matrix has been issued: release its buffer
                        if (!per_step && mt > 0) umma_commit(bar(B_MAT_EMPTY + ((mt - 1) % kFwdMatBufs)));
                        mb_cur = mt % kFwdMatBufs;
                        if (!mbar_wait(bar(B_MAT_FULL + mb_cur), (mt / kFwdMatBufs) & 1, abort_flag, 2)) break;
                        cur_head = hi;
                        ++mt;
                    }
                    if (!mbar_wait(bar(B_FULL + s), ph, abort_flag, 3)) break;
                    if (!mbar_wait(bar(B_ACC_EMPTY + acc), aph ^ 1, abort_flag, 4)) break;
                    tc_fence_after_sync();
                    const uint32_t a_base = sbase + FwdSmem::mat + mb_cur * kMatBytes;
                    const uint32_t b_base = sbase + FwdSmem::x + s * kTileBytes;
#pragma unroll
                    for (int kb = 0; kb < QT / 16; ++kb) {
                        const uint64_t ad = make_desc_sw128(a_base + (kb >> 2) * (QT * 128) + (kb & 3) * 32, 16, 1024);
                        const uint64_t bd = make_desc_sw128(b_base + kb * 2048, kTileBytes, 1024);
                        umma_bf16(tmem_base + acc * DT, ad, bd, kIdesc, kb > 0 ? 1u : 0u);
                    }
                    umma_commit(bar(B_EMPTY + s));
                    umma_commit(bar(B_ACC_FULL + acc));
                    if (per_step) umma_commit(bar(B_MAT_EMPTY + mb_cur));
                }
            }
        }
    } else if (tid < kBuildThread0) {
        // ---------------- epilogue ----------------
        // 8 warps: TMEM lane quadrant q = warp % 4 (hardware rule), column half = 0 for warps 2-5, 1 for 6-9.
        // Thread (q, lane, half) owns row m = 32 q + lane and channels [32 half, 32 half + 32) of the tile.
        const int q = warp & 3;
        const int half = (warp - kEpiThread0 / 32) >> 2;
        const int m = q * 32 + lane;
        const int cb = half * 32;
        const bool e0 = tid == kEpiThread0;
        uint32_t it = 0, mt = 0;
        int cur_head = -1;
        for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int dtile = static_cast<int>(item % p.n_dtiles);
            const int64_t row = item / p.n_dtiles;
            const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
            const int c0 = dtile * DT;
            if (m < DT && half == 0) {
                const bool ok = c0 + m < p.d;
                const float v = (p.init_state && ok) ? p.init_state[row * p.d + c0 + m] : 0.f;
                h_sm[(it & 1) * DT + m] = v;
                if (p.chunk_states && ok) p.chunk_states[(row * p.n_chunks) * p.d + c0 + m] = v;
            }
            bar_sync(1, kEpiThreads);
            for (int k = 0; k < p.n_tiles; ++k, ++it) {
                const int acc = it & 1, par = it & 1;
                const uint32_t aph = (it >> 1) & 1;
                const bool new_mat = per_step || hi != cur_head;
                if (new_mat) { cur_head = hi; ++mt; }
                mbar_wait(bar(B_ACC_FULL + acc), aph, abort_flag, 5);
                __syncwarp();  // the polling loop may leave the lanes diverged; tcgen05.ld is warp-collective
                tc_fence_after_sync();
                const float E = e_sm[((mt - 1) & 3) * QT + m];
                float y[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * DT + cb, y);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(bar(B_ACC_EMPTY + acc));

                const float *hin = h_sm + par * DT;
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    const float4 hv = *reinterpret_cast<const float4 *>(hin + cb + c);
                    y[c] = fmaf(E, hv.x, y[c]);
                    y[c + 1] = fmaf(E, hv.y, y[c + 1]);
                    y[c + 2] = fmaf(E, hv.z, y[c + 2]);
                    y[c + 3] = fmaf(E, hv.w, y[c + 3]);
                }
                const int t = k * QT + m;
                if (m == QT - 1) {  // the last row is the state handed to the next tile
                    float *hout = h_sm + (par ^ 1) * DT + cb;
#pragma unroll
                    for (int c = 0; c < 32; c += 4)
                        *reinterpret_cast<float4 *>(hout + c) = make_float4(y[c], y[c + 1], y[c + 2], y[c + 3]);
                }
                // saved states at 64-step granularity: the entering state is written straight from shared
                // memory (one coalesced line); the state after row 63 goes through shared memory so that 64
                // threads can write it the same way after the barrier
                if (p.tile_states) {
                    if (half == 0 && m < DT && c0 + m < p.d)
                        p.tile_states[(row * p.n_tiles64 + 2 * k) * p.d + c0 + m] = hin[m];
                    if (m == 63) {
                        float *mo = mid_sm + par * DT + cb;
#pragma unroll
                        for (int c = 0; c < 32; c += 4)
                            *reinterpret_cast<float4 *>(mo + c) = make_float4(y[c], y[c + 1], y[c + 2], y[c + 3]);
                    }
                }
                if (p.chunk_states && t + 1 < L && (t + 1) % p.chunk == 0) {
                    float *cs = p.chunk_states + (row * p.n_chunks + (t + 1) / p.chunk) * p.d + c0 + cb;
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (c0 + cb + c < p.d) cs[c] = y[c];
                }
                if (p.final_state && t == L - 1) {
                    float *fs = p.final_state + row * p.d + c0 + cb;
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (c0 + cb + c < p.d) fs[c] = y[c];
                }
                // bf16 half-row -> staging buffer in the TMA's 128-byte swizzle
                uint8_t *stg = smem + FwdSmem::ystage + (it & 1) * kTileBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 qv = make_uint4(pack_bf16x2(y[8 * j], y[8 * j + 1]), pack_bf16x2(y[8 * j + 2], y[8 * j + 3]),
                                                pack_bf16x2(y[8 * j + 4], y[8 * j + 5]), pack_bf16x2(y[8 * j + 6], y[8 * j + 7]));
                    *reinterpret_cast<uint4 *>(stg + sw128_offset(m, half * 4 + j)) = qv;
                }
                fence_proxy_async();
                if (e0) tma_store_wait_read<0>();  // the other staging buffer is free for the next tile
                bar_sync(1, kEpiThreads);
                if (e0) {
                    tma_store_4d(&tm_y, sbase + FwdSmem::ystage + (it & 1) * kTileBytes, c0, hi, k * QT, bi);
                    tma_store_commit();
                }
                // mid_sm[par] is rewritten two tiles later, i.e. after everybody has passed the next barrier
                if (p.tile_states && half == 0 && m < DT && c0 + m < p.d && 2 * k + 1 < p.n_tiles64)
                    p.tile_states[(row * p.n_tiles64 + 2 * k + 1) * p.d + c0 + m] = mid_sm[par * DT + m];
            }
        }
        if (e0) tma_store_wait_all();
    } else {
        // ---------------- matrix builders ----------------
        const int r = tid - kBuildThread0;
        uint32_t mt = 0;
        int cur_head = -1;
        for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int64_t row = item / p.n_dtiles;
            const int dtile = static_cast<int>(item % p.n_dtiles);
            const int64_t bi = row / p.h, hi = row % p.h;
            const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
            float logsum = 0.f;
            if (!per_step) {
                if (static_cast<int>(hi) != cur_head) {
                    cur_head = static_cast<int>(hi);
                    const float a = decay_a(arow[0]);
                    const int mb = mt % kFwdMatBufs;
                    bar_sync(2, 128);
                    a_sm[r] = a;
                    p_sm[r] = conv ? 1.f : 1.f - a;
                    bar_sync(2, 128);
                    mbar_wait(bar(B_MAT_EMPTY + mb), ((mt / kFwdMatBufs) & 1) ^ 1, abort_flag, 6);
                    const float E = build_lower_row<0>(smem + FwdSmem::mat + mb * kMatBytes, r, a_sm, p_sm, 0.f);
                    e_sm[(mt & 3) * QT + r] = E;
                    fence_proxy_async();
                    mbar_arrive(bar(B_MAT_FULL + mb));
                    ++mt;
                }
                if (p.log_decay_sum && r == 0 && dtile == 0)
                    p.log_decay_sum[row] = static_cast<float>(L) * logf(decay_a(arow[0]));
                continue;
            }
            float a_next = 1.f;
            {
                const int t = r;
                if (t < L) a_next = decay_a(arow[static_cast<int64_t>(t) * p.a_sl]);
            }
            for (int k = 0; k < p.n_tiles; ++k, ++mt) {
                const float a = a_next;
                if (k + 1 < p.n_tiles) {
                    const int t = (k + 1) * QT + r;
                    a_next = t < L ? decay_a(arow[static_cast<int64_t>(t) * p.a_sl]) : 1.f;
                }
                const int mb = mt % kFwdMatBufs;
                bar_sync(2, 128);  // everyone has finished reading the previous tile's a_sm / p_sm / red_sm
                a_sm[r] = a;
                p_sm[r] = conv ? 1.f : 1.f - a;
                if (p.log_decay_sum) {
                    float lg = logf(a);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) lg += __shfl_xor_sync(0xffffffffu, lg, o);
                    if (lane == 0) red_sm[warp - kBuildThread0 / 32] = lg;
                }
                bar_sync(2, 128);
                if (p.log_decay_sum && r == 0) logsum += (red_sm[0] + red_sm[1]) + (red_sm[2] + red_sm[3]);
                mbar_wait(bar(B_MAT_EMPTY + mb), ((mt / kFwdMatBufs) & 1) ^ 1, abort_flag, 7);
                const float E = build_lower_row<0>(smem + FwdSmem::mat + mb * kMatBytes, r, a_sm, p_sm, 0.f);
                e_sm[(mt & 3) * QT + r] = E;
                fence_proxy_async();
                mbar_arrive(bar(B_MAT_FULL + mb));
            }
            if (p.log_decay_sum && r == 0 && dtile == 0) p.log_decay_sum[row] = logsum;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // give copies that were still in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 128);
    }
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------
// Per tile (walked from the end of the sequence to its start), with h the saved state entering the tile
// and g the adjoint entering it from the right:
//     Z = A1 X  + Eprev h^T      Z_m = y_{m-1} - x_m  (north-star) or y_{m-1} (pre-scaled)
//     Lam = U dY + F g^T         Lam_m = lambda_m
// A1[m,k] = p_k prod_{j=k+1..m-1} a_j (k < m), A1[m,m] = -1 | 0;  U[m,k] = prod_{j=m+1..k} a_j (k >= m);
// Eprev_m = prod_{j<m} a_j;  F_m = prod_{j=m+1..128} a_j (a_128 = first decay of the next tile, 1 past L).
// Then dx_m = p_m Lam_m, ddecay_m = sum_c Lam_mc Z_mc (times a_m for the log-decay convention), and row 0
// of Lam is the adjoint handed to the previous tile.

// Upper-triangular row r of U, left to right from the diagonal; returns prod_{j=r+1..127} a_j.
__device__ __forceinline__ float build_upper_row(uint8_t *mat, int r, const float *a_sm) {
    float run = 1.f;
    for (int c = 0; c < QT / 8; ++c) {
        if (c < (r >> 3)) continue;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int k = c * 8 + e;
            float val = 0.f;
            if (k == r) {
                val = 1.f;
            } else if (k > r) {
                run *= a_sm[k];
                val = run;
            }
            v[e] = val;
        }
        const uint4 q = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                                   pack_bf16x2(v[6], v[7]));
        *reinterpret_cast<uint4 *>(mat + (c >> 3) * (QT * 128) + sw128_offset(r, c & 7)) = q;
    }
    return run;
}

struct TcBwdParams {
    const float *decay;
    const float *tile_states;
    const float *dfinal_state;
    float *dinit_state;
    float *da_partial;
    int64_t b, L, h, d;
    int64_t a_sb, a_sl, a_sh;
    int decay_mode, convention;
    int n_tiles, n_tiles64, n_dtiles, n_items;
    int64_t head_partial_offset;
};

constexpr int kBwdStages = 3;
struct BwdSmem {
    static constexpr int mat_a1 = 0;
    static constexpr int mat_u = mat_a1 + kMatBytes;
    static constexpr int xg = mat_u + kMatBytes;                       // stages of [x tile | dy tile]
    static constexpr int ostage = xg + kBwdStages * 2 * kTileBytes;    // dx staging, 2 buffers
    static constexpr int hs = ostage + 2 * kTileBytes;                 // float[2][64] saved state entering the tile
    static constexpr int g = hs + 2 * DT * 4;                          // float[2][64] adjoint carry
    static constexpr int rowsc = g + 2 * DT * 4;                       // float[4][4][128]: Eprev, F, p, a per build
    static constexpr int da = rowsc + 4 * 4 * QT * 4;                  // float[2][128] decay-gradient halves
    static constexpr int a = da + 2 * QT * 4;                          // float[129]
    static constexpr int pw = a + (QT + 4) * 4;                        // float[128]
    static constexpr int bars = pw + QT * 4;
    static constexpr int n_bars = 2 * kBwdStages + 4 + 2;
    static constexpr int tmem_slot = bars + n_bars * 8;
    static constexpr int abort_flag = tmem_slot + 4;
    static constexpr int total = abort_flag + 4;
};
constexpr int kBwdSmemBytes = BwdSmem::total + 1024;
static_assert(kBwdSmemBytes <= 227 * 1024, "backward shared memory exceeds the per-CTA limit");

__global__ void __launch_bounds__(kThreads, 1)
ema_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_g,
                  const __grid_constant__ CUtensorMap tm_o, const TcBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool per_step = p.decay_mode == EMA_DECAY_PER_STEP;
    const int conv = p.convention;
    const int L = static_cast<int>(p.L);

    float *hs_sm = reinterpret_cast<float *>(smem + BwdSmem::hs);
    float *g_sm = reinterpret_cast<float *>(smem + BwdSmem::g);
    float *rowsc = reinterpret_cast<float *>(smem + BwdSmem::rowsc);
    float *da_sm = reinterpret_cast<float *>(smem + BwdSmem::da);
    float *a_sm = reinterpret_cast<float *>(smem + BwdSmem::a);
    float *p_sm = reinterpret_cast<float *>(smem + BwdSmem::pw);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + BwdSmem::abort_flag);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + BwdSmem::tmem_slot);
    auto bar = [&](int i) { return sbase + BwdSmem::bars + i * 8; };
    constexpr int B_FULL = 0, B_EMPTY = kBwdStages, B_ACC_FULL = 2 * kBwdStages, B_ACC_EMPTY = B_ACC_FULL + 2,
                  B_MAT_FULL = B_ACC_EMPTY + 2, B_MAT_EMPTY = B_MAT_FULL + 1;
    constexpr uint32_t kTmemCols = 256;  // 2 stages x (Z | Lam) x 64 columns

    if (tid == 0) {
        for (int i = 0; i < kBwdStages; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), kEpiThreads); }
        mbar_init(bar(B_MAT_FULL), 128);
        mbar_init(bar(B_MAT_EMPTY), 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_g);
        prefetch_tmap(&tm_o);
    }
    for (int i = tid; i < 2 * kMatBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(smem + BwdSmem::mat_a1)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 1) {
        tmem_alloc(sbase + BwdSmem::tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t n_items = p.n_items;
    auto decay_a = [&](float v) { return conv ? expf(v) : v; };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            for (int64_t item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x) {
                const int dtile = static_cast<int>(item % p.n_dtiles);
                const int64_t row = item / p.n_dtiles;
                const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
                for (int k = p.n_tiles - 1; k >= 0; --k, ++it) {
                    const int s = it % kBwdStages;
                    const uint32_t ph = (it / kBwdStages) & 1;
                    if (!mbar_wait(bar(B_EMPTY + s), ph ^ 1, abort_flag, 11)) break;
                    mbar_expect_tx(bar(B_FULL + s), 2 * kTileBytes);
                    const uint32_t dst = sbase + BwdSmem::xg + s * 2 * kTileBytes;
                    tma_load_4d(dst, &tm_x, bar(B_FULL + s), dtile * DT, hi, k * QT, bi);
                    tma_load_4d(dst + kTileBytes, &tm_g, bar(B_FULL + s), dtile * DT, hi, k * QT, bi);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, mt = 0;
            int cur_head = -1;
            for (int64_t item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x) {
                const int hi = static_cast<int>((item / p.n_dtiles) % p.h);
                for (int k = p.n_tiles - 1; k >= 0; --k, ++it) {
                    const int s = it % kBwdStages;
                    const uint32_t ph = (it / kBwdStages) & 1;
                    const int acc = it & 1;
                    const uint32_t aph = (it >> 1) & 1;
                    const bool new_mat = per_step || hi != cur_head;
                    if (new_mat) {
                        // single matrix buffer: hand it back to the builders once the MMAs issued so far are done
                        if (!per_step && mt > 0) umma_commit(bar(B_MAT_EMPTY));
                        if (!mbar_wait(bar(B_MAT_FULL), mt & 1, abort_flag, 12)) break;
                        cur_head = hi;
                        ++mt;
                    }
                    if (!mbar_wait(bar(B_FULL + s), ph, abort_flag, 13)) break;
                    if (!mbar_wait(bar(B_ACC_EMPTY + acc), aph ^ 1, abort_flag, 14)) break;
                    tc_fence_after_sync();
                    const uint32_t x_base = sbase + BwdSmem::xg + s * 2 * kTileBytes;
                    const uint32_t d_z = tmem_base + acc * 2 * DT, d_l = d_z + DT;
#pragma unroll
                    for (int kb = 0; kb < QT / 16; ++kb) {
                        const uint32_t koff = (kb >> 2) * (QT * 128) + (kb & 3) * 32;
                        umma_bf16(d_z, make_desc_sw128(sbase + BwdSmem::mat_a1 + koff, 16, 1024),
                                  make_desc_sw128(x_base + kb * 2048, kTileBytes, 1024), kIdesc, kb > 0 ? 1u : 0u);
                    }
#pragma unroll
                    for (int kb = 0; kb < QT / 16; ++kb) {
                        const uint32_t koff = (kb >> 2) * (QT * 128) + (kb & 3) * 32;
                        umma_bf16(d_l, make_desc_sw128(sbase + BwdSmem::mat_u + koff, 16, 1024),
                                  make_desc_sw128(x_base + kTileBytes + kb * 2048, kTileBytes, 1024), kIdesc,
                                  kb > 0 ? 1u : 0u);
                    }
                    umma_commit(bar(B_EMPTY + s));
                    umma_commit(bar(B_ACC_FULL + acc));
                    if (per_step) umma_commit(bar(B_MAT_EMPTY));
                }
            }
        }
    } else if (tid < kBuildThread0) {
        // ---------------- epilogue ----------------
        // thread (q, lane, half): row m = 32 q + lane, channels [32 half, 32 half + 32) of the tile
        const int q = warp & 3;
        const int half = (warp - kEpiThread0 / 32) >> 2;
        const int m = q * 32 + lane;
        const int cb = half * 32;
        const bool e0 = tid == kEpiThread0;
        uint32_t it = 0, mt = 0;
        int cur_head = -1;
        for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int dtile = static_cast<int>(item % p.n_dtiles);
            const int64_t row = item / p.n_dtiles;
            const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
            const int c0 = dtile * DT;
            const int64_t blk = row * p.n_dtiles + dtile;
            const bool loader = half == 0 && m < DT;         // these 64 threads move per-channel vectors
            const bool ch_ok = loader && c0 + m < p.d;
            // saved state of the first (rightmost) tile and the adjoint entering the sequence from the right
            float hs_next = 0.f;
            if (loader) {
                hs_sm[(it & 1) * DT + m] =
                    ch_ok ? p.tile_states[(row * p.n_tiles64 + 2 * (p.n_tiles - 1)) * p.d + c0 + m] : 0.f;
                g_sm[(it & 1) * DT + m] = (p.dfinal_state && ch_ok) ? p.dfinal_state[row * p.d + c0 + m] : 0.f;
            }
            bar_sync(1, kEpiThreads);
            for (int k = p.n_tiles - 1; k >= 0; --k, ++it) {
                const int acc = it & 1, par = it & 1;
                const uint32_t aph = (it >> 1) & 1;
                if (per_step || hi != cur_head) { cur_head = hi; ++mt; }
                // prefetch the saved state of the next tile to the left while this one is being finished
                if (loader && k > 0)
                    hs_next = ch_ok ? p.tile_states[(row * p.n_tiles64 + 2 * (k - 1)) * p.d + c0 + m] : 0.f;
                mbar_wait(bar(B_ACC_FULL + acc), aph, abort_flag, 15);
                __syncwarp();
                tc_fence_after_sync();
                const float *rs = rowsc + ((mt - 1) & 3) * 4 * QT;
                const float Eprev = rs[m], a_m = rs[3 * QT + m], p_m = rs[2 * QT + m];
                // F: a time-invariant decay uses one Toeplitz table; the rightmost tile of the sequence stops at
                // step L-1, where the adjoint entering from the right applies undamped
                float F = rs[QT + m];
                if (!per_step && k == p.n_tiles - 1) {
                    const int lim = L - k * QT;  // valid rows in this tile
                    float f = 1.f;
                    for (int j = m + 1; j < lim; ++j) f *= a_m;
                    F = f;
                }
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 2 * DT + cb;
                float z[32], lam[32];
                tmem_ld32(taddr, z);
                tmem_ld32(taddr + DT, lam);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(bar(B_ACC_EMPTY + acc));

                const float *hin = hs_sm + par * DT + cb;
                const float *gin = g_sm + par * DT + cb;
                const int t = k * QT + m;
                float dacc = 0.f;
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    const float4 hv = *reinterpret_cast<const float4 *>(hin + c);
                    const float4 gv = *reinterpret_cast<const float4 *>(gin + c);
                    z[c] = fmaf(Eprev, hv.x, z[c]);         lam[c] = fmaf(F, gv.x, lam[c]);
                    z[c + 1] = fmaf(Eprev, hv.y, z[c + 1]); lam[c + 1] = fmaf(F, gv.y, lam[c + 1]);
                    z[c + 2] = fmaf(Eprev, hv.z, z[c + 2]); lam[c + 2] = fmaf(F, gv.z, lam[c + 2]);
                    z[c + 3] = fmaf(Eprev, hv.w, z[c + 3]); lam[c + 3] = fmaf(F, gv.w, lam[c + 3]);
                }
#pragma unroll
                for (int c = 0; c < 32; ++c) dacc = fmaf(lam[c], z[c], dacc);
                if (m == 0) {  // row 0 of the adjoint is what the tile to the left receives
                    float *gout = g_sm + (par ^ 1) * DT + cb;
#pragma unroll
                    for (int c = 0; c < 32; c += 4)
                        *reinterpret_cast<float4 *>(gout + c) = make_float4(lam[c], lam[c + 1], lam[c + 2], lam[c + 3]);
                    if (k == 0 && p.dinit_state) {
                        float *di = p.dinit_state + row * p.d + c0 + cb;
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (c0 + cb + c < p.d) di[c] = a_m * lam[c];
                    }
                }
                uint8_t *stg = smem + BwdSmem::ostage + (it & 1) * kTileBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 qv = make_uint4(pack_bf16x2(p_m * lam[8 * j], p_m * lam[8 * j + 1]),
                                                pack_bf16x2(p_m * lam[8 * j + 2], p_m * lam[8 * j + 3]),
                                                pack_bf16x2(p_m * lam[8 * j + 4], p_m * lam[8 * j + 5]),
                                                pack_bf16x2(p_m * lam[8 * j + 6], p_m * lam[8 * j + 7]));
                    *reinterpret_cast<uint4 *>(stg + sw128_offset(m, half * 4 + j)) = qv;
                }
                if (conv) dacc *= a_m;
                if (t >= L) dacc = 0.f;
                if (per_step) {
                    // the two column halves of a row meet in shared memory; half 0 writes the sum after the barrier
                    if (half == 1) da_sm[par * QT + m] = dacc;
                } else {
                    float wsum = dacc;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
                    const int k64 = 2 * k + (q >> 1);
                    if (lane == 0 && k64 < p.n_tiles64)
                        p.da_partial[p.head_partial_offset + (blk * p.n_tiles64 + k64) * 4 + (q & 1) * 2 + half] = wsum;
                }
                if (loader) hs_sm[(par ^ 1) * DT + m] = hs_next;
                fence_proxy_async();
                if (e0) tma_store_wait_read<0>();
                bar_sync(1, kEpiThreads);
                if (e0) {
                    tma_store_4d(&tm_o, sbase + BwdSmem::ostage + (it & 1) * kTileBytes, c0, hi, k * QT, bi);
                    tma_store_commit();
                }
                // da_sm[par] is rewritten two tiles later, after everybody has passed the next barrier
                if (per_step && half == 0 && t < L)
                    p.da_partial[blk * (static_cast<int64_t>(p.n_tiles64) * 64) + t] = dacc + da_sm[par * QT + m];
            }
        }
        if (e0) tma_store_wait_all();
    } else {
        // ---------------- matrix builders ----------------
        const int r = tid - kBuildThread0;
        uint32_t mt = 0;
        int cur_head = -1;
        const float diag = conv ? 0.f : -1.f;
        auto build = [&](float a_r, float a_edge) {
            // a_r: decay of step r of the tile; a_edge: decay of the step right after the tile
            bar_sync(2, 128);
            a_sm[r] = a_r;
            p_sm[r] = conv ? 1.f : 1.f - a_r;
            if (r == 0) a_sm[QT] = a_edge;
            bar_sync(2, 128);
            mbar_wait(bar(B_MAT_EMPTY), (mt & 1) ^ 1, abort_flag, 16);
            const float Eprev = build_lower_row<1>(smem + BwdSmem::mat_a1, r, a_sm, p_sm, diag);
            const float Fr = build_upper_row(smem + BwdSmem::mat_u, r, a_sm) * a_sm[QT];
            float *rs = rowsc + (mt & 3) * 4 * QT;
            rs[r] = Eprev;
            rs[QT + r] = Fr;
            rs[2 * QT + r] = p_sm[r];
            rs[3 * QT + r] = a_r;
            fence_proxy_async();
            mbar_arrive(bar(B_MAT_FULL));
            ++mt;
        };
        for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int64_t row = item / p.n_dtiles;
            const int64_t bi = row / p.h, hi = row % p.h;
            const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
            if (!per_step) {
                if (static_cast<int>(hi) != cur_head) {
                    cur_head = static_cast<int>(hi);
                    const float a = decay_a(arow[0]);
                    build(a, a);
                }
                continue;
            }
            auto load_a = [&](int t) { return (t >= 0 && t < L) ? decay_a(arow[static_cast<int64_t>(t) * p.a_sl]) : 1.f; };
            float a_next = load_a((p.n_tiles - 1) * QT + r);
            float edge_next = 1.f;  // decay of step n_tiles*128 >= L
            for (int k = p.n_tiles - 1; k >= 0; --k) {
                const float a = a_next, edge = edge_next;
                if (k > 0) {
                    a_next = load_a((k - 1) * QT + r);
                    edge_next = load_a(k * QT);
                }
                build(a, edge);
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace tc

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// bf16 tensor [b, L, h, d] with element strides (sb, sl, sh), box = [64 channels, 1, 128 steps, 1],
// 128-byte swizzle; out-of-range parts of a box read as zero and are not written.
int make_tmap(CUtensorMap *tm, const void *base, int64_t b, int64_t L, int64_t h, int64_t d, int64_t sb,
              int64_t sl, int64_t sh) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return EMA_ERR_CUDA;
    // a dimension of extent 1 may carry any stride; give it a legal one
    if (h == 1) sh = d;
    if (L == 1) sl = h * d;
    if (b == 1) sb = L * sl;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(L),
                                static_cast<cuuint64_t>(b)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(sh) * 2, static_cast<cuuint64_t>(sl) * 2,
                                   static_cast<cuuint64_t>(sb) * 2};
    const cuuint32_t box[4] = {tc::DT, 1, tc::QT, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? EMA_OK : EMA_ERR_UNSUPPORTED;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

}  // namespace

// Can the tensor-core path take a bf16 tensor with these strides?  TMA wants a 16-byte aligned base
// and 16-byte multiples for every stride.
bool tc_tensor_ok(const void *base, int64_t d, int64_t sb, int64_t sl, int64_t sh, int64_t b, int64_t L, int64_t h) {
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || d % 8 != 0) return false;
    if (h > 1 && (sh % 8 != 0 || sh <= 0)) return false;
    if (L > 1 && (sl % 8 != 0 || sl <= 0)) return false;
    if (b > 1 && (sb % 8 != 0 || sb <= 0)) return false;
    return encode_fn() != nullptr;
}

int launch_fused_fwd_tc(const FusedParams &fp, cudaStream_t stream) {
    CUtensorMap tm_x, tm_y;
    int rc = make_tmap(&tm_x, fp.x, fp.b, fp.L, fp.h, fp.d, fp.x_sb, fp.x_sl, fp.x_sh);
    if (rc) return rc;
    rc = make_tmap(&tm_y, fp.out, fp.b, fp.L, fp.h, fp.d, fp.o_sb, fp.o_sl, fp.o_sh);
    if (rc) return rc;
    tc::TcParams p;
    p.decay = fp.decay;
    p.chunk_states = fp.chunk_states; p.tile_states = fp.tile_states; p.final_state = fp.final_state;
    p.log_decay_sum = fp.log_decay_sum; p.init_state = fp.init_state;
    p.b = fp.b; p.L = fp.L; p.h = fp.h; p.d = fp.d;
    p.a_sb = fp.a_sb; p.a_sl = fp.a_sl; p.a_sh = fp.a_sh;
    p.decay_mode = fp.decay_mode; p.convention = fp.convention; p.chunk = fp.chunk;
    p.n_tiles = static_cast<int>((fp.L + tc::QT - 1) / tc::QT);
    p.n_tiles64 = fp.n_tiles;
    p.n_dtiles = static_cast<int>((fp.d + tc::DT - 1) / tc::DT);
    p.n_items = static_cast<int>(fp.b * fp.h * p.n_dtiles);
    p.n_chunks = fp.n_chunks;
    const int sms = sm_count();
    const int rounds = (p.n_items + sms - 1) / sms;
    const int grid = (p.n_items + rounds - 1) / rounds;
    cudaError_t e = cudaFuncSetAttribute(tc::ema_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tc::kFwdSmemBytes);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    tc::ema_fwd_tc_kernel<<<grid, tc::kThreads, tc::kFwdSmemBytes, stream>>>(tm_x, tm_y, p);
    return check_launch();
}

int launch_fused_bwd_tc(const FusedParams &fp, cudaStream_t stream) {
    CUtensorMap tm_x, tm_g, tm_o;
    int rc = make_tmap(&tm_x, fp.x, fp.b, fp.L, fp.h, fp.d, fp.x_sb, fp.x_sl, fp.x_sh);
    if (rc) return rc;
    rc = make_tmap(&tm_g, fp.dy, fp.b, fp.L, fp.h, fp.d, fp.g_sb, fp.g_sl, fp.g_sh);
    if (rc) return rc;
    rc = make_tmap(&tm_o, fp.out, fp.b, fp.L, fp.h, fp.d, fp.o_sb, fp.o_sl, fp.o_sh);
    if (rc) return rc;
    tc::TcBwdParams p;
    p.decay = fp.decay;
    p.tile_states = fp.tile_states;
    p.dfinal_state = fp.dfinal_state;
    p.dinit_state = fp.dinit_state;
    p.da_partial = fp.da_partial;
    p.b = fp.b; p.L = fp.L; p.h = fp.h; p.d = fp.d;
    p.a_sb = fp.a_sb; p.a_sl = fp.a_sl; p.a_sh = fp.a_sh;
    p.decay_mode = fp.decay_mode; p.convention = fp.convention;
    p.n_tiles = static_cast<int>((fp.L + tc::QT - 1) / tc::QT);
    p.n_tiles64 = fp.n_tiles;
    p.n_dtiles = static_cast<int>((fp.d + tc::DT - 1) / tc::DT);
    p.n_items = static_cast<int>(fp.b * fp.h * p.n_dtiles);
    p.head_partial_offset = kHeadPartialOffset(fp.b * fp.h);
    const int sms = sm_count();
    const int rounds = (p.n_items + sms - 1) / sms;
    const int grid = (p.n_items + rounds - 1) / rounds;
    cudaError_t e = cudaFuncSetAttribute(tc::ema_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tc::kBwdSmemBytes);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    tc::ema_bwd_tc_kernel<<<grid, tc::kThreads, tc::kBwdSmemBytes, stream>>>(tm_x, tm_g, tm_o, p);
    return check_launch();
}

// reads (and optionally clears) the device-side status word of the tensor-core kernels; synchronises
int read_tc_status(int clear) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, tc::g_tc_status, sizeof(int));
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    if (clear && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tc::g_tc_status, &zero, sizeof(int));
    }
    return v == 0 ? EMA_OK : EMA_ERR_TIMEOUT;
}

}  // namespace ema
