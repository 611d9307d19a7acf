// Fused EMA scan on the Blackwell tensor cores (bf16 in/out, fp32 accumulate and carries).
//
// Within a tile of 128 steps the scan is a dense contraction: with decays a_j and input weights p_k
//     y_m = sum_{k<=m} p_k (prod_{j=k+1..m} a_j) x_k  +  (prod_{j<=m} a_j) h
// i.e. Y = G X + E h^T with G a 128x128 lower-triangular matrix that depends on the decays only and is
// shared by all channels.  G is written to shared memory as bf16 (K-major, 128-byte swizzle), the x
// tile [128 steps x 128 channels] lands next to it by TMA as two 64-channel blocks, exactly as the MMA
// wants its B operand (MN-major, 128-byte swizzle), tcgen05.mma accumulates Y in TMEM (fp32), and the
// epilogue warps add the carry term in fp32, hand the last row on as the next carry, and bf16 y leaves by
// TMA store from the very shared-memory stage the x tile arrived in.
//
// Why 128 channels per MMA: one M=128, K=16 tcgen05.mma costs about 120 cycles whatever N <= 128 is, and
// a tile needs K = 128, i.e. 8 of them per product; at N = 64 that alone exceeds the time HBM needs to
// move the tile.
//
// One persistent CTA per SM walks its work items (scan row, 128-channel tile) and, inside an item, the
// tiles in sequence order.  20 warps in five warpgroups, each warp with one job:
//   warp 0       TMA producer (x tiles, and dy tiles in the backward) into a ring of stages
//   warp 1       MMA issuer; owns the TMEM allocation
//   warp 2       issues the TMA stores of finished tiles and hands the stages back to the producer
//   warp 3       idle (fills the first warpgroup)
//   warps 4-11   epilogue: TMEM lane quadrant (warp % 4) x one half of the 128 channels
//   warps 12-19  build the decay matrices (once per head for a time-invariant decay, per tile otherwise)
// Registers follow the work (setmaxnreg): the first warpgroup and the builders give theirs up, the epilogue
// warpgroups take them.
// The warps meet only through mbarriers: stage full/empty, accumulator full/empty, matrix full/empty,
// carry ready (a ring of 4 so that the warp on the serial carry chain can run ahead of the others), and
// stage staged.  Every wait is bounded (ema_tc_common.cuh): after a timeout the roles run their loops to
// the end without waiting, the CTA tears down normally and the host sees EMA_ERR_TIMEOUT.
#include <atomic>
#include <cstdlib>
#include <cuda_fp16.h>

#include "ema_common.cuh"
#include "ema_tc_common.cuh"
#include "ema_fwd_fma_kernel.cuh"
#include "ema_bwd_fma_kernel.cuh"

namespace ema {
namespace tc {

constexpr int QT = 128;                    // steps per tile = MMA M = MMA K extent
constexpr int DT = 128;                    // channels per tile = MMA N
constexpr int kBlockCols = 64;             // channels per 128-byte-swizzled block (one TMA box)
constexpr int kBlockBytes = QT * 128;      // [128 steps x 64 channels] bf16
constexpr int kTileBytes = 2 * kBlockBytes;
constexpr int kMatBytes = QT * QT * 2;
constexpr int kThreads = 640;              // 20 warps
constexpr int kStoreThread = 64;           // warp 2, lane 0
constexpr int kEpiThread0 = 128;           // warps 4-11
constexpr int kEpiThreads = 256;
constexpr int kEpiWarps = kEpiThreads / 32;
constexpr int kBuildThread0 = 384;         // warps 12-19
constexpr int kBuildThreads = 256;
constexpr int kBuildWarps = kBuildThreads / 32;
// Registers per thread after setmaxnreg.  The thread block starts with 96 x 640 = 61440 and the roles must add up to
// that: 128 light threads, 256 epilogue threads, 256 builder threads.  BUILD_HEAVY gives the builders 8 more and the
// epilogue 8 fewer: 2-12 % faster in the backward with a per-step decay (two matrices and their tables live in the
// builders' registers), faster or slower in the weighted forward depending on the launch (its launcher chooses), 1-4 %
// slower in the plain forward, which keeps 136 / 80.
constexpr int kRegsLight = 48;
template <bool BUILD_HEAVY>
struct RoleRegs {
    static constexpr int epilogue = BUILD_HEAVY ? 128 : 136, builder = BUILD_HEAVY ? 88 : 80;
    static_assert(128 * kRegsLight + 256 * epilogue + 256 * builder == 96 * kThreads, "register pool of the thread block");
};
constexpr int kRing = 4;                   // depth of the forward kernel's ring of per-build carry factors
constexpr uint32_t kIdesc = make_idesc_bf16(QT, DT, 0, 1);

// named barriers (id 0 is __syncthreads)
__device__ __forceinline__ void bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------------------------------------
// Decay matrices.  With cs[j] = sum_{i<=j} log2 a_i over the tile (cs[-1] = 0):
//   LOWER, shift 0:  M[m,k] = p_k 2^(cs[m]   - cs[k]),  k <= m            forward G
//   LOWER, shift 1:  M[m,k] = p_k 2^(cs[m-1] - cs[k]),  k <= m-1;  M[m,m] = diag      backward A1
//   UPPER:           M[m,k] =     2^(cs[k]   - cs[m]),  k >= m                        backward U
// A chunk is 8 consecutive k of one row (16 bytes of bf16).  The chunk that holds the diagonal costs one ex2
// per element.  Every other chunk is a row scalar times a per-column table: the exponent is split at the end
// (LOWER) or the start (UPPER) of the chunk, both parts <= 0, so nothing overflows however small a decay is:
//   LOWER: 2^(cs[m'] - cs[k]) = 2^(cs[m'] - cs[8j+7]) * 2^(cs[8j+7] - cs[k]),   m' = m - shift >= 8j+7
//   UPPER: 2^(cs[k]  - cs[m]) = 2^(cs[8j-1] - cs[m])  * 2^(cs[k] - cs[8j-1]),   m <= 8j-1
// wlo[k] = p_k 2^(cs[8j+7] - cs[k]) and rup[k] = 2^(cs[k] - cs[8j-1]) (j = k / 8) are tables in shared memory.
// Work split over the 256 builder threads: thread t makes one half (4 elements) of the diagonal chunk of row
// t % 128 and every fourth one of the 15 other chunks of the row pair (t % 64, 127 - t % 64).  Which chunks a
// thread owns, and where they are read from and written to, never changes: those offsets are worked out once
// per kernel (OffGeom, DiagGeom), so that a build is little more than loads, multiplies, packs and stores.
// Values are produced into registers first and stored once the matrix buffer has been released by the MMAs
// that were reading it.
// ---------------------------------------------------------------------------------------------
constexpr int kOffSlots = 4;
struct RowChunks {
    uint4 v[kOffSlots];   // off-diagonal chunks
    uint2 dg;             // this thread's half of a diagonal chunk
};
// Off-diagonal chunks of one matrix, per register slot.  All offsets in bytes.
struct OffGeom {
    uint32_t a[kOffSlots];    // into the cs table: the row's entry, cs[m - shift] (LOWER) or cs[m] (UPPER)
    uint32_t c[kOffSlots];    // into a 128-float table: first column of the chunk (8 * chunk floats)
    uint32_t st[kOffSlots];   // destination of the chunk, relative to the start of the matrix storage
    bool last_valid;          // the last slot is empty for a quarter of the threads
};
// This thread's half of the diagonal chunk of row m = t % 128.
struct DiagGeom {
    uint32_t k;      // byte offset of its 4 columns in a 128-float table
    uint32_t top;    // byte offset of cs[m - shift] (LOWER; 0 with has_top false when m - shift < 0) or cs[m] (UPPER)
    uint32_t st;     // destination, relative to the start of the matrix storage
    int lim;         // element e of the half is inside the triangle iff e <= lim (LOWER) or e >= lim (UPPER)
    bool has_top;
};

// Calls f(register slot, row, chunk) for this thread's off-diagonal chunks, in a fixed order.
template <bool UPPER, typename F>
__device__ __forceinline__ void for_off_chunks(int t, F f) {
    const int pr = t & 63, sel = t >> 6;
    const int row_long = UPPER ? pr : 127 - pr;   // the row of the pair with more off-diagonal chunks
    const int row_short = 127 - row_long;
    const int n_long = UPPER ? 15 - (row_long >> 3) : (row_long >> 3);
#pragma unroll
    for (int s = 0; s < kOffSlots; ++s) {   // s is a compile-time register index; i the position in the 15-chunk list
        const int i = 4 * s + sel;
        if (i >= 15) continue;
        const bool in_long = i < n_long;
        const int row = in_long ? row_long : row_short;
        const int j = in_long ? i : i - n_long;                       // index inside the row's chunk list
        const int chunk = UPPER ? (row >> 3) + 1 + j : j;
        f(s, row, chunk);
    }
}
// store_off(row, chunk) -> byte offset of a chunk in the matrix storage
template <bool UPPER, int SHIFT, typename F>
__device__ __forceinline__ void make_geom(int t, OffGeom &og, DiagGeom &dg, F store_off) {
#pragma unroll
    for (int s = 0; s < kOffSlots; ++s) og.a[s] = og.c[s] = og.st[s] = 0;
    og.last_valid = 4 * (kOffSlots - 1) + (t >> 6) < 15;
    for_off_chunks<UPPER>(t, [&](int s, int m, int c) {
        og.a[s] = 4u * static_cast<uint32_t>(UPPER ? m : m - SHIFT);
        og.c[s] = 32u * static_cast<uint32_t>(c);
        og.st[s] = store_off(m, c);
    });
    const int m = t & 127, hb = t >> 7, k0 = (m >> 3) * 8 + 4 * hb;
    dg.k = 4u * static_cast<uint32_t>(k0);
    dg.has_top = UPPER || m - SHIFT >= 0;
    dg.top = dg.has_top ? 4u * static_cast<uint32_t>(UPPER ? m : m - SHIFT) : 0u;
    dg.st = store_off(m, m >> 3) + 8u * static_cast<uint32_t>(hb);
    dg.lim = UPPER ? m - k0 : m - SHIFT - k0;
}

__device__ __forceinline__ float ld_f32(const uint8_t *base, uint32_t off) {
    return *reinterpret_cast<const float *>(base + off);
}
__device__ __forceinline__ float4 ld_f32x4(const uint8_t *base, uint32_t off) {
    return *reinterpret_cast<const float4 *>(base + off);
}

// off-diagonal chunks: row scalar x column table
// (PACKED: two products per instruction; measured faster in the backward kernel, slower in the forward one)
template <bool UPPER, bool PACKED>
__device__ __forceinline__ void compute_off(const OffGeom &g, const uint8_t *cs_b, const uint8_t *tab_b, RowChunks &out) {
#pragma unroll
    for (int s = 0; s < kOffSlots; ++s) {
        if (s == kOffSlots - 1 && !g.last_valid) continue;
        const float ca = ld_f32(cs_b, g.a[s]);
        const float cb = ld_f32(cs_b, UPPER ? g.c[s] - 4u : g.c[s] + 28u);   // cs[8c - 1] | cs[8c + 7]
        const float sc = ex2_approx(UPPER ? cb - ca : ca - cb);     // <= 0 either way
        const float4 w0 = ld_f32x4(tab_b, g.c[s]), w1 = ld_f32x4(tab_b, g.c[s] + 16);
        if constexpr (PACKED) {
            const float2 sc2 = make_float2(sc, sc);
            const float2 v0 = __fmul2_rn(make_float2(w0.x, w0.y), sc2), v1 = __fmul2_rn(make_float2(w0.z, w0.w), sc2),
                         v2 = __fmul2_rn(make_float2(w1.x, w1.y), sc2), v3 = __fmul2_rn(make_float2(w1.z, w1.w), sc2);
            out.v[s] = make_uint4(pack_bf16x2(v0.x, v0.y), pack_bf16x2(v1.x, v1.y), pack_bf16x2(v2.x, v2.y),
                                  pack_bf16x2(v3.x, v3.y));
        } else {
            out.v[s] = make_uint4(pack_bf16x2(w0.x * sc, w0.y * sc), pack_bf16x2(w0.z * sc, w0.w * sc),
                                  pack_bf16x2(w1.x * sc, w1.y * sc), pack_bf16x2(w1.z * sc, w1.w * sc));
        }
    }
}
// diagonal half chunks: one ex2 per element; `diag` is the value on the diagonal itself (SHIFT = 1 only)
template <int SHIFT>
__device__ __forceinline__ void compute_diag_lower(const DiagGeom &g, const uint8_t *cs_b, const uint8_t *p_b, float diag,
                                                   RowChunks &out) {
    const float cm = g.has_top ? ld_f32(cs_b, g.top) : 0.f;
    const float4 c4 = ld_f32x4(cs_b, g.k), p4 = ld_f32x4(p_b, g.k);
    const float cs4[4] = {c4.x, c4.y, c4.z, c4.w}, pw4[4] = {p4.x, p4.y, p4.z, p4.w};
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        // past the diagonal the exponent is positive: clamp it so that the discarded value stays finite
        const float gv = pw4[e] * ex2_approx(fminf(cm - cs4[e], 0.f));
        v[e] = (e <= g.lim) ? gv : ((SHIFT == 1 && e == g.lim + 1) ? diag : 0.f);
    }
    out.dg = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}
__device__ __forceinline__ void compute_diag_upper(const DiagGeom &g, const uint8_t *cs_b, RowChunks &out) {
    const float cm = ld_f32(cs_b, g.top);
    const float4 c4 = ld_f32x4(cs_b, g.k);
    const float cs4[4] = {c4.x, c4.y, c4.z, c4.w};
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = (e >= g.lim) ? ex2_approx(fminf(cs4[e] - cm, 0.f)) : 0.f;
    out.dg = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}
__device__ __forceinline__ void store_matrix(const OffGeom &og, const DiagGeom &dg, uint8_t *mat, const RowChunks &in) {
#pragma unroll
    for (int s = 0; s < kOffSlots; ++s) {
        if (s == kOffSlots - 1 && !og.last_valid) continue;
        *reinterpret_cast<uint4 *>(mat + og.st[s]) = in.v[s];
    }
    *reinterpret_cast<uint2 *>(mat + dg.st) = in.dg;
}

// The same with the column table in half precision (8 halves = one 16-byte load), two products per instruction.
// Tables that carry an input weight (the lower matrices) are stored times 2^kHalfShift, so that weights down to
// 2^-24 (the smallest 1 - a above 0 in fp32) stay normal halves; the row scalar takes the factor back.  What still
// underflows is below 2^-24 of the largest element of its chunk row.
constexpr int kHalfShift = 10;
template <bool UPPER>
__device__ __forceinline__ void compute_off_half(const OffGeom &g, const uint8_t *cs_b, const uint8_t *tab_b, RowChunks &out) {
#pragma unroll
    for (int s = 0; s < kOffSlots; ++s) {
        if (s == kOffSlots - 1 && !g.last_valid) continue;
        const float ca = ld_f32(cs_b, g.a[s]);
        const float cb = ld_f32(cs_b, UPPER ? g.c[s] - 4u : g.c[s] + 28u);   // cs[8c - 1] | cs[8c + 7]
        const float sc = ex2_approx(UPPER ? cb - ca : ca - cb - static_cast<float>(kHalfShift));
        const uint4 t = *reinterpret_cast<const uint4 *>(tab_b + (g.c[s] >> 1));
        const float2 sc2 = make_float2(sc, sc);
        const float2 v0 = __fmul2_rn(__half22float2(*reinterpret_cast<const __half2 *>(&t.x)), sc2),
                     v1 = __fmul2_rn(__half22float2(*reinterpret_cast<const __half2 *>(&t.y)), sc2),
                     v2 = __fmul2_rn(__half22float2(*reinterpret_cast<const __half2 *>(&t.z)), sc2),
                     v3 = __fmul2_rn(__half22float2(*reinterpret_cast<const __half2 *>(&t.w)), sc2);
        out.v[s] = make_uint4(pack_bf16x2(v0.x, v0.y), pack_bf16x2(v1.x, v1.y), pack_bf16x2(v2.x, v2.y),
                              pack_bf16x2(v3.x, v3.y));
    }
}
// Diagonal half chunk of a lower matrix with the input weights in half precision, scaled by 2^kHalfShift.
template <int SHIFT>
__device__ __forceinline__ void compute_diag_lower_half(const DiagGeom &g, const uint8_t *cs_b, const uint8_t *p_b, float diag,
                                                        RowChunks &out) {
    const float cm = (g.has_top ? ld_f32(cs_b, g.top) : 0.f) - static_cast<float>(kHalfShift);
    const float4 c4 = ld_f32x4(cs_b, g.k);
    const uint2 pp = *reinterpret_cast<const uint2 *>(p_b + (g.k >> 1));
    const float2 p01 = __half22float2(*reinterpret_cast<const __half2 *>(&pp.x)),
                 p23 = __half22float2(*reinterpret_cast<const __half2 *>(&pp.y));
    const float cs4[4] = {c4.x, c4.y, c4.z, c4.w}, pw4[4] = {p01.x, p01.y, p23.x, p23.y};
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        // past the diagonal the exponent is positive: clamp it so that the discarded value stays finite
        const float gv = pw4[e] * ex2_approx(fminf(cm - cs4[e], -static_cast<float>(kHalfShift)));
        v[e] = (e <= g.lim) ? gv : ((SHIFT == 1 && e == g.lim + 1) ? diag : 0.f);
    }
    out.dg = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}
// Inclusive scan of one value per row (builder threads 0-127, 4 warps) through shared memory; all 256 builder
// threads call it.  Leaves cs_sm[r] = sum_{i<=r} v_i, visible to the first 128 threads only: the caller's next
// 256-thread barrier publishes it.  The first barrier also fences the previous use of the tables.
// to_end = cs[8j+7] - cs[r] and from_start = cs[r] - cs[8j-1] for r's group of eight, j = r / 8.
__device__ __forceinline__ void builder_scan(float v, int t, float *cs_sm, float *warp_tot, float &to_end,
                                             float &from_start) {
    const int lane = t & 31, w = t >> 5;
    const bool scanner = t < 128;
    if (scanner) {
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float n = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += n;
        }
        const float v_end = __shfl_sync(0xffffffffu, v, lane | 7);
        const float v_before = __shfl_sync(0xffffffffu, v, lane < 8 ? 0 : (lane & ~7) - 1);
        to_end = v_end - v;
        from_start = lane < 8 ? v : v - v_before;
    }
    bar_sync(2, kBuildThreads);  // everybody has finished reading the previous tile's tables
    if (scanner) {
        if (lane == 31) warp_tot[w] = v;
        bar_sync(3, 128);
        float off = 0.f;
#pragma unroll
        for (int i = 0; i < 3; ++i)
            if (i < w) off += warp_tot[i];
        cs_sm[t] = v + off;
    }
}

// dst[0..min(32, n_valid)) = y; deliberately not inlined (see the forward epilogue)
struct BoundsRef {   // what EMA_AT needs from a parameter block
    BoundsTable *bounds;
};
__device__ __noinline__ void store_row32(float *dst, const float (&y)[32], int n_valid, BoundsRef br) {
#pragma unroll
    for (int c = 0; c < 32; ++c)
        if (c < n_valid) *EMA_AT(br, dst + c, 100) = y[c];
}

// MMA descriptors of a [128 steps x 128 channels] tile: two 64-channel blocks kBlockBytes apart (LBO),
// 8-step groups 1024 bytes apart (SBO); K step kb starts 16 rows = 2048 bytes further down.
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) { return make_desc_sw128(addr, kBlockBytes, 1024); }

struct TcParams {
    const float *decay;
    float *chunk_states, *tile_states, *final_state, *log_decay_sum;
    // optional per-step weights [b, L, h] with the decay's strides (per-step decay only): in_weight replaces the
    // convention's input weight inside the decay matrix, out_weight scales the rows of what is written
    const float *in_weight, *out_weight;
    const float *init_state;
    int64_t b, L, h, d;
    int64_t a_sb, a_sl, a_sh;
    int decay_mode, convention, chunk;
    int n_tiles;      // 128-step tiles; one saved state per tile and row (layout shared with the CUDA-core path)
    int n_dtiles, n_items;
    int sub, n_groups;   // channel tiles per work item (1 or 2) and work items per scan row
    int64_t n_chunks;
    // split schedule (see Sched): carries handed from CTA to CTA, 128 floats and one arrival counter per cut,
    // indexed by the number of the CTA on the right-hand side of the cut
    int split;
    float *carry;
    unsigned *flags;
    // aggregate schedule (split == 2): per-tile aggregates [rows, n_tiles, d] and decay products [rows, n_tiles] made
    // by tile_aggregate_kernel; a piece that starts inside an item folds the aggregates of the tiles before it
    const float *agg_vec, *agg_fac;
    BoundsTable *bounds;   // bounds-checking build only
};

// ---------------------------------------------------------------------------------------------
// Which tiles a CTA works on.  Whole items dealt round-robin (split = 0) leave SMs idle when the item count is
// not a multiple of the grid (256 items on 148 SMs: 128 CTAs x 2).  With split = 1 the tiles of all items, in
// item-major order, are cut into one contiguous range per CTA.  A range is at least one item long, so it is a
// possibly partial first item, whole items, and a possibly partial last item, and every item is cut at most
// once.  The CTA that owns the first part of a cut item hands the carry to the owner of the second part through
// global memory (128 floats + an arrival counter per cut; cut j lies between the ranges of CTA j - 1 and CTA j).  Each CTA works on the piece that somebody waits
// for FIRST and on the piece that waits for somebody LAST, so that a carry is published a whole range ahead of
// its use and no wait depends on another wait; the wait itself is bounded like every other wait of the kernel.
// ---------------------------------------------------------------------------------------------
// split = 2 (few work items): the same contiguous ranges, now of any length, but nothing is handed from CTA to CTA.
// A separate pass (tile_aggregate_kernel) has reduced every tile to its aggregate, and a piece that starts inside an
// item computes the state (adjoint) entering it by folding the aggregates of the tiles before (after) it - the
// reference's chunk-state / state-passing / chunk-scan split, with the serial carry done where it is needed.
struct Piece {
    int64_t item;
    int k0, k1;   // tiles [k0, k1) of the item
};
struct Sched {
    int64_t first, stride;
    int n, n_tiles, head_k0, tail_k1;
    bool split;
    __device__ Sched(int n_items, int n_tiles_, bool split_) : n_tiles(n_tiles_), split(split_) {
        if (!split_) {
            first = blockIdx.x;
            stride = gridDim.x;
            n = n_items > static_cast<int>(blockIdx.x) ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
            head_k0 = 0;
            tail_k1 = n_tiles_;
        } else {
            const int64_t units = static_cast<int64_t>(n_items) * n_tiles_;
            const int64_t u0 = blockIdx.x * units / gridDim.x, u1 = (blockIdx.x + 1) * units / gridDim.x;
            first = u0 / n_tiles_;
            const int64_t last = (u1 - 1) / n_tiles_;
            stride = 1;
            n = static_cast<int>(last - first + 1);
            head_k0 = static_cast<int>(u0 - first * n_tiles_);
            tail_k1 = static_cast<int>(u1 - last * n_tiles_);
        }
    }
    // idx-th piece in working order.  FORWARD scan: a cut last item starts at tile 0 (somebody waits for it), a cut
    // first item needs a carry: [last, middle ..., first].  BACKWARD scan: the roles are swapped, ascending order.
    template <bool FORWARD>
    __device__ Piece get(int idx) const {
        int q = idx;
        if (FORWARD && split && n > 1) q = idx == 0 ? n - 1 : (idx == n - 1 ? 0 : idx);
        Piece pc;
        pc.item = first + q * stride;
        pc.k0 = q == 0 ? head_k0 : 0;
        pc.k1 = q == n - 1 ? tail_k1 : n_tiles;
        return pc;
    }
};
// State entering tile k0 of a row's channel c: h <- P_j h + S_j over the tiles j < k0 (vec, fac: this row's aggregates).
// Kept out of line: it runs once per piece, and the epilogue's hot loop must stay small.
// (kFoldBatch aggregates are fetched at a time - independent loads, so one memory round trip per batch - and then folded
// in order, one FMA each: the thread block that starts deepest inside an item would otherwise pay a round trip per tile.)
constexpr int kFoldBatch = 32;
__device__ __noinline__ float fold_state_before(const float *vec, const float *fac, int64_t d, int k0, float h,
                                                BoundsRef br) {
    for (int j = 0; j < k0; j += kFoldBatch) {
        float s[kFoldBatch], f[kFoldBatch];
#pragma unroll
        for (int i = 0; i < kFoldBatch; ++i) {
            const bool ok = j + i < k0;   // past the end: the identity step
            s[i] = ok ? __ldg(EMA_AT(br, vec + static_cast<int64_t>(j + i) * d, 101)) : 0.f;
            f[i] = ok ? __ldg(EMA_AT(br, fac + j + i, 102)) : 1.f;
        }
#pragma unroll
        for (int i = 0; i < kFoldBatch; ++i) h = fmaf(f[i], h, s[i]);
    }
    return h;
}
// Adjoint entering tile k1 - 1 from the right: g <- G_j + F_j g over the tiles j = n_tiles - 1 .. k1.
__device__ __noinline__ float fold_adjoint_after(const float *vec, const float *fac, int64_t d, int k1, int n_tiles, float g,
                                                 BoundsRef br) {
    for (int j = n_tiles - 1; j >= k1; j -= kFoldBatch) {
        float s[kFoldBatch], f[kFoldBatch];
#pragma unroll
        for (int i = 0; i < kFoldBatch; ++i) {
            const bool ok = j - i >= k1;
            s[i] = ok ? __ldg(EMA_AT(br, vec + static_cast<int64_t>(j - i) * d, 103)) : 0.f;
            f[i] = ok ? __ldg(EMA_AT(br, fac + j - i, 104)) : 1.f;
        }
#pragma unroll
        for (int i = 0; i < kFoldBatch; ++i) g = fmaf(f[i], g, s[i]);
    }
    return g;
}
constexpr int kCarryFloats = 2 * DT;   // per cut: the carries of up to two channel tiles
// Bounded wait for a carry: one arrival per 64-channel half of every channel tile of the item.
__device__ __forceinline__ bool wait_carry(const unsigned *flag, unsigned need, volatile int *abort_flag, int site,
                                           uint32_t limit = kWaitLimit) {
    for (uint32_t i = 0; i < limit; ++i) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= need) return true;
        if (*abort_flag) return false;
        __nanosleep(64);
    }
    *abort_flag = 1;
    atomicCAS(&g_tc_status, 0, 0x100 | (site & 0xff));
    return false;
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
// Five stages of one [128 x 128] bf16 tile and ONE matrix buffer (198 KB in all).  Measured against four stages and two
// matrix buffers: 1.7 % faster on the headline shape with either kind of decay, 4-7 % on narrow heads (d = 64, 128),
// 17-25 % for the weighted scan - a fifth tile in flight is worth more than building the next matrix while the MMAs
// still read the current one (with paired channel tiles the builders have a tile's time to spare anyway).
constexpr int kFwdStages = 5;
constexpr int kFwdMatBufs = 1;
// A forward work item may hold two channel tiles of one scan row, walked side by side (tile k of the first, tile k of
// the second, tile k + 1 of the first, ...), so that one decay matrix serves two products: with a per-step decay the
// builders are the bottleneck otherwise.  A carry is then used two sub-tiles after it was made, which takes a deeper
// ring than kRing (the fastest epilogue warp may be two sub-tiles ahead of the slowest).
constexpr int kFwdHRing = 8;
struct FwdSmem {
    static constexpr int mat = 0;
    static constexpr int x = mat + kFwdMatBufs * kMatBytes;   // stages: x tile in, y tile out
    static constexpr int h = x + kFwdStages * kTileBytes;     // float[kFwdHRing][128] carry entering a sub-tile
    static constexpr int e = h + kFwdHRing * DT * 4;           // float[kRing][128] E_m per build
    static constexpr int cs = e + kRing * QT * 4;              // float[128] cumulative log2 decay
    static constexpr int pw = cs + QT * 4;                     // float[128] input weights
    static constexpr int wlo = pw + QT * 4;                    // float[128] column table of the off-diagonal chunks
    static constexpr int ow = wlo + QT * 4;                    // float[kRing][128] output weight per row and build (weighted scan)
    static constexpr int wt = ow + kRing * QT * 4;             // float[4] scan scratch
    static constexpr int bars = wt + 16;
    // stage full/empty/staged, acc full/empty, matrix full/empty, carry ready
    static constexpr int n_bars = 3 * kFwdStages + 4 + 2 * kFwdMatBufs + kFwdHRing;
    static constexpr int tmem_slot = bars + n_bars * 8;
    static constexpr int abort_flag = tmem_slot + 4;
    static constexpr int total = abort_flag + 4;
};
constexpr int kFwdSmemBytes = FwdSmem::total + 1024;  // + slack for the manual 1024-byte alignment
static_assert(kFwdSmemBytes <= 227 * 1024, "forward shared memory exceeds the per-CTA limit");

// WEIGHTED: per-step input weights inside the decay matrix and output weights on the rows of what is written, as its
// own instantiation: in the plain kernel even a never-taken branch for them costs 40 % of the per-step speed (the
// five roles' code competes for the instruction cache).
// AGG: the aggregate schedule (split = 2), also its own instantiation.  The state entering every tile is then the
// fold of the per-tile aggregates, h_{k+1} = P_k h_k + S_k, carried in a register by the thread that owns the
// channel - the same fp32 chain wherever the pieces are cut, so the results do not depend on the grid - and the last
// row of the product is no longer on a serial chain.
// BUILD_HEAVY: the register split of RoleRegs (weighted scans only; chosen by the launcher).
template <bool WEIGHTED, bool AGG, bool BUILD_HEAVY = false>
__global__ void __launch_bounds__(kThreads, 1)
ema_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                  const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool per_step = p.decay_mode == EMA_DECAY_PER_STEP;
    const int conv = p.convention;
    const int L = static_cast<int>(p.L);

    float *h_sm = reinterpret_cast<float *>(smem + FwdSmem::h);
    float *e_sm = reinterpret_cast<float *>(smem + FwdSmem::e);
    float *cs_sm = reinterpret_cast<float *>(smem + FwdSmem::cs);
    float *p_sm = reinterpret_cast<float *>(smem + FwdSmem::pw);
    float *wlo_sm = reinterpret_cast<float *>(smem + FwdSmem::wlo);
    float *ow_sm = reinterpret_cast<float *>(smem + FwdSmem::ow);
    float *wt_sm = reinterpret_cast<float *>(smem + FwdSmem::wt);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + FwdSmem::abort_flag);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + FwdSmem::tmem_slot);
    auto bar = [&](int i) { return sbase + FwdSmem::bars + i * 8; };
    constexpr int B_FULL = 0, B_EMPTY = kFwdStages, B_STAGED = 2 * kFwdStages, B_ACC_FULL = 3 * kFwdStages,
                  B_ACC_EMPTY = B_ACC_FULL + 2, B_MAT_FULL = B_ACC_EMPTY + 2, B_MAT_EMPTY = B_MAT_FULL + kFwdMatBufs,
                  B_H = B_MAT_EMPTY + kFwdMatBufs;
    constexpr uint32_t kTmemCols = 2 * DT;

    if (tid == 0) {
        for (int i = 0; i < kFwdStages; ++i) {
            mbar_init(bar(B_FULL + i), 1);
            mbar_init(bar(B_EMPTY + i), 1);
            mbar_init(bar(B_STAGED + i), kEpiWarps);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), kEpiWarps); }
        for (int i = 0; i < kFwdMatBufs; ++i) { mbar_init(bar(B_MAT_FULL + i), kBuildWarps); mbar_init(bar(B_MAT_EMPTY + i), 1); }
        // carry ready: one arrival per channel half (row 127's two threads), or per loader warp with aggregates
        for (int i = 0; i < kFwdHRing; ++i) mbar_init(bar(B_H + i), AGG ? 4 : 2);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_y);
    }
    // the matrices start as zeros; the builders only ever write the lower triangle
    for (int i = tid; i < kFwdMatBufs * kMatBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(smem + FwdSmem::mat)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 1) {
        tmem_alloc(sbase + FwdSmem::tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done; nothing before this line has touched global memory, everything after it may depend on the kernel
    // before this one on the stream
    grid_dependency_wait();

    const Sched sched(p.n_items, p.n_tiles, p.split != 0);
    // item -> scan row, first channel tile, number of channel tiles (1 or 2)
    auto item_row = [&](int64_t item) { return item / p.n_groups; };
    auto item_dt0 = [&](int64_t item) { return static_cast<int>(item % p.n_groups) * p.sub; };
    auto item_nsub = [&](int64_t item) {
        const int left = p.n_dtiles - static_cast<int>(item % p.n_groups) * p.sub;
        return left < p.sub ? left : p.sub;
    };
    // log2 of the multiplicative decay of one step
    // (clamped: a decay of exactly 0 would make the prefix sums -inf and their differences NaN; 2^-160 is 0 in fp32,
    // and a small bound keeps the prefix sums of a tile with many such steps precise)
    // lg2.approx (absolute error 2^-22): the decays end up in bf16 matrix elements and in carry factors over 128 steps
    auto log2_decay = [&](float v) { return fmaxf(conv ? v * 1.4426950408889634f : __log2f(v), -160.f); };

    if (warp < 4) {
        reg_dec<kRegsLight>();
        if (warp == 0) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                uint32_t it = 0;
                for (int pi = 0; pi < sched.n && !*abort_flag; ++pi) {
                    // whole items, several per thread block: the SMs that other thread blocks leave early are better used
                    // by the next kernel's set-up from the last item on (see the end of this loop)
                    if (!sched.split && sched.n > 1 && pi == sched.n - 1) grid_dependents_launch();
                    const Piece pc = sched.get<true>(pi);
                    const int dt0 = item_dt0(pc.item), nsub = item_nsub(pc.item);
                    const int64_t row = item_row(pc.item);
                    const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
                    for (int k = pc.k0; k < pc.k1 && !*abort_flag; ++k) {
                        for (int u = 0; u < nsub; ++u, ++it) {
                            const int dtile = dt0 + u;
                            const int s = it % kFwdStages;
                            const uint32_t ph = (it / kFwdStages) & 1;
                            if (!mbar_wait(bar(B_EMPTY + s), ph ^ 1, abort_flag, 1)) break;
                            mbar_expect_tx(bar(B_FULL + s), kTileBytes);
                            const uint32_t dst = sbase + FwdSmem::x + s * kTileBytes;
                            tma_load_4d(dst, &tm_x, bar(B_FULL + s), dtile * DT, hi, k * QT, bi);
                            tma_load_4d(dst + kBlockBytes, &tm_x, bar(B_FULL + s), dtile * DT + kBlockCols, hi, k * QT, bi);
                        }
                    }
                }
                // The last loads are on their way: from here on the next kernel on the stream may be brought in (it
                // does its set-up on the SMs that free up and waits for this grid to finish before touching memory).
                // Not from the start: thread blocks of the next kernel that sit waiting on the idle SMs for a whole
                // kernel would keep small kernels of other streams - a collective - from finding room.
                grid_dependents_launch();
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                // A matrix is built per tile (per-step decay) or whenever the head changes (time-invariant
                // decay); the MMA issuer, the epilogue and the builders evaluate the same predicate, so they
                // agree on the build counter mt without talking to each other.
                uint32_t it = 0, mt = 0;
                int cur_head = -1, mb_cur = 0;
                for (int pi = 0; pi < sched.n && !*abort_flag; ++pi) {
                    const Piece pc = sched.get<true>(pi);
                    const int hi = static_cast<int>(item_row(pc.item) % p.h);
                    const int nsub = item_nsub(pc.item);
                    for (int k = pc.k0; k < pc.k1 && !*abort_flag; ++k)
                    for (int u = 0; u < nsub; ++u, ++it) {
                        const int s = it % kFwdStages;
                        const uint32_t ph = (it / kFwdStages) & 1;
                        const int acc = it & 1;
                        const uint32_t aph = (it >> 1) & 1;
                        if (u == 0 && (per_step || hi != cur_head)) {
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
                        const uint64_t ad0 = make_desc_sw128(sbase + FwdSmem::mat + mb_cur * kMatBytes, 16, 1024);
                        const uint64_t bd0 = tile_desc(sbase + FwdSmem::x + s * kTileBytes);
    #pragma unroll
                        for (int kb = 0; kb < QT / 16; ++kb) {
                            // descriptor start addresses are in 16-byte units: next K step inside / across 64-wide K blocks
                            const uint64_t ad = ad0 + (((kb >> 2) * (QT * 128) + (kb & 3) * 32) >> 4);
                            const uint64_t bd = bd0 + ((kb * 2048) >> 4);
                            umma_bf16(tmem_base + acc * DT, ad, bd, kIdesc, kb > 0 ? 1u : 0u);
                        }
                        umma_commit(bar(B_ACC_FULL + acc));
                        if (per_step && u == nsub - 1) umma_commit(bar(B_MAT_EMPTY + mb_cur));
                    }
                }
            }
        } else {
            // ---------------- TMA store issuer ----------------
            if (tid == kStoreThread) {
                uint32_t it = 0;
                for (int pi = 0; pi < sched.n && !*abort_flag; ++pi) {
                    const Piece pc = sched.get<true>(pi);
                    const int dt0 = item_dt0(pc.item), nsub = item_nsub(pc.item);
                    const int64_t row = item_row(pc.item);
                    const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
                    for (int k = pc.k0; k < pc.k1 && !*abort_flag; ++k)
                    for (int u = 0; u < nsub; ++u, ++it) {
                        const int dtile = dt0 + u;
                        const bool two = dtile * DT + kBlockCols < p.d;   // the second 64-channel block exists
                        const int s = it % kFwdStages;
                        if (!mbar_wait(bar(B_STAGED + s), (it / kFwdStages) & 1, abort_flag, 9)) break;
                        const uint32_t src = sbase + FwdSmem::x + s * kTileBytes;
                        tma_store_4d(&tm_y, src, dtile * DT, hi, k * QT, bi);
                        if (two) tma_store_4d(&tm_y, src + kBlockBytes, dtile * DT + kBlockCols, hi, k * QT, bi);
                        tma_store_commit();
                        tma_store_wait_read<0>();          // the stage has been read: hand it back to the producer
                        mbar_arrive(bar(B_EMPTY + s));
                    }
                }
                tma_store_wait_all();
            }
        }
    } else if (tid < kBuildThread0) {
        reg_inc<RoleRegs<BUILD_HEAVY>::epilogue>();
        // ---------------- epilogue ----------------
        // Thread (q, lane, half) owns row m = 32 q + lane and channels [64 half, 64 half + 64) of the tile,
        // handled 32 at a time.  The two threads of row 127 are the serial carry chain: they publish the
        // state entering the next tile as soon as they have it; nobody else waits for anything but that
        // state and the accumulator.
        const int q = warp & 3;
        const int half = (warp - kEpiThread0 / 32) >> 2;
        const int m = q * 32 + lane;
        const bool loader = half == 0;   // 128 threads that move per-channel vectors: thread m <-> channel m
        uint32_t it = 0, mt = 0;
        int cur_head = -1;
        // AGG (loaders): the state entering the current tile for channel m of each of the (at most two) sub-tiles, and the
        // current tile's aggregates, fetched one tile ahead.  Plain scalars selected by the sub-tile index: an array
        // indexed at run time would live in local memory, and storing a value just loaded there waits for the load.
        float h_reg0 = 0.f, h_reg1 = 0.f, agg_s0 = 0.f, agg_s1 = 0.f, agg_p = 0.f;
        for (int pi = 0; pi < sched.n; ++pi) {
            const Piece pc = sched.get<true>(pi);
            const int dt0 = item_dt0(pc.item), nsub = item_nsub(pc.item);
            const int64_t row = item_row(pc.item);
            const int hi = static_cast<int>(row % p.h);
            const bool publish = !AGG && pc.k1 < p.n_tiles;   // the item continues in another CTA: hand it the state
            // a piece that ends inside an item hands its state to the next CTA (cut blockIdx.x + 1); a piece that starts
            // inside an item takes it from the previous one (cut blockIdx.x); kCarryFloats floats per cut
            float *carry_out = p.carry + static_cast<int64_t>(blockIdx.x + 1) * kCarryFloats;
            if (loader) {
                if (!AGG && pc.k0 > 0) {   // second part of a cut item: the state comes from the CTA that made the first part
                    if (lane == 0) wait_carry(EMA_AT(p, p.flags + blockIdx.x, 105), 2u * nsub, abort_flag, 22);
                    __syncwarp();
                }
                for (int u = 0; u < nsub; ++u) {
                    const int c0u = (dt0 + u) * DT;
                    const bool ok = c0u + m < p.d;
                    float v;
                    if (AGG || pc.k0 == 0) {
                        v = (p.init_state && ok) ? *EMA_AT(p, p.init_state + row * p.d + c0u + m, 106) : 0.f;
                        if (pc.k0 == 0 && p.chunk_states && ok)
                            *EMA_AT(p, p.chunk_states + (row * p.n_chunks) * p.d + c0u + m, 107) = v;
                        if (AGG && pc.k0 > 0 && ok)
                            v = fold_state_before(p.agg_vec + row * p.n_tiles * p.d + c0u + m,
                                                  p.agg_fac + row * p.n_tiles, p.d, pc.k0, v, BoundsRef{p.bounds});
                    } else {
                        v = __ldcg(EMA_AT(p, p.carry + static_cast<int64_t>(blockIdx.x) * kCarryFloats + u * DT + m, 108));
                    }
                    h_sm[((it + u) & (kFwdHRing - 1)) * DT + m] = v;
                    if (u == 0) h_reg0 = v; else h_reg1 = v;
                }
            }
            bar_sync(1, kEpiThreads);  // once per piece: the previous one is finished everywhere, the state is in place
            if (AGG ? (loader && lane == 0) : (m == QT - 1))
                for (int u = 0; u < nsub; ++u) mbar_arrive(bar(B_H + ((it + u) & (kFwdHRing - 1))));
            if (AGG && loader && pc.k0 + 1 < pc.k1) {   // aggregates of the piece's first tile
                agg_p = __ldg(EMA_AT(p, p.agg_fac + row * p.n_tiles + pc.k0, 109));
                const float *av = p.agg_vec + (row * p.n_tiles + pc.k0) * p.d + dt0 * DT + m;
                agg_s0 = (dt0 * DT + m < p.d) ? __ldg(EMA_AT(p, av, 110)) : 0.f;
                agg_s1 = (nsub > 1 && (dt0 + 1) * DT + m < p.d) ? __ldg(EMA_AT(p, av + DT, 111)) : 0.f;
            }
            for (int k = pc.k0; k < pc.k1; ++k)
            for (int u = 0; u < nsub; ++u, ++it) {
                const int c0 = (dt0 + u) * DT;
                const bool ch_ok = loader && c0 + m < p.d;
                float *ts_item = p.tile_states ? p.tile_states + row * p.n_tiles * p.d + c0 : nullptr;
                const int acc = it & 1, slot = it & (kFwdHRing - 1), s = it % kFwdStages;
                const uint32_t aph = (it >> 1) & 1, hph = (it / kFwdHRing) & 1;
                if (u == 0 && (per_step || hi != cur_head)) { cur_head = hi; ++mt; }
                if (AGG && loader && k + 1 < pc.k1) {   // the state entering this channel tile's next tile
                    const float hn = fmaf(agg_p, u == 0 ? h_reg0 : h_reg1, u == 0 ? agg_s0 : agg_s1);
                    if (u == 0) h_reg0 = hn; else h_reg1 = hn;
                    h_sm[((it + nsub) & (kFwdHRing - 1)) * DT + m] = hn;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_H + ((it + nsub) & (kFwdHRing - 1))));
                    // the next tile's aggregates: a whole tile's time to arrive
                    if (k + 2 < pc.k1) {
                        const float *an = p.agg_vec + (row * p.n_tiles + k + 1) * p.d + c0 + m;
                        if (ch_ok && u == 0) agg_s0 = __ldg(EMA_AT(p, an, 113));
                        if (ch_ok && u != 0) agg_s1 = __ldg(EMA_AT(p, an, 114));
                        if (u == nsub - 1) agg_p = __ldg(EMA_AT(p, p.agg_fac + row * p.n_tiles + k + 1, 115));
                    }
                }
                if (lane == 0) mbar_wait(bar(B_ACC_FULL + acc), aph, abort_flag, 5);  // one poller per warp
                __syncwarp();
                tc_fence_after_sync();
                const float E = e_sm[((mt - 1) & (kRing - 1)) * QT + m];
                // the row's output weight comes with the matrix, fetched by the builders a tile ahead: a global load
                // here would put the latency of loaded DRAM into every tile
                float out_w = 1.f;
                if constexpr (WEIGHTED) out_w = ow_sm[((mt - 1) & (kRing - 1)) * QT + m];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * DT + half * 64;
                if (lane == 0) mbar_wait(bar(B_H + slot), hph, abort_flag, 6);
                __syncwarp();
                const float *hin = h_sm + slot * DT;
                const int t = k * QT + m;
                // ACC_FULL says the MMAs have finished reading the x tile: its stage now takes the y tile
                uint8_t *stg = smem + FwdSmem::x + s * kTileBytes + half * kBlockBytes;
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {
                    float y[32];
                    __syncwarp();  // single-thread branches of the previous pass have rejoined
                    tmem_ld32(taddr + pass * 32, y);
                    tmem_ld_wait();
                    if (pass == 1) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + acc));  // one arrival per warp
                    }
                    const int cb = half * 64 + pass * 32;
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {   // (packed fp32 FMAs were measured slower here)
                        const float4 hv = *reinterpret_cast<const float4 *>(hin + cb + c);
                        y[c] = fmaf(E, hv.x, y[c]);
                        y[c + 1] = fmaf(E, hv.y, y[c + 1]);
                        y[c + 2] = fmaf(E, hv.z, y[c + 2]);
                        y[c + 3] = fmaf(E, hv.w, y[c + 3]);
                    }
                    if (!AGG && m == QT - 1 && k + 1 < pc.k1) {  // the last row is the state entering this channel tile's next tile
                        float *hout = h_sm + ((it + nsub) & (kFwdHRing - 1)) * DT + cb;
#pragma unroll
                        for (int c = 0; c < 32; c += 4)
                            *reinterpret_cast<float4 *>(hout + c) = make_float4(y[c], y[c + 1], y[c + 2], y[c + 3]);
                        if (pass == 1) mbar_arrive(bar(B_H + ((it + nsub) & (kFwdHRing - 1))));
                    }
                    // rare side outputs (a chunk boundary, the last step): kept out of line so that they do not
                    // cost the common path registers
                    const bool at_chunk_end = p.chunk_states && t + 1 < L && (t + 1) % p.chunk == 0;
                    const bool at_last_step = p.final_state && t == L - 1;
                    const bool at_cut = publish && m == QT - 1 && k + 1 == pc.k1;
                    if (at_chunk_end || at_last_step || at_cut) {
                        float tmp[32];  // a copy, so that y itself never has its address taken and stays in registers
#pragma unroll
                        for (int c = 0; c < 32; ++c) tmp[c] = y[c];
                        const int n_valid = static_cast<int>(p.d) - (c0 + cb);
                        if (at_chunk_end)
                            store_row32(p.chunk_states + (row * p.n_chunks + (t + 1) / p.chunk) * p.d + c0 + cb, tmp, n_valid,
                                        BoundsRef{p.bounds});
                        if (at_last_step) store_row32(p.final_state + row * p.d + c0 + cb, tmp, n_valid, BoundsRef{p.bounds});
                        if (at_cut) {
                            store_row32(carry_out + u * DT + cb, tmp, 32, BoundsRef{p.bounds});
                            if (pass == 1) {   // this half of the carry is complete
                                __threadfence();
                                atomicAdd(EMA_AT(p, p.flags + blockIdx.x + 1, 116), 1u);
                            }
                        }
                    }
                    if constexpr (WEIGHTED) {   // (1 without output weights; the states above are the unweighted ones)
                        const float2 w2 = make_float2(out_w, out_w);
#pragma unroll
                        for (int c = 0; c < 32; c += 2) {   // two products per instruction: the code must stay small
                            const float2 v = __fmul2_rn(make_float2(y[c], y[c + 1]), w2);
                            y[c] = v.x; y[c + 1] = v.y;
                        }
                    }
                    // bf16 -> the stage, in the TMA's 128-byte swizzle
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 qv = make_uint4(pack_bf16x2(y[8 * j], y[8 * j + 1]), pack_bf16x2(y[8 * j + 2], y[8 * j + 3]),
                                                    pack_bf16x2(y[8 * j + 4], y[8 * j + 5]), pack_bf16x2(y[8 * j + 6], y[8 * j + 7]));
                        *reinterpret_cast<uint4 *>(stg + sw128_offset(m, pass * 4 + j)) = qv;
                    }
                }
                // state entering the tile -> saved state k, one coalesced line per 32 threads
                if (ts_item && ch_ok) *EMA_AT(p, ts_item + static_cast<int64_t>(k) * p.d + m, 117) = hin[m];
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_STAGED + s));
            }
        }
    } else {
        reg_dec<RoleRegs<BUILD_HEAVY>::builder>();
        // ---------------- matrix builders ----------------
        const int bt = tid - kBuildThread0;   // 0-255; threads 0-127 also own row r = bt of the per-row tables
        const int r = bt & 127;
        const bool row_owner = bt < 128;
        uint32_t mt = 0;
        int cur_head = -1;
        OffGeom og;
        DiagGeom dgm;
        // a forward matrix is two 64-wide K blocks of [128 rows x 128 B], one after the other
        make_geom<false, 0>(bt, og, dgm, [](int m, int c) {
            return static_cast<uint32_t>((c >> 3) * (QT * 128)) + sw128_offset(m, c & 7);
        });
        const uint8_t *cs_b = smem + FwdSmem::cs, *p_b = smem + FwdSmem::pw, *wlo_b = smem + FwdSmem::wlo;
        // one build: scan log2 a, produce the matrix into registers, then store it when the buffer is free
        // (l2, pw and the row's output weight ow are read from the row owners only)
        auto build = [&](float l2, float pw, float ow) {
            const int mb = mt % kFwdMatBufs;
            float to_end = 0.f, from_start = 0.f;
            builder_scan(l2, bt, cs_sm, wt_sm, to_end, from_start);
            if (row_owner) {
                p_sm[r] = pw;
                wlo_sm[r] = pw * ex2_approx(to_end);
            }
            bar_sync(2, kBuildThreads);
            RowChunks g;
            compute_diag_lower<0>(dgm, cs_b, p_b, 0.f, g);
            compute_off<false, false>(og, cs_b, wlo_b, g);
            const float E = ex2_approx(cs_sm[r]);
            if (lane == 0) mbar_wait(bar(B_MAT_EMPTY + mb), ((mt / kFwdMatBufs) & 1) ^ 1, abort_flag, 8);
            __syncwarp();
            store_matrix(og, dgm, smem + FwdSmem::mat + mb * kMatBytes, g);
            if (row_owner) {
                e_sm[(mt & (kRing - 1)) * QT + r] = E;
                if constexpr (WEIGHTED) ow_sm[(mt & (kRing - 1)) * QT + r] = ow;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_MAT_FULL + mb));
            ++mt;
        };
        for (int pi = 0; pi < sched.n; ++pi) {
            const Piece pc = sched.get<true>(pi);
            const int64_t row = item_row(pc.item);
            const int dtile = item_dt0(pc.item);
            const int64_t bi = row / p.h, hi = row % p.h;
            const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
            if (!per_step) {
                const float v = *EMA_AT(p, arow, 118);
                if (static_cast<int>(hi) != cur_head) {
                    cur_head = static_cast<int>(hi);
                    build(log2_decay(v), conv ? 1.f : 1.f - v, 1.f);
                }
                if (p.log_decay_sum && bt == 0 && dtile == 0)
                    *EMA_AT(p, p.log_decay_sum + row, 119) = static_cast<float>(L) * (conv ? v : logf(v));
                continue;
            }
            // per-step decay: the raw value of step r of the next tile is fetched one tile ahead
            float logsum = 0.f;
            const float ident = conv ? 0.f : 1.f;   // raw value of an identity step (past L)
            float v_next = (row_owner && pc.k0 * QT + r < L) ? *EMA_AT(p, arow + static_cast<int64_t>(pc.k0 * QT + r) * p.a_sl, 120)
                                                             : ident;
            // input weights (WEIGHTED only): same strides as the decay; free of branches on the pointer (without an
            // input-weight tensor the decay is simply read twice)
            const bool has_w = WEIGHTED && p.in_weight != nullptr;
            const float *wrow = (has_w ? p.in_weight : p.decay) + bi * p.a_sb + hi * p.a_sh;
            float w_next = 0.f;
            if constexpr (WEIGHTED)
                w_next = (row_owner && pc.k0 * QT + r < L) ? *EMA_AT(p, wrow + static_cast<int64_t>(pc.k0 * QT + r) * p.a_sl, 121)
                                                           : 0.f;
            // output weights (WEIGHTED only): fetched like the input weights and handed to the epilogue with the matrix
            // (1 without an output-weight tensor, 0 past the end of the sequence)
            const float *orow = p.out_weight ? p.out_weight + bi * p.a_sb + hi * p.a_sh : nullptr;
            auto out_weight_at = [&](int t) {
                if (!orow) return 1.f;
                return (row_owner && t < L) ? *EMA_AT(p, orow + static_cast<int64_t>(t) * p.a_sl, 112) : 0.f;
            };
            float o_next = 1.f;
            if constexpr (WEIGHTED) o_next = out_weight_at(pc.k0 * QT + r);
            for (int k = pc.k0; k < pc.k1; ++k) {
                const float v = v_next, w = w_next, ow = o_next;
                if (k + 1 < pc.k1) {
                    const int t = (k + 1) * QT + r;
                    v_next = (row_owner && t < L) ? *EMA_AT(p, arow + static_cast<int64_t>(t) * p.a_sl, 122) : ident;
                    if constexpr (WEIGHTED) {
                        w_next = (row_owner && t < L) ? *EMA_AT(p, wrow + static_cast<int64_t>(t) * p.a_sl, 123) : 0.f;
                        o_next = out_weight_at(t);
                    }
                }
                build(log2_decay(v), has_w ? w : (conv ? 1.f : 1.f - v), ow);
                // cs_sm[127] now holds log2 of the product of this tile's decays
                if (p.log_decay_sum && bt == 0) logsum += cs_sm[QT - 1] * 0.6931471805599453f;
            }
            if (p.log_decay_sum && bt == 0 && dtile == 0) *EMA_AT(p, p.log_decay_sum + row, 124) = logsum;
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
        tmem_dealloc(tmem_base, kTmemCols);
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
struct TcBwdParams {
    const float *decay;
    const float *tile_states;
    const float *dfinal_state;
    float *dinit_state;
    float *da_partial;
    int64_t b, L, h, d;
    int64_t a_sb, a_sl, a_sh;
    int decay_mode, convention;
    int n_tiles, n_dtiles, n_items;
    int sub, n_groups;   // channel tiles per work item (1 or 2) and work items per scan row (see the forward kernel)
    int n_dt64;       // 64-channel slices per row in the partial-sum buffer
    int64_t head_partial_offset;
    // split schedule (see Sched): adjoint carries handed from CTA to CTA
    int split;
    float *carry;
    unsigned *flags;
    // aggregate schedule (split == 2): adjoint aggregates [rows, n_tiles, d] and products [rows, n_tiles]
    const float *agg_vec, *agg_fac;
    BoundsTable *bounds;   // bounds-checking build only
};

constexpr int kBwdStages = 2;
constexpr int kRowRing = 3;   // per-row scalar tables: a build's table is read early in the tile that uses it
// Depth of the carry rings (saved state and adjoint entering a sub-tile).  With two channel tiles per item a carry is
// used two sub-tiles after it was made and the fastest epilogue warp may be two sub-tiles ahead of the slowest: five
// slots.  (Shared memory is full: to make room the builders' column tables are kept in half precision - they only
// multiply into bf16 matrix elements.)
constexpr int kBwdCRing = 5;
// The two matrices are triangular: the upper-right 64x64 quadrant of A1 and the lower-left one of U are zero.
// Stored by 64-wide K blocks (rows of 128 bytes), the zero quadrants are one shared 8 KB region Z:
//   [A1 K-block 0, rows 0-127][U K-block 0, rows 0-63][Z][A1 K-block 1, rows 64-127][U K-block 1, rows 0-127]
// so that U K-block 0 = (U rows 0-63, Z) and A1 K-block 1 = (Z, A1 rows 64-127) are each contiguous.
struct BwdSmem {
    static constexpr int m_a1k0 = 0;
    static constexpr int m_u00 = m_a1k0 + kBlockBytes;
    static constexpr int m_z = m_u00 + kBlockBytes / 2;
    static constexpr int m_a111 = m_z + kBlockBytes / 2;
    static constexpr int m_uk1 = m_a111 + kBlockBytes / 2;
    static constexpr int mat_bytes = m_uk1 + kBlockBytes;              // 56 KB
    static constexpr int xg = mat_bytes;                               // stages of [x tile | dy tile]
    static constexpr int ostage = xg + kBwdStages * 2 * kTileBytes;    // dx staging: one tile, a 64-channel block per half
    static constexpr int hs = ostage + kTileBytes;                     // float[kBwdCRing][128] saved state entering the sub-tile
    static constexpr int g = hs + kBwdCRing * DT * 4;                  // float[kBwdCRing][128] adjoint carry
    static constexpr int rowsc = g + kBwdCRing * DT * 4;               // float[kRowRing][3][128]: Eprev, F, a per build
    static constexpr int cs = rowsc + kRowRing * 3 * QT * 4;           // float[128]
    static constexpr int pw = cs + QT * 4;                             // half[128] input weights * 2^kHalfShift
    static constexpr int wlo = pw + QT * 2;                            // half[128] column table, lower matrix (same scale)
    static constexpr int rup = wlo + QT * 2;                           // half[128] column table, upper matrix
    static constexpr int wt = rup + QT * 2;                            // float[4]
    static constexpr int bars = wt + 16;
    // stage full/empty, staging full/empty per half, acc full/empty, matrix full/empty, carry ready
    static constexpr int n_bars = 2 * kBwdStages + 4 + 4 + 2 + kBwdCRing;
    static constexpr int tmem_slot = bars + n_bars * 8;
    static constexpr int abort_flag = tmem_slot + 4;
    static constexpr int total = abort_flag + 4;
};
constexpr int kBwdSmemBytes = BwdSmem::total;   // no alignment slack: see the kernel
static_assert(kBwdSmemBytes <= 227 * 1024, "backward shared memory exceeds the per-CTA limit");

// AGG: the aggregate schedule (split = 2) as its own instantiation: the adjoint entering every tile is the fold of
// the per-tile adjoint aggregates, g_{k-1} = G_k + F_k g_k, carried in a register by the thread that owns the channel.
// PER_STEP: the kind of decay, also as instantiations: 1 % (time-invariant decay) to 2-4 % (per-step decay, long sequences)
// faster under sustained load than one kernel that branches on it.  (The same split of the forward kernel measured
// 3-4 % slower with a per-step decay and 20 % slower for the weighted scan, and was not kept.)
// CONV: the decay convention (1: the decay is given as its logarithm and x comes pre-scaled), instantiated as well:
// another 5-6 % off the launch with a per-step decay, nothing lost with a time-invariant one.
// CUT: the tile-range schedule (split = 1: items cut between thread blocks, adjoints handed on through global memory);
// without it the hand-over code is not in the kernel: 2-3 % faster under sustained load on whole items.
template <bool AGG, bool PER_STEP, bool CONV, bool CUT>
__global__ void __launch_bounds__(kThreads, 1)
ema_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_g,
                  const __grid_constant__ CUtensorMap tm_o, const TcBwdParams p) {
    // The 128-byte-swizzled TMA boxes and MMA descriptors need a 1024-byte-aligned base.  This kernel uses all of
    // the shared memory a CTA may have, so there is no room for aligning by hand: the declaration asks for the
    // alignment, and a base that lacks it ends the kernel before anything is set up (status 0x2ff).
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw;
    const uint32_t sbase = smem_u32(smem);
    if (sbase & 1023u) {
        if (threadIdx.x == 0) atomicCAS(&g_tc_status, 0, 0x2ff);
        return;
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr bool per_step = PER_STEP;
    constexpr int conv = CONV ? 1 : 0;
    const int L = static_cast<int>(p.L);

    float *hs_sm = reinterpret_cast<float *>(smem + BwdSmem::hs);
    float *g_sm = reinterpret_cast<float *>(smem + BwdSmem::g);
    float *rowsc = reinterpret_cast<float *>(smem + BwdSmem::rowsc);
    float *cs_sm = reinterpret_cast<float *>(smem + BwdSmem::cs);
    __half *p_sm = reinterpret_cast<__half *>(smem + BwdSmem::pw);
    __half *wlo_sm = reinterpret_cast<__half *>(smem + BwdSmem::wlo);
    __half *rup_sm = reinterpret_cast<__half *>(smem + BwdSmem::rup);
    float *wt_sm = reinterpret_cast<float *>(smem + BwdSmem::wt);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + BwdSmem::abort_flag);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + BwdSmem::tmem_slot);
    auto bar = [&](int i) { return sbase + BwdSmem::bars + i * 8; };
    constexpr int B_FULL = 0, B_EMPTY = kBwdStages, B_STG_FULL = 2 * kBwdStages, B_STG_EMPTY = B_STG_FULL + 2,
                  B_ACC_FULL = B_STG_EMPTY + 2, B_ACC_EMPTY = B_ACC_FULL + 2, B_MAT_FULL = B_ACC_EMPTY + 2,
                  B_MAT_EMPTY = B_MAT_FULL + 1, B_G = B_MAT_EMPTY + 1;
    constexpr uint32_t kTmemCols = 512;  // 2 stages x (Z | Lam) x 128 columns

    if (tid == 0) {
        for (int i = 0; i < kBwdStages; ++i) { mbar_init(bar(B_FULL + i), 1); mbar_init(bar(B_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_STG_FULL + i), kEpiWarps / 2); mbar_init(bar(B_STG_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar(B_ACC_FULL + i), 1); mbar_init(bar(B_ACC_EMPTY + i), kEpiWarps); }
        mbar_init(bar(B_MAT_FULL), kBuildWarps);
        mbar_init(bar(B_MAT_EMPTY), 1);
        // carry ready: the two halves of the adjoint row and the four warps that fetch the saved state (with
        // aggregates those four warps bring the adjoint as well)
        for (int i = 0; i < kBwdCRing; ++i) mbar_init(bar(B_G + i), AGG ? 4 : 6);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_g);
        prefetch_tmap(&tm_o);
    }
    for (int i = tid; i < BwdSmem::mat_bytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(smem + BwdSmem::m_a1k0)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (warp == 1) {
        tmem_alloc(sbase + BwdSmem::tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done; nothing before this line has touched global memory, everything after it may depend on the kernel
    // before this one on the stream
    grid_dependency_wait();

    // arrival counter of the per-head reduction that follows this kernel (it sits right before the partial sums)
    if (!per_step && blockIdx.x == 0 && tid == 0)
        *reinterpret_cast<unsigned *>(EMA_AT(p, p.da_partial + p.head_partial_offset - 4, 165)) = 0u;
    const Sched sched(p.n_items, p.n_tiles, AGG || CUT);
    // item -> scan row, first channel tile, number of channel tiles (1 or 2)
    auto item_row = [&](int64_t item) { return item / p.n_groups; };
    auto item_dt0 = [&](int64_t item) { return static_cast<int>(item % p.n_groups) * p.sub; };
    // (with a time-invariant decay a work item is always one channel tile: the launcher pairs tiles only to share
    // per-step matrices)
    auto item_nsub = [&](int64_t item) {
        if constexpr (!PER_STEP) return 1;
        const int left = p.n_dtiles - static_cast<int>(item % p.n_groups) * p.sub;
        return left < p.sub ? left : p.sub;
    };
    // (clamped: a decay of exactly 0 would make the prefix sums -inf and their differences NaN; 2^-160 is 0 in fp32,
    // and a small bound keeps the prefix sums of a tile with many such steps precise)
    // lg2.approx (absolute error 2^-22): the decays end up in bf16 matrix elements and in carry factors over 128 steps
    auto log2_decay = [&](float v) { return fmaxf(conv ? v * 1.4426950408889634f : __log2f(v), -160.f); };

    if (warp < 4) {
        reg_dec<kRegsLight>();
        if (warp == 0) {
            // ---------------- TMA producer ----------------
            if (lane == 0) {
                uint32_t it = 0;
                for (int pi = 0; pi < sched.n && !*abort_flag; ++pi) {
                    if (!sched.split && sched.n > 1 && pi == sched.n - 1) grid_dependents_launch();   // (see the forward kernel)
                    const Piece pc = sched.get<false>(pi);
                    const int dt0 = item_dt0(pc.item), nsub = item_nsub(pc.item);
                    const int64_t row = item_row(pc.item);
                    const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
                    for (int k = pc.k1 - 1; k >= pc.k0 && !*abort_flag; --k)
                    for (int u = 0; u < nsub; ++u, ++it) {
                        const int s = it % kBwdStages;
                        const uint32_t ph = (it / kBwdStages) & 1;
                        if (!mbar_wait(bar(B_EMPTY + s), ph ^ 1, abort_flag, 11)) break;
                        mbar_expect_tx(bar(B_FULL + s), 2 * kTileBytes);
                        const uint32_t dst = sbase + BwdSmem::xg + s * 2 * kTileBytes;
                        const int c0 = (dt0 + u) * DT;
                        tma_load_4d(dst, &tm_x, bar(B_FULL + s), c0, hi, k * QT, bi);
                        tma_load_4d(dst + kBlockBytes, &tm_x, bar(B_FULL + s), c0 + kBlockCols, hi, k * QT, bi);
                        tma_load_4d(dst + kTileBytes, &tm_g, bar(B_FULL + s), c0, hi, k * QT, bi);
                        tma_load_4d(dst + kTileBytes + kBlockBytes, &tm_g, bar(B_FULL + s), c0 + kBlockCols, hi, k * QT, bi);
                    }
                }
                grid_dependents_launch();   // the last loads are on their way (see the forward kernel)
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0) {
                uint32_t it = 0, mt = 0;
                int cur_head = -1;
                // K block 0 / 1 of each matrix (see BwdSmem): descriptor bases
                const uint64_t a1d[2] = {make_desc_sw128(sbase + BwdSmem::m_a1k0, 16, 1024),
                                         make_desc_sw128(sbase + BwdSmem::m_z, 16, 1024)};
                const uint64_t ud[2] = {make_desc_sw128(sbase + BwdSmem::m_u00, 16, 1024),
                                        make_desc_sw128(sbase + BwdSmem::m_uk1, 16, 1024)};
                for (int pi = 0; pi < sched.n && !*abort_flag; ++pi) {
                    const Piece pc = sched.get<false>(pi);
                    const int hi = static_cast<int>(item_row(pc.item) % p.h);
                    const int nsub = item_nsub(pc.item);
                    for (int k = pc.k1 - 1; k >= pc.k0 && !*abort_flag; --k)
                    for (int u = 0; u < nsub; ++u, ++it) {
                        const int s = it % kBwdStages;
                        const uint32_t ph = (it / kBwdStages) & 1;
                        const int acc = it & 1;
                        const uint32_t aph = (it >> 1) & 1;
                        if (u == 0 && (per_step || hi != cur_head)) {
                            // single matrix buffer: hand it back to the builders once the MMAs issued so far are done
                            if (!per_step && mt > 0) umma_commit(bar(B_MAT_EMPTY));
                            if (!mbar_wait(bar(B_MAT_FULL), mt & 1, abort_flag, 12)) break;
                            cur_head = hi;
                            ++mt;
                        }
                        if (!mbar_wait(bar(B_FULL + s), ph, abort_flag, 13)) break;
                        if (!mbar_wait(bar(B_ACC_EMPTY + acc), aph ^ 1, abort_flag, 14)) break;
                        tc_fence_after_sync();
                        const uint64_t xd0 = tile_desc(sbase + BwdSmem::xg + s * 2 * kTileBytes);
                        const uint64_t gd0 = xd0 + (kTileBytes >> 4);
                        const uint32_t d_z = tmem_base + acc * 2 * DT, d_l = d_z + DT;
    #pragma unroll
                        for (int kb = 0; kb < QT / 16; ++kb)
                            umma_bf16(d_z, a1d[kb >> 2] + (((kb & 3) * 32) >> 4), xd0 + ((kb * 2048) >> 4), kIdesc, kb > 0 ? 1u : 0u);
    #pragma unroll
                        for (int kb = 0; kb < QT / 16; ++kb)
                            umma_bf16(d_l, ud[kb >> 2] + (((kb & 3) * 32) >> 4), gd0 + ((kb * 2048) >> 4), kIdesc, kb > 0 ? 1u : 0u);
                        umma_commit(bar(B_EMPTY + s));   // the stage is free as soon as the MMAs have read it
                        umma_commit(bar(B_ACC_FULL + acc));
                        if (per_step && u == nsub - 1) umma_commit(bar(B_MAT_EMPTY));
                    }
                }
            }
        } else {
            // ---------------- TMA store issuer ----------------
            if (tid == kStoreThread) {
                uint32_t it = 0;
                for (int pi = 0; pi < sched.n && !*abort_flag; ++pi) {
                    const Piece pc = sched.get<false>(pi);
                    const int dt0 = item_dt0(pc.item), nsub = item_nsub(pc.item);
                    const int64_t row = item_row(pc.item);
                    const int bi = static_cast<int>(row / p.h), hi = static_cast<int>(row % p.h);
                    for (int k = pc.k1 - 1; k >= pc.k0 && !*abort_flag; --k)
                    for (int u = 0; u < nsub; ++u, ++it) {
                        const int dtile = dt0 + u;
                        const bool two = dtile * DT + kBlockCols < p.d;   // the second 64-channel block exists
                        const uint32_t src = sbase + BwdSmem::ostage;
                        if (!mbar_wait(bar(B_STG_FULL + 0), it & 1, abort_flag, 19)) break;
                        tma_store_4d(&tm_o, src, dtile * DT, hi, k * QT, bi);
                        tma_store_commit();
                        if (!mbar_wait(bar(B_STG_FULL + 1), it & 1, abort_flag, 20)) break;
                        if (two) tma_store_4d(&tm_o, src + kBlockBytes, dtile * DT + kBlockCols, hi, k * QT, bi);
                        tma_store_commit();
                        tma_store_wait_read<1>();          // block 0 has been read: hand it back to its four warps
                        mbar_arrive(bar(B_STG_EMPTY + 0));
                        tma_store_wait_read<0>();
                        mbar_arrive(bar(B_STG_EMPTY + 1));
                    }
                }
                tma_store_wait_all();
            }
        }
    } else if (tid < kBuildThread0) {
        reg_inc<RoleRegs<PER_STEP>::epilogue>();
        // ---------------- epilogue ----------------
        // thread (q, lane, half): row m = 32 q + lane, channels [64 half, 64 half + 64) of the tile, 32 at a time.
        // The two threads of row 0 are the serial carry chain (the adjoint handed to the tile on the left).
        const int q = warp & 3;
        const int half = (warp - kEpiThread0 / 32) >> 2;
        const int m = q * 32 + lane;
        const bool loader = half == 0;  // 128 threads: thread m fetches channel m of the saved states
        uint32_t it = 0, mt = 0;
        int cur_head = -1;
        for (int pi = 0; pi < sched.n; ++pi) {
            const Piece pc = sched.get<false>(pi);
            const int dt0 = item_dt0(pc.item), nsub = item_nsub(pc.item);
            const int64_t row = item_row(pc.item);
            const int hi = static_cast<int>(row % p.h);
            const bool publish = CUT && pc.k0 > 0;   // the item continues to the left in another CTA: hand it the adjoint
            // cut blockIdx.x is this CTA's left edge (it publishes there), cut blockIdx.x + 1 its right edge (it reads there)
            float *carry_out = p.carry + static_cast<int64_t>(blockIdx.x) * kCarryFloats;
            float hs_next = 0.f;
            float g_reg0 = 0.f, g_reg1 = 0.f;   // AGG: the adjoint entering the current tile, channel m of each sub-tile (loaders)
            if (loader) {
                if (CUT && pc.k1 < p.n_tiles) {   // left part of a cut item: the adjoint comes from the CTA that made the right part
                    if (lane == 0) wait_carry(EMA_AT(p, p.flags + blockIdx.x + 1, 150), 2u * nsub, abort_flag, 23);
                    __syncwarp();
                }
                for (int u = 0; u < nsub; ++u) {
                    const int c0u = (dt0 + u) * DT;
                    const bool ok = c0u + m < p.d;
                    const int slot0 = (it + u) % kBwdCRing;
                    hs_sm[slot0 * DT + m] =
                        ok ? *EMA_AT(p, p.tile_states + (row * p.n_tiles + (pc.k1 - 1)) * p.d + c0u + m, 151) : 0.f;
                    float gv;
                    if (CUT && pc.k1 < p.n_tiles) {
                        gv = __ldcg(EMA_AT(p, p.carry + static_cast<int64_t>(blockIdx.x + 1) * kCarryFloats + u * DT + m, 152));
                    } else {
                        gv = (p.dfinal_state && ok) ? *EMA_AT(p, p.dfinal_state + row * p.d + c0u + m, 153) : 0.f;
                        if (AGG && pc.k1 < p.n_tiles && ok)
                            gv = fold_adjoint_after(p.agg_vec + row * p.n_tiles * p.d + c0u + m,
                                                    p.agg_fac + row * p.n_tiles, p.d, pc.k1, p.n_tiles, gv,
                                                    BoundsRef{p.bounds});
                    }
                    g_sm[slot0 * DT + m] = gv;
                    if (u == 0) g_reg0 = gv; else g_reg1 = gv;
                }
            }
            bar_sync(1, kEpiThreads);
            for (int u = 0; u < nsub; ++u) {
                if (!AGG && m == 0) mbar_arrive(bar(B_G + (it + u) % kBwdCRing));
                if (loader && lane == 0) mbar_arrive(bar(B_G + (it + u) % kBwdCRing));
            }
            for (int k = pc.k1 - 1; k >= pc.k0; --k)
            for (int u = 0; u < nsub; ++u, ++it) {
                const int dtile = dt0 + u;
                const int c0 = dtile * DT;
                const bool ch_ok = loader && c0 + m < p.d;
                const float *ts_item = p.tile_states + row * p.n_tiles * p.d + c0 + m;
                // Partial sums of the decay gradient, in the layout of the CUDA-core kernel (so that a suffix re-scan by
                // that kernel can overwrite some tiles of a pass made by this one): one slice per 64 channels,
                // [row][slice][t] for a per-step decay, [row][slice][tile][8] for a per-head decay.
                const int slice = 2 * dtile + half;
                const bool slice_ok = slice < p.n_dt64;   // the second half of the last tile may hold no channels
                float *dap_step = p.da_partial + (row * p.n_dt64 + slice) * (static_cast<int64_t>(p.n_tiles) * QT);
                float *dap_head = p.da_partial + p.head_partial_offset + (row * p.n_dt64 + slice) * p.n_tiles * 8;
                const int acc = it & 1, slot = it % kBwdCRing, nslot = (it + nsub) % kBwdCRing;
                const uint32_t aph = (it >> 1) & 1, gph = (it / kBwdCRing) & 1;
                if (u == 0 && (per_step || hi != cur_head)) { cur_head = hi; ++mt; }
                // prefetch the saved state of the next tile to the left while this one is being finished
                if (loader && k > pc.k0) hs_next = ch_ok ? *EMA_AT(p, ts_item + static_cast<int64_t>(k - 1) * p.d, 154) : 0.f;
                // AGG: this tile's adjoint aggregate, for the adjoint the tile on the left receives
                float agg_g = 0.f, agg_f = 0.f;
                if (AGG && loader && k > pc.k0) {
                    agg_f = *EMA_AT(p, p.agg_fac + row * p.n_tiles + k, 155);
                    if (ch_ok) agg_g = *EMA_AT(p, p.agg_vec + (row * p.n_tiles + k) * p.d + c0 + m, 156);
                }
                if (lane == 0) mbar_wait(bar(B_ACC_FULL + acc), aph, abort_flag, 15);
                __syncwarp();
                tc_fence_after_sync();
                const float *rs = rowsc + ((mt - 1) % kRowRing) * 3 * QT;
                const float Eprev = rs[m], a_m = rs[2 * QT + m];
                const float p_m = conv ? 1.f : 1.f - a_m;
                // F: a time-invariant decay uses one Toeplitz table; the rightmost tile of the sequence stops at
                // step L-1, where the adjoint entering from the right applies undamped
                float F = rs[QT + m];
                if (!per_step && k == p.n_tiles - 1) {   // (always the first tile of a piece that starts at the end)
                    const int lim = L - k * QT;  // valid rows in this tile
                    float f = 1.f;
                    for (int j = m + 1; j < lim; ++j) f *= a_m;
                    F = f;
                }
                if (lane == 0) mbar_wait(bar(B_G + slot), gph, abort_flag, 16);
                __syncwarp();
                const int t = k * QT + m;
                float2 dacc2 = make_float2(0.f, 0.f);   // even / odd columns
                // dx staging: this half's 64-channel block, free once the store of the previous tile has read it
                uint8_t *stg = smem + BwdSmem::ostage + half * kBlockBytes;
                if (lane == 0) mbar_wait(bar(B_STG_EMPTY + half), (it & 1) ^ 1, abort_flag, 17);
                __syncwarp();
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {
                    const int cb = half * 64 + pass * 32;
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 2 * DT + cb;
                    float z[32], lam[32];
                    __syncwarp();  // single-thread branches of the previous pass have rejoined
                    tmem_ld32(taddr, z);
                    tmem_ld32(taddr + DT, lam);
                    tmem_ld_wait();
                    if (pass == 1) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(B_ACC_EMPTY + acc));
                    }
                    const float *hin = hs_sm + slot * DT + cb;
                    const float *gin = g_sm + slot * DT + cb;
                    const float2 F2 = make_float2(F, F);   // two columns per instruction (packed fp32 math) throughout
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const float4 gv = *reinterpret_cast<const float4 *>(gin + c);
                        const float2 lo = __ffma2_rn(F2, make_float2(gv.x, gv.y), make_float2(lam[c], lam[c + 1]));
                        const float2 hi2 = __ffma2_rn(F2, make_float2(gv.z, gv.w), make_float2(lam[c + 2], lam[c + 3]));
                        lam[c] = lo.x; lam[c + 1] = lo.y; lam[c + 2] = hi2.x; lam[c + 3] = hi2.y;
                    }
                    if (m == 0 && !(AGG && k > pc.k0)) {
                        if (k > pc.k0) {  // row 0 of the adjoint is what the tile on the left receives
                            float *gout = g_sm + nslot * DT + cb;
#pragma unroll
                            for (int c = 0; c < 32; c += 4)
                                *reinterpret_cast<float4 *>(gout + c) = make_float4(lam[c], lam[c + 1], lam[c + 2], lam[c + 3]);
                            if (pass == 1) mbar_arrive(bar(B_G + nslot));
                        } else if (publish) {   // the tile on the left is another CTA's
                            float *co = carry_out + u * DT + cb;
#pragma unroll
                            for (int c = 0; c < 32; c += 4)
                                *reinterpret_cast<float4 *>(EMA_ATN(p, co + c, 157, 16)) =
                                    make_float4(lam[c], lam[c + 1], lam[c + 2], lam[c + 3]);
                            if (pass == 1) {   // this half of the carry is complete
                                __threadfence();
                                atomicAdd(EMA_AT(p, p.flags + blockIdx.x, 158), 1u);
                            }
                        } else if (p.dinit_state && pc.k0 == 0) {
                            float *di = p.dinit_state + row * p.d + c0 + cb;
#pragma unroll
                            for (int c = 0; c < 32; ++c)
                                if (c0 + cb + c < p.d) *EMA_AT(p, di + c, 159) = a_m * lam[c];
                        }
                    }
                    const float2 Ep2 = make_float2(Eprev, Eprev), p2 = make_float2(p_m, p_m);
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const float4 hv = *reinterpret_cast<const float4 *>(hin + c);
                        const float2 z0 = __ffma2_rn(Ep2, make_float2(hv.x, hv.y), make_float2(z[c], z[c + 1]));
                        const float2 z1 = __ffma2_rn(Ep2, make_float2(hv.z, hv.w), make_float2(z[c + 2], z[c + 3]));
                        dacc2 = __ffma2_rn(make_float2(lam[c], lam[c + 1]), z0, dacc2);
                        dacc2 = __ffma2_rn(make_float2(lam[c + 2], lam[c + 3]), z1, dacc2);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 d0 = __fmul2_rn(p2, make_float2(lam[8 * j], lam[8 * j + 1]));
                        const float2 d1 = __fmul2_rn(p2, make_float2(lam[8 * j + 2], lam[8 * j + 3]));
                        const float2 d2 = __fmul2_rn(p2, make_float2(lam[8 * j + 4], lam[8 * j + 5]));
                        const float2 d3 = __fmul2_rn(p2, make_float2(lam[8 * j + 6], lam[8 * j + 7]));
                        const uint4 qv = make_uint4(pack_bf16x2(d0.x, d0.y), pack_bf16x2(d1.x, d1.y),
                                                    pack_bf16x2(d2.x, d2.y), pack_bf16x2(d3.x, d3.y));
                        *reinterpret_cast<uint4 *>(stg + sw128_offset(m, pass * 4 + j)) = qv;
                    }
                }
                if (loader && k > pc.k0) {  // the saved state the tile on the left will need
                    if (AGG) {   // and the adjoint entering it
                        const float gn = fmaf(agg_f, u == 0 ? g_reg0 : g_reg1, agg_g);
                        if (u == 0) g_reg0 = gn; else g_reg1 = gn;
                        g_sm[nslot * DT + m] = gn;
                    }
                    hs_sm[nslot * DT + m] = hs_next;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_G + nslot));
                }
                float dacc = dacc2.x + dacc2.y;
                if (conv) dacc *= a_m;
                if (t >= L) dacc = 0.f;
                if (per_step) {
                    if (t < L && slice_ok) *EMA_AT(p, dap_step + t, 160) = dacc;
                } else {
                    float wsum = dacc;
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
                    if (lane == 0 && slice_ok) {   // four warps per slice fill its eight slots
                        *EMA_AT(p, dap_head + k * 8 + q * 2, 161) = wsum;
                        *EMA_AT(p, dap_head + k * 8 + q * 2 + 1, 162) = 0.f;
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_STG_FULL + half));
            }
        }
    } else {
        reg_dec<RoleRegs<PER_STEP>::builder>();
        // ---------------- matrix builders ----------------
        const int bt = tid - kBuildThread0;   // 0-255; threads 0-127 also own row r = bt of the per-row tables
        const int r = bt & 127;
        const bool row_owner = bt < 128;
        uint32_t mt = 0;
        int cur_head = -1;
        const float diag = conv ? 0.f : -1.f;
        OffGeom oga, ogu;
        DiagGeom dga, dgu;
        // A1: K block 0 holds every row; K block 1 only rows 64-127 (stored from row 64 on)
        make_geom<false, 1>(bt, oga, dga, [](int m, int c) {
            return c < 8 ? BwdSmem::m_a1k0 + sw128_offset(m, c) : BwdSmem::m_a111 + sw128_offset(m - 64, c - 8);
        });
        // U: K block 0 only rows 0-63; K block 1 every row
        make_geom<true, 0>(bt, ogu, dgu, [](int m, int c) {
            return c < 8 ? BwdSmem::m_u00 + sw128_offset(m, c) : BwdSmem::m_uk1 + sw128_offset(m, c - 8);
        });
        const uint8_t *cs_b = smem + BwdSmem::cs, *p_b = smem + BwdSmem::pw, *wlo_b = smem + BwdSmem::wlo,
                      *rup_b = smem + BwdSmem::rup;
        // v: raw decay value of step r of the tile; v_edge: of the step right after the tile (identity past L);
        // both are read from the row owners only
        auto build = [&](float v, float v_edge) {
            const float l2 = log2_decay(v);
            float to_end = 0.f, from_start = 0.f;
            builder_scan(l2, bt, cs_sm, wt_sm, to_end, from_start);
            if (row_owner) {
                const float pw = conv ? 1.f : 1.f - v;
                const float pws = pw * static_cast<float>(1 << kHalfShift);
                p_sm[r] = __float2half_rn(pws);
                wlo_sm[r] = __float2half_rn(pws * ex2_approx(to_end));
                rup_sm[r] = __float2half_rn(ex2_approx(from_start));
            }
            bar_sync(2, kBuildThreads);
            RowChunks ca, cu;
            compute_diag_lower_half<1>(dga, cs_b, p_b, diag, ca);
            compute_off_half<false>(oga, cs_b, wlo_b, ca);
            compute_diag_upper(dgu, cs_b, cu);
            compute_off_half<true>(ogu, cs_b, rup_b, cu);
            const float cs_r = cs_sm[r];
            const float Eprev = ex2_approx(cs_r - l2);                       // prod_{j<r} a_j
            const float Fr = ex2_approx(cs_sm[QT - 1] - cs_r + log2_decay(v_edge));
            if (lane == 0) mbar_wait(bar(B_MAT_EMPTY), (mt & 1) ^ 1, abort_flag, 18);
            __syncwarp();
            store_matrix(oga, dga, smem, ca);
            store_matrix(ogu, dgu, smem, cu);
            if (row_owner) {
                float *rs = rowsc + (mt % kRowRing) * 3 * QT;
                rs[r] = Eprev;
                rs[QT + r] = Fr;
                rs[2 * QT + r] = conv ? ex2_approx(l2) : v;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_MAT_FULL));
            ++mt;
        };
        const float ident = conv ? 0.f : 1.f;  // raw value of an identity step
        for (int pi = 0; pi < sched.n; ++pi) {
            const Piece pc = sched.get<false>(pi);
            const int64_t row = item_row(pc.item);
            const int64_t bi = row / p.h, hi = row % p.h;
            const float *arow = p.decay + (per_step ? bi * p.a_sb + hi * p.a_sh : hi * p.a_sh);
            if (!per_step) {
                if (static_cast<int>(hi) != cur_head) {
                    cur_head = static_cast<int>(hi);
                    const float v = *EMA_AT(p, arow, 163);
                    build(v, v);
                }
                continue;
            }
            auto load_v = [&](int t) {
                return (row_owner && t >= 0 && t < L) ? *EMA_AT(p, arow + static_cast<int64_t>(t) * p.a_sl, 164) : ident;
            };
            float v_next = load_v((pc.k1 - 1) * QT + r);
            float edge_next = load_v(pc.k1 * QT);  // past the end (identity) unless the item continues in another CTA
            for (int k = pc.k1 - 1; k >= pc.k0; --k) {
                const float v = v_next, edge = edge_next;
                if (k > pc.k0) {
                    v_next = load_v((k - 1) * QT + r);
                    edge_next = load_v(k * QT);
                }
                build(v, edge);
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

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded waits: one small thread block waits, with a short limit, for something that never
// happens - an mbarrier nobody arrives on (mode 0) or a global arrival counter nobody increments (mode 1) - through
// the very wait functions the kernels above use.  The wait runs out, records 0x100 | site in the status word and
// returns; nothing else is in flight (no copies, no tensor memory), so the kernel simply ends.
// ---------------------------------------------------------------------------------------------
__global__ void selftest_wait_kernel(int mode, uint32_t limit, const unsigned *never_set) {
    __shared__ __align__(8) uint64_t bar_storage;
    __shared__ int abort_flag_sm;
    volatile int *abort_flag = &abort_flag_sm;
    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(smem_u32(&bar_storage), 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (mode == 0) mbar_wait_limit(smem_u32(&bar_storage), 0, abort_flag, 0x7e, limit);
        else wait_carry(never_set, 1u, abort_flag, 0x7f, limit);
    }
    __syncthreads();
    // every other thread sees the abort flag the way the roles of the real kernels do
    if (threadIdx.x == 1 && !*abort_flag) atomicCAS(&g_tc_status, 0, 0x3ff);
}

}  // namespace tc

// ---------------------------------------------------------------------------------------------
// fp32 forward on the CUDA cores, fed by TMA
// ---------------------------------------------------------------------------------------------
// The exact fp32 recurrence of the CUDA-core family (same function template, same arithmetic, bit-identical results)
// with the x tiles brought in by TMA: a ring of three [128 steps x 64 channels] fp32 boxes per thread block and two
// thread blocks per SM keep 192 KB of loads in flight per SM, where the register prefetch of the plain kernel
// keeps 64 KB.  One thread issues the copies; a stage is refilled right after the tile's block-wide barrier, by which
// time every thread has taken its values out of it.
namespace tmafeed {

constexpr int kStages = 3;
constexpr int kChannels = kFmaCT * 4;                       // 64 channels per thread block (one TMA box)
constexpr int kStageBytes = kFmaTile * kChannels * 4;       // 32 KB
constexpr int kCtrlBytes = 64;                              // mbarriers, abort flag
static_assert(kChannels == tc::kBlockCols && kFmaTile == tc::QT, "the tensor map's box is [128 steps x 64 channels]");

// T: element type (fp32: 32 KB stages; bf16: 16 KB stages); STAGES: depth of the ring
template <typename T, int STAGES>
struct TmaFeed {
    static constexpr int kRowBytes = kChannels * static_cast<int>(sizeof(T));
    static constexpr int kStageBytes = kFmaTile * kRowBytes;
    static constexpr int kStages = STAGES;
    static constexpr int kSmemBytes = STAGES * kStageBytes + kCtrlBytes + 128;   // + slack to align the ring to 128 bytes
    raw_t<T, 4> cur[kFmaSB];
    const CUtensorMap *tm;
    uint8_t *stages;
    uint32_t bars;            // shared-space address of kStages mbarriers
    volatile int *abort_flag;
    int c0, hi, bi, n_tiles, tid, off;   // off: bytes from the start of a stage to this thread's first value

    __device__ __forceinline__ void issue(int k) {   // one thread
        const int s = k % kStages;
        tc::mbar_expect_tx(bars + 8 * s, kStageBytes);
        tc::tma_load_4d(tc::smem_u32(stages + s * kStageBytes), tm, bars + 8 * s, c0, hi, k * kFmaTile, bi);
    }
    __device__ __forceinline__ void init(const FusedParams &, const T *, bool, int, int) {
        if (tid == 0) {
            for (int s = 0; s < kStages; ++s) tc::mbar_init(bars + 8 * s, 1);
            *abort_flag = 0;
            tc::fence_barrier_init();
            for (int k = 0; k < kStages && k < n_tiles; ++k) issue(k);
        }
    }
    __device__ __forceinline__ void begin(int k, bool) {
        const int s = k % kStages;
        tc::mbar_wait(bars + 8 * s, (k / kStages) & 1, abort_flag, 40);   // bounded; steps and channels past the end arrive as zeros
        const uint8_t *src = stages + s * kStageBytes + off;
#pragma unroll
        for (int i = 0; i < kFmaSB; ++i) cur[i] = *reinterpret_cast<const raw_t<T, 4> *>(src + i * kRowBytes);
    }
    __device__ __forceinline__ void after_barrier(int k) {
        if (tid == 0 && k + kStages < n_tiles && !*abort_flag) issue(k + kStages);
    }
    __device__ __forceinline__ void end() {}
    __device__ __forceinline__ void finish() {
        if (*abort_flag)   // a wait ran out: give copies still in flight time to land before shared memory is released
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
};

template <typename T, int STAGES, bool WEIGHTED>
__global__ void __launch_bounds__(kFmaThreads, 2)
ema_fwd_fma_tma_kernel(const __grid_constant__ CUtensorMap tm_x, const FusedParams p) {
    extern __shared__ uint8_t dyn_smem[];
    uint8_t *base = dyn_smem + ((128u - (tc::smem_u32(dyn_smem) & 127u)) & 127u);
    using Feed = TmaFeed<T, STAGES>;
    Feed feed;
    feed.tm = &tm_x;
    feed.stages = base;
    feed.bars = tc::smem_u32(base + STAGES * Feed::kStageBytes);
    feed.abort_flag = reinterpret_cast<volatile int *>(base + STAGES * Feed::kStageBytes + 8 * STAGES);
    feed.tid = threadIdx.x;
    const int lc = threadIdx.x % kFmaCT, sub = threadIdx.x / kFmaCT;
    feed.off = (sub * kFmaSB * kChannels + lc * 4) * static_cast<int>(sizeof(T));
    const int64_t row = blockIdx.x / p.n_dtiles;
    feed.c0 = static_cast<int>(blockIdx.x % p.n_dtiles) * kChannels;
    feed.bi = static_cast<int>(row / p.h);
    feed.hi = static_cast<int>(row % p.h);
    feed.n_tiles = p.n_tiles;
    ema_fwd_fma_body<T, 4, WEIGHTED>(p, feed);
}

// Backward: x and dy tiles of the same steps share a stage (64 KB); three stages and one thread block per SM (the
// backward's registers allow no more) keep 192 KB in flight.  Tiles are walked from the last to the first.
constexpr int kBwdStageBytes = 2 * kStageBytes;
constexpr int kBwdSmemBytes = kStages * kBwdStageBytes + kCtrlBytes + 128;   // + slack to align the ring to 128 bytes

struct TmaFeedBwd {
    uint4 xc[kFmaSB], gc[kFmaSB];
    const CUtensorMap *tm_x, *tm_g;
    uint8_t *stages;
    uint32_t bars;
    volatile int *abort_flag;
    int c0, hi, bi, n_tiles, tid, off;

    __device__ __forceinline__ void issue(int kk) {   // one thread; iteration kk handles tile n_tiles - 1 - kk
        const int s = kk % kStages, t0 = (n_tiles - 1 - kk) * kFmaTile;
        const uint32_t dst = tc::smem_u32(stages + s * kBwdStageBytes);
        tc::mbar_expect_tx(bars + 8 * s, kBwdStageBytes);
        tc::tma_load_4d(dst, tm_x, bars + 8 * s, c0, hi, t0, bi);
        tc::tma_load_4d(dst + kStageBytes, tm_g, bars + 8 * s, c0, hi, t0, bi);
    }
    __device__ __forceinline__ void fetch(int kk) {
        const int s = kk % kStages;
        tc::mbar_wait(bars + 8 * s, (kk / kStages) & 1, abort_flag, 41);   // bounded; steps and channels past the end are zeros
        const uint8_t *src = stages + s * kBwdStageBytes + off;
#pragma unroll
        for (int i = 0; i < kFmaSB; ++i) {
            xc[i] = *reinterpret_cast<const uint4 *>(src + i * kChannels * 4);
            gc[i] = *reinterpret_cast<const uint4 *>(src + kStageBytes + i * kChannels * 4);
        }
    }
    __device__ __forceinline__ void init(const FusedParams &, const float *, const float *, bool, int, int, int) {
        if (tid == 0) {
            for (int s = 0; s < kStages; ++s) tc::mbar_init(bars + 8 * s, 1);
            *abort_flag = 0;
            tc::fence_barrier_init();
            for (int kk = 0; kk < kStages && kk < n_tiles; ++kk) issue(kk);
        }
        __syncthreads();   // the barriers exist before anyone waits on them
        fetch(0);
    }
    __device__ __forceinline__ void begin(int kk, int, bool) {
        if (kk > 0) fetch(kk);
    }
    __device__ __forceinline__ void after_barrier(int kk) {
        if (tid == 0 && kk + kStages < n_tiles && !*abort_flag) issue(kk + kStages);
    }
    __device__ __forceinline__ void end(int, bool) {}
    __device__ __forceinline__ void finish() {
        if (*abort_flag)
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
};

__global__ void __launch_bounds__(kFmaThreads, 1)
ema_bwd_fma_tma_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_g,
                       const FusedParams p) {
    extern __shared__ uint8_t dyn_smem[];
    uint8_t *base = dyn_smem + ((128u - (tc::smem_u32(dyn_smem) & 127u)) & 127u);
    TmaFeedBwd feed;
    feed.tm_x = &tm_x;
    feed.tm_g = &tm_g;
    feed.stages = base;
    feed.bars = tc::smem_u32(base + kStages * kBwdStageBytes);
    feed.abort_flag = reinterpret_cast<volatile int *>(base + kStages * kBwdStageBytes + 8 * kStages);
    feed.tid = threadIdx.x;
    const int lc = threadIdx.x % kFmaCT, sub = threadIdx.x / kFmaCT;
    feed.off = (sub * kFmaSB * kChannels + lc * 4) * 4;
    const int64_t row = blockIdx.x / p.n_dtiles;
    feed.c0 = static_cast<int>(blockIdx.x % p.n_dtiles) * kChannels;
    feed.bi = static_cast<int>(row / p.h);
    feed.hi = static_cast<int>(row % p.h);
    feed.n_tiles = p.n_tiles;
    ema_bwd_fma_body<float, 4>(p, feed);
}

}  // namespace tmafeed

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// looked up once; the initialisation of a function-local static is safe when several host threads arrive together
EncodeTiledFn encode_fn() {
    static const EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(ptr);
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}

// bf16 tensor [b, L, h, d] with element strides (sb, sl, sh), box = [64 channels, 1, 128 steps, 1] (half a tile),
// 128-byte swizzle; out-of-range parts of a box read as zero and are not written.
// bf16 (the default): 64-channel boxes in the 128-byte swizzle the MMA descriptors expect; fp32: dense 64-channel boxes
int make_tmap(CUtensorMap *tm, const void *base, int64_t b, int64_t L, int64_t h, int64_t d, int64_t sb,
              int64_t sl, int64_t sh, bool f32 = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return EMA_ERR_CUDA;
    // cuTensorMapEncodeTiled is a driver call and wants a context current on this thread.  A thread that has
    // made no runtime call yet (e.g. an autograd worker on device 0) has none: bind the device's primary context.
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return EMA_ERR_CUDA;
    // a dimension of extent 1 may carry any stride; give it a legal one
    if (h == 1) sh = d;
    if (L == 1) sl = h * d;
    if (b == 1) sb = L * sl;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(L),
                                static_cast<cuuint64_t>(b)};
    const cuuint64_t es = f32 ? 4 : 2;
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(sh) * es, static_cast<cuuint64_t>(sl) * es,
                                   static_cast<cuuint64_t>(sb) * es};
    const cuuint32_t box[4] = {tc::kBlockCols, 1, tc::QT, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    f32 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? EMA_OK : EMA_ERR_UNSUPPORTED;
}

// SM count of the CURRENT device, cached per device (a process may drive GPUs of different sizes)
int sm_count() {
    constexpr int kMaxDev = 64;
    static std::atomic<int> cache[kMaxDev];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < kMaxDev) {
        const int c = cache[dev].load(std::memory_order_relaxed);
        if (c > 0) return c;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < kMaxDev) cache[dev].store(n, std::memory_order_relaxed);
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

// Scratch of the split schedule: one arrival counter and 128 floats of carry per cut between two thread blocks'
// ranges, for up to kMaxSplitGrid thread blocks (one per SM).  Its size does not depend on the problem.
constexpr int kMaxSplitGrid = 512;
static size_t sync_flag_bytes() { return static_cast<size_t>(kMaxSplitGrid + 1) * 4 / 256 * 256 + 256; }
static size_t carry_bytes() {
    return sync_flag_bytes() + static_cast<size_t>(kMaxSplitGrid + 1) * tc::kCarryFloats * sizeof(float);
}
// 0: whole items only; 1: cut items when that fills the GPU better (default); 2: as 1, and use the aggregate
// schedule for every problem it can take, however small (tests)
static std::atomic<int> g_split{-1};
static int split_setting() {
    int v = g_split.load(std::memory_order_relaxed);
    if (v < 0) {
        const char *e = getenv("EMA_B200_SPLIT");
        v = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
        g_split.store(v, std::memory_order_relaxed);
    }
    return v;
}
int tc_set_split(int on) {
    const int before = split_setting();
    g_split.store(on < 0 ? 0 : (on > 2 ? 2 : on), std::memory_order_relaxed);
    return before;
}
// SMs the split schedule leaves free for small kernels of other streams (a collective that overlaps the scan):
// a thread block that has to wait for such a kernel to leave its SM would finish late by that kernel's run time
// and hold the whole grid back.
static int spare_sms() {
    static const int n = [] {
        const char *e = getenv("EMA_B200_SPARE_SMS");
        const int v = e ? atoi(e) : 2;
        return v < 0 ? 0 : (v > 16 ? 16 : v);
    }();
    return n;
}
// Few work items: with one item per thread block fewer than this share (percent) of the SMs would have work.  Then the
// items are cut into pieces that start from folded per-tile aggregates (one more pass over x, or dy, to make them).
static int few_items_percent() {
    static const int n = [] {
        const char *e = getenv("EMA_B200_AGG_BELOW");
        const int v = e ? atoi(e) : 65;
        return v < 0 ? 0 : (v > 100 ? 100 : v);
    }();
    return n;
}
// Would the aggregate schedule be used for a problem of this size (given scratch)?  rows = scan rows.
bool tc_wants_aggregates(int64_t rows, int64_t L, int64_t d) {
    const int setting = split_setting();
    if (setting == 0 || rows <= 0 || L <= 0 || d <= 0) return false;
    const int sms = sm_count();
    const int64_t n_tiles = (L + tc::QT - 1) / tc::QT, n_dtiles = (d + tc::DT - 1) / tc::DT;
    if (n_tiles < 2 || sms > kMaxSplitGrid) return false;
    if (setting == 2) return true;
    return n_tiles >= 4 && rows * n_dtiles * 100 < static_cast<int64_t>(sms) * few_items_percent();
}
// scratch of the tensor-core kernels for one direction: the carries of the split schedule, and one buffer of
// per-tile aggregates when the problem is one the aggregate schedule would take
size_t tc_sync_bytes(int64_t rows, int64_t L, int64_t d) {
    return carry_bytes() + (tc_wants_aggregates(rows, L, d) ? tile_aggregate_bytes(rows, L, d) : 0);
}

static thread_local int g_last_schedule = -1;
int tc_last_schedule() { return g_last_schedule; }

// How a launch is laid out: the grid, the schedule, and how channel tiles are grouped into work items.
struct Plan {
    int grid, split, sub, n_groups, n_items;
    float *carry;
    unsigned *flags;
    float *agg;
};
// Decides the schedule.  Aggregates (split 2) when there are few work items and the caller gave scratch for them;
// otherwise whole items per CTA when they divide evenly (or when there is no scratch), else one CTA per SM, each with a
// contiguous range of tiles (tc::Sched, split 1; clears the arrival counters on the stream).
static int make_plan(const FusedParams &fp, bool allow_carry_split, bool allow_aggregates, cudaStream_t stream, Plan *pl) {
    const int sms = sm_count();
    const int64_t rows = fp.b * fp.h;
    const int n_tiles = static_cast<int>((fp.L + tc::QT - 1) / tc::QT);
    const int n_dtiles = static_cast<int>((fp.d + tc::DT - 1) / tc::DT);
    const bool per_step = fp.decay_mode == EMA_DECAY_PER_STEP;
    pl->carry = nullptr; pl->flags = nullptr; pl->agg = nullptr; pl->split = 0;
    const bool have_carry_ws = fp.sync_ws && fp.sync_ws_bytes >= carry_bytes();
    if (allow_aggregates && tc_wants_aggregates(rows, fp.L, fp.d) &&
        fp.sync_ws && fp.sync_ws_bytes >= carry_bytes() + tile_aggregate_bytes(rows, fp.L, fp.d)) {
        // tiles are dealt evenly whatever the item count, so a per-step decay always shares one matrix between two
        // channel tiles
        pl->sub = (per_step && n_dtiles > 1) ? 2 : 1;
        pl->n_groups = (n_dtiles + pl->sub - 1) / pl->sub;
        pl->n_items = static_cast<int>(rows * pl->n_groups);
        const int64_t units = static_cast<int64_t>(pl->n_items) * n_tiles;
        const int want = sms - spare_sms();
        pl->grid = static_cast<int>(units < want ? units : want);
        pl->split = 2;
        pl->agg = reinterpret_cast<float *>(static_cast<uint8_t *>(fp.sync_ws) + carry_bytes());
        return EMA_OK;
    }
    // With a per-step decay every tile needs its own matrix and the builders set the pace: let one matrix serve two
    // channel tiles of the row, unless halving the number of work items would leave noticeably more SMs without one.
    {
        const int64_t single = rows * n_dtiles, paired = rows * ((n_dtiles + 1) / 2);
        const int64_t busy_single = single < sms ? single : sms, busy_paired = paired < sms ? paired : sms;
        pl->sub = (per_step && n_dtiles > 1 && busy_paired * 100 >= busy_single * 85) ? 2 : 1;
    }
    pl->n_groups = (n_dtiles + pl->sub - 1) / pl->sub;
    pl->n_items = static_cast<int>(rows * pl->n_groups);
    const int n_items = pl->n_items;
    const int rounds = (n_items + sms - 1) / sms;
    pl->grid = (n_items + rounds - 1) / rounds;
    // Cutting pays only when whole items would leave a large share of the SM-rounds idle.  At 256 items on 148 SMs
    // (13.5 % idle) it does not: 128 thread blocks with two items each already move 6.0 TB/s when the clocks are high,
    // and under the power cap the 18 extra thread blocks of the cut schedule cost in clock what they add in width
    // (0.530 ms against 0.537 ms per headline step, measured back to back on one GPU).
    const bool uneven = static_cast<int64_t>(rounds) * sms * 85 > static_cast<int64_t>(n_items) * 100;
    // (with fewer items than SMs a cut that hands carries on cannot help: an item's tiles are a sequential chain, and
    // the thread blocks that would share it only wait for one another - measured 30-40 % slower)
    if (!allow_carry_split || split_setting() == 0 || n_items < sms || sms > kMaxSplitGrid || !uneven || !have_carry_ws)
        return EMA_OK;
    const size_t fb = sync_flag_bytes();
    cudaError_t e = cudaMemsetAsync(fp.sync_ws, 0, fb, stream);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    pl->flags = static_cast<unsigned *>(fp.sync_ws);
    pl->carry = reinterpret_cast<float *>(static_cast<uint8_t *>(fp.sync_ws) + fb);
    pl->grid = sms - spare_sms();
    pl->split = 1;
    return EMA_OK;
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
    p.in_weight = fp.in_weight; p.out_weight = fp.out_weight;
    p.b = fp.b; p.L = fp.L; p.h = fp.h; p.d = fp.d;
    p.a_sb = fp.a_sb; p.a_sl = fp.a_sl; p.a_sh = fp.a_sh;
    p.decay_mode = fp.decay_mode; p.convention = fp.convention; p.chunk = fp.chunk;
    p.n_tiles = static_cast<int>((fp.L + tc::QT - 1) / tc::QT);
    p.n_dtiles = static_cast<int>((fp.d + tc::DT - 1) / tc::DT);
    p.n_chunks = fp.n_chunks;
    p.bounds = fp.bounds;
    // the sum of the log decays is accumulated per item by one CTA: no cutting when it is asked for; the weighted
    // scan has no aggregate pass
    Plan pl;
    const bool weighted = fp.in_weight || fp.out_weight;
    rc = make_plan(fp, fp.log_decay_sum == nullptr, fp.log_decay_sum == nullptr && !weighted, stream, &pl);
    if (rc) return rc;
    p.sub = pl.sub; p.n_groups = pl.n_groups; p.n_items = pl.n_items;
    p.split = pl.split; p.carry = pl.carry; p.flags = pl.flags;
    p.agg_vec = p.agg_fac = nullptr;
    if (pl.split == 2) {
        rc = launch_tile_aggregates(fp, 0, pl.agg, stream);
        if (rc) return rc;
        p.agg_vec = pl.agg;
        p.agg_fac = pl.agg + fp.b * fp.h * p.n_tiles * fp.d;
    }
    const int grid = pl.grid;
    g_last_schedule = pl.split;
    // weighted scan: the builders' larger register share pays when most SMs are busy and a matrix serves two channel
    // tiles (measured: 5-6 % faster at d = 256 and 1024 with 128 thread blocks, 5-10 % slower with 64 thread blocks or
    // one channel tile per item)
    const bool heavy = weighted && p.sub == 2 && grid >= 100;
    auto kernel = weighted ? (heavy ? tc::ema_fwd_tc_kernel<true, false, true> : tc::ema_fwd_tc_kernel<true, false, false>)
                           : (pl.split == 2 ? tc::ema_fwd_tc_kernel<false, true> : tc::ema_fwd_tc_kernel<false, false>);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::kFwdSmemBytes);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    e = launch_overlapped(kernel, dim3(grid), dim3(tc::kThreads), tc::kFwdSmemBytes, stream, tm_x, tm_y, p);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
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
    p.n_dtiles = static_cast<int>((fp.d + tc::DT - 1) / tc::DT);
    p.n_dt64 = static_cast<int>((fp.d + 63) / 64);
    p.head_partial_offset = kHeadPartialOffset(fp.b * fp.h);
    p.bounds = fp.bounds;
    Plan pl;
    rc = make_plan(fp, true, true, stream, &pl);
    if (rc) return rc;
    p.sub = pl.sub; p.n_groups = pl.n_groups; p.n_items = pl.n_items;
    p.split = pl.split; p.carry = pl.carry; p.flags = pl.flags;
    p.agg_vec = p.agg_fac = nullptr;
    if (pl.split == 2) {
        rc = launch_tile_aggregates(fp, 1, pl.agg, stream);
        if (rc) return rc;
        p.agg_vec = pl.agg;
        p.agg_fac = pl.agg + fp.b * fp.h * p.n_tiles * fp.d;
    }
    const int grid = pl.grid;
    g_last_schedule = pl.split;
    const bool ps = p.decay_mode == EMA_DECAY_PER_STEP;
    const bool cv = p.convention != 0;
    // one instantiation per schedule (aggregates, tile ranges, whole items) x kind of decay x convention
    const int variant = (pl.split == 2 ? 0 : pl.split == 1 ? 1 : 2) * 4 + (ps ? 2 : 0) + (cv ? 1 : 0);
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const tc::TcBwdParams);
    static const KernelFn kernels[12] = {
        tc::ema_bwd_tc_kernel<true, false, false, false>,  tc::ema_bwd_tc_kernel<true, false, true, false>,
        tc::ema_bwd_tc_kernel<true, true, false, false>,   tc::ema_bwd_tc_kernel<true, true, true, false>,
        tc::ema_bwd_tc_kernel<false, false, false, true>,  tc::ema_bwd_tc_kernel<false, false, true, true>,
        tc::ema_bwd_tc_kernel<false, true, false, true>,   tc::ema_bwd_tc_kernel<false, true, true, true>,
        tc::ema_bwd_tc_kernel<false, false, false, false>, tc::ema_bwd_tc_kernel<false, false, true, false>,
        tc::ema_bwd_tc_kernel<false, true, false, false>,  tc::ema_bwd_tc_kernel<false, true, true, false>};
    const KernelFn kernel = kernels[variant];
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::kBwdSmemBytes);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    e = launch_overlapped(kernel, dim3(grid), dim3(tc::kThreads), tc::kBwdSmemBytes, stream, tm_x, tm_g, tm_o, p);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    return check_launch();
}

static bool tma_f32_ok(const void *base, int64_t d, int64_t sb, int64_t sl, int64_t sh, int64_t b, int64_t L, int64_t h);

// fp32 forward, CUDA cores fed by TMA.  Takes what the widest-vector CUDA-core kernel takes (d and the strides multiples of
// 4 elements, 16-byte aligned base) when the whole sequence is scanned; EMA_ERR_UNSUPPORTED sends the caller to the
// plain kernel.
template <typename T, int STAGES>
static int launch_fwd_fma_tma(const CUtensorMap &tm_x, const FusedParams &fp, cudaStream_t stream) {
    const bool weighted = fp.in_weight || fp.out_weight;
    auto kernel = weighted ? tmafeed::ema_fwd_fma_tma_kernel<T, STAGES, true> : tmafeed::ema_fwd_fma_tma_kernel<T, STAGES, false>;
    constexpr int smem = tmafeed::TmaFeed<T, STAGES>::kSmemBytes;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    const int64_t blocks = fp.b * fp.h * fp.n_dtiles;   // n_dtiles counts 64-channel tiles here
    kernel<<<static_cast<unsigned>(blocks), kFmaThreads, smem, stream>>>(tm_x, fp);
    return check_launch();
}

// (The feed is generic in the element type, but only fp32 is built: for bf16 the same kernel measured 4.8 TB/s with a
// per-head and 3.9 TB/s with a per-step decay on the headline shape, against 5.3 and 5.1 TB/s for the tensor-core kernel.)
int launch_fused_fwd_fma_tma(const FusedParams &fp, cudaStream_t stream) {
    if (fp.stop_below > 0.f || encode_fn() == nullptr) return EMA_ERR_UNSUPPORTED;
    if (!tma_f32_ok(fp.x, fp.d, fp.x_sb, fp.x_sl, fp.x_sh, fp.b, fp.L, fp.h)) return EMA_ERR_UNSUPPORTED;
    CUtensorMap tm_x;
    int rc = make_tmap(&tm_x, fp.x, fp.b, fp.L, fp.h, fp.d, fp.x_sb, fp.x_sl, fp.x_sh, true);
    if (rc) return rc;
    return launch_fwd_fma_tma<float, 3>(tm_x, fp, stream);
}

static bool tma_f32_ok(const void *base, int64_t d, int64_t sb, int64_t sl, int64_t sh, int64_t b, int64_t L, int64_t h) {
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || d % 4 != 0) return false;
    return !((h > 1 && (sh % 4 != 0 || sh <= 0)) || (L > 1 && (sl % 4 != 0 || sl <= 0)) || (b > 1 && (sb % 4 != 0 || sb <= 0)));
}

// fp32 backward, CUDA cores fed by TMA: same conditions as the forward, for x and dy.
int launch_fused_bwd_fma_tma(const FusedParams &fp, cudaStream_t stream) {
    if (fp.stop_below > 0.f || encode_fn() == nullptr) return EMA_ERR_UNSUPPORTED;
    if (!tma_f32_ok(fp.x, fp.d, fp.x_sb, fp.x_sl, fp.x_sh, fp.b, fp.L, fp.h) ||
        !tma_f32_ok(fp.dy, fp.d, fp.g_sb, fp.g_sl, fp.g_sh, fp.b, fp.L, fp.h))
        return EMA_ERR_UNSUPPORTED;
    CUtensorMap tm_x, tm_g;
    int rc = make_tmap(&tm_x, fp.x, fp.b, fp.L, fp.h, fp.d, fp.x_sb, fp.x_sl, fp.x_sh, true);
    if (rc) return rc;
    rc = make_tmap(&tm_g, fp.dy, fp.b, fp.L, fp.h, fp.d, fp.g_sb, fp.g_sl, fp.g_sh, true);
    if (rc) return rc;
    cudaError_t e = cudaFuncSetAttribute(tmafeed::ema_bwd_fma_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         tmafeed::kBwdSmemBytes);
    if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
    const int64_t blocks = fp.b * fp.h * fp.n_dtiles;
    tmafeed::ema_bwd_fma_tma_kernel<<<static_cast<unsigned>(blocks), kFmaThreads, tmafeed::kBwdSmemBytes, stream>>>(
        tm_x, tm_g, fp);
    return check_launch();
}

// Launches the bounded-wait self-test (see tc::selftest_wait_kernel); `scratch` is one zeroed 32-bit word in device
// memory that nothing ever writes (mode 1 only).
int launch_selftest_wait(int mode, unsigned polls, const unsigned *scratch, cudaStream_t stream) {
    tc::selftest_wait_kernel<<<1, 32, 0, stream>>>(mode, polls, scratch);
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
