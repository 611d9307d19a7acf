// Sequence-parallel support: folding the carries the ranks exchanged into the state (or adjoint) that enters
// this rank's segment.  The reference has no multi-GPU path; the algebra is its chunk-level carry
// (kernels/ema_kernels/ema_state_pass.py:100-120: h <- exp(cs_last) h + S) applied to whole segments.
//
// Every rank contributes one record: the state its segment ends in when scanned from zero (F[rows, d]) followed by
// the sum of its log decays (logP[rows]), kept in the log domain because the product of 65536 decays underflows.
// After the all-gather a rank holds `world` such records, in rank order, in its own memory.
#include "ema_common.cuh"

namespace ema {
namespace {

// records[j] = [F_j (rows * d floats) | logP_j (rows floats)], j = 0 .. world - 1.
// forward : out = fold over j = 0 .. rank - 1, left to right:      c <- exp(logP_j) c + F_j
// reverse : out = fold over j = world - 1 .. rank + 1, right to left (F_j is then the adjoint leaving segment j)
struct BoundsRef {   // what EMA_AT needs from a parameter block
    BoundsTable *bounds;
};
__global__ void fold_records_kernel(const float *__restrict__ records, int world, int rank, int64_t rows,
                                    int64_t d, int reverse, float *__restrict__ out, BoundsRef br) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= rows * d) return;
    const int64_t row = i / d;
    const int64_t rec = rows * d + rows;
    float c = 0.f;
    if (!reverse) {
        for (int j = 0; j < rank; ++j) {
            const float *r = records + j * rec;
            c = fmaf(expf(*EMA_AT(br, r + rows * d + row, 240)), c, *EMA_AT(br, r + i, 241));
        }
    } else {
        for (int j = world - 1; j > rank; --j) {
            const float *r = records + j * rec;
            c = fmaf(expf(*EMA_AT(br, r + rows * d + row, 242)), c, *EMA_AT(br, r + i, 243));
        }
    }
    *EMA_AT(br, out + i, 244) = c;
}

}  // namespace
}  // namespace ema

extern "C" int ema_b200_fold_records(const float *records, int world, int rank, int64_t rows, int64_t d,
                                     int reverse, float *out, void *stream) {
    using namespace ema;
    if (world <= 0 || rank < 0 || rank >= world || rows < 0 || d < 0) return EMA_ERR_BADARG;
    const int64_t n = rows * d;
    if (n == 0) return EMA_OK;
    if (!records || !out) return EMA_ERR_BADARG;
    if (n >= (1ll << 31) * 256) return EMA_ERR_UNSUPPORTED;
    BoundsRef br{nullptr};
    if (ema_b200_bounds_checked()) {
        const BoundsRange ranges[] = {{out, static_cast<size_t>(n) * 4},
                                      {records, static_cast<size_t>(world) * static_cast<size_t>(n + rows) * 4}};
        br.bounds = bounds_prepare(ranges, 2, static_cast<cudaStream_t>(stream));
        if (!br.bounds) return EMA_ERR_CUDA;
    }
    fold_records_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        records, world, rank, rows, d, reverse, out, br);
    return check_launch();
}
