// C-ABI entry points of the fused path: argument checks, kernel selection, launches.
#include "ema_common.cuh"

#include <atomic>
#include <cstddef>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace ema {

static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = static_cast<int>(e); }
bool overlapped_launches() {
    static const bool on = [] {
        const char *e = std::getenv("EMA_B200_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

namespace {

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int check_problem(const ema_b200_problem *p) {
    if (!p) return EMA_ERR_BADARG;
    if (p->b < 0 || p->L < 0 || p->h < 0 || p->d < 0) return EMA_ERR_BADARG;
    if (p->dtype != EMA_F32 && p->dtype != EMA_BF16) return EMA_ERR_UNSUPPORTED;
    if (p->decay_mode != EMA_DECAY_PER_STEP && p->decay_mode != EMA_DECAY_PER_HEAD) return EMA_ERR_BADARG;
    if (p->convention != EMA_CONV_NORTH_STAR && p->convention != EMA_CONV_PRESCALED_LOG) return EMA_ERR_BADARG;
    if (p->chunk < 0) return EMA_ERR_BADARG;
    if (p->L >= (1ll << 31) - 4096) return EMA_ERR_UNSUPPORTED;
    if (p->b * p->h > (1ll << 24) || p->d > (1ll << 24)) return EMA_ERR_UNSUPPORTED;
    return EMA_OK;
}

// widest vector the FMA kernels may use on every big tensor of this call
int pick_vec(const ema_b200_problem *p, const void *x, const void *out, const void *dy) {
    const size_t es = p->dtype == EMA_F32 ? 4 : 2;
    bool ok = p->d % 4 == 0;
    auto strides_ok = [](int64_t a, int64_t b, int64_t c) { return a % 4 == 0 && b % 4 == 0 && c % 4 == 0; };
    ok = ok && strides_ok(p->x_sb, p->x_sl, p->x_sh) && strides_ok(p->y_sb, p->y_sl, p->y_sh);
    ok = ok && aligned(x, 4 * es) && aligned(out, 4 * es);
    if (dy) ok = ok && strides_ok(p->g_sb, p->g_sl, p->g_sh) && aligned(dy, 4 * es);
    return ok ? 4 : 1;
}

// Kernel family for bf16 problems: 0 = tensor cores where the layout allows (default), 1 = CUDA cores
// only.  Set by ema_b200_set_path or, once, by the environment variable EMA_B200_PATH=fma.
std::atomic<int> g_path{-1};
thread_local int g_last_path = -1;  // kernel family of the last fused launch on this thread: 1 tensor cores, 0 CUDA cores
bool tc_enabled() {
    int v = g_path.load(std::memory_order_relaxed);
    if (v < 0) {
        const char *e = std::getenv("EMA_B200_PATH");
        v = (e && std::strcmp(e, "fma") == 0) ? 1 : 0;
        g_path.store(v, std::memory_order_relaxed);
    }
    return v == 0;
}

// ---- bounds-checking build: the address ranges of a call's buffers ---------------------------------------------
// bytes spanned by a [b, L, h, d] tensor with element strides sb, sl, sh (d contiguous), es bytes per element
size_t span4(const ema_b200_problem *p, int64_t sb, int64_t sl, int64_t sh, size_t es) {
    if (p->b <= 0 || p->L <= 0 || p->h <= 0 || p->d <= 0) return 0;
    return static_cast<size_t>((p->b - 1) * sb + (p->L - 1) * sl + (p->h - 1) * sh + p->d) * es;
}
// bytes spanned by the decay (and everything shaped like it: its gradient, the per-step weights and theirs)
size_t span_decay(const ema_b200_problem *p) {
    if (p->b <= 0 || p->L <= 0 || p->h <= 0) return 0;
    if (p->decay_mode == EMA_DECAY_PER_STEP)
        return static_cast<size_t>((p->b - 1) * p->a_sb + (p->L - 1) * p->a_sl + (p->h - 1) * p->a_sh + 1) * 4;
    return static_cast<size_t>((p->h - 1) * p->a_sh + 1) * 4;
}
#ifdef EMA_BOUNDS_CHECK
thread_local size_t g_shrink_next = 0;
BoundsTable *device_table() {   // one table per device, made on first use
    static std::mutex mu;
    static BoundsTable *tabs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!tabs[dev]) {
        BoundsTable *t = nullptr;
        if (cudaMalloc(&t, sizeof(BoundsTable)) != cudaSuccess) return nullptr;
        if (cudaMemset(t, 0, sizeof(BoundsTable)) != cudaSuccess) return nullptr;
        tabs[dev] = t;
    }
    return tabs[dev];
}
#endif

void fill_params(FusedParams &fp, const ema_b200_problem *p, int vec) {
    std::memset(&fp, 0, sizeof(fp));
    fp.b = p->b; fp.L = p->L; fp.h = p->h; fp.d = p->d;
    fp.x_sb = p->x_sb; fp.x_sl = p->x_sl; fp.x_sh = p->x_sh;
    fp.o_sb = p->y_sb; fp.o_sl = p->y_sl; fp.o_sh = p->y_sh;
    fp.g_sb = p->g_sb; fp.g_sl = p->g_sl; fp.g_sh = p->g_sh;
    fp.a_sb = p->a_sb; fp.a_sl = p->a_sl; fp.a_sh = p->a_sh;
    fp.decay_mode = p->decay_mode;
    fp.convention = p->convention;
    fp.chunk = p->chunk;
    fp.n_tiles = static_cast<int>((p->L + kFmaTile - 1) / kFmaTile);
    const int dt = kFmaCT * vec;
    fp.n_dtiles = static_cast<int>((p->d + dt - 1) / dt);
    fp.n_chunks = p->chunk > 0 ? (p->L + p->chunk - 1) / p->chunk : 0;
}

}  // namespace

// ranges[0] is the call's output tensor (the one ema_b200_bounds_shrink_next shortens)
BoundsTable *bounds_prepare(const BoundsRange *ranges, int n, cudaStream_t stream) {
#ifdef EMA_BOUNDS_CHECK
    BoundsTable *tb = device_table();
    if (!tb) return nullptr;
    BoundsTable h;
    std::memset(&h, 0, sizeof(h));
    for (int i = 0; i < n && h.n < kBoundsMaxRanges; ++i) {
        if (!ranges[i].ptr || ranges[i].bytes == 0) continue;
        size_t bytes = ranges[i].bytes;
        if (i == 0 && g_shrink_next) bytes = bytes > g_shrink_next ? bytes - g_shrink_next : 0;
        h.lo[h.n] = reinterpret_cast<unsigned long long>(ranges[i].ptr);
        h.hi[h.n] = h.lo[h.n] + bytes;
        ++h.n;
    }
    g_shrink_next = 0;
    // everything between the status word and the sink (pageable source: staged before the call returns)
    const size_t off = offsetof(BoundsTable, n), len = offsetof(BoundsTable, sink) - off;
    if (cudaMemcpyAsync(reinterpret_cast<char *>(tb) + off, reinterpret_cast<const char *>(&h) + off, len,
                        cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return nullptr;
    return tb;
#else
    (void)ranges; (void)n; (void)stream;
    return nullptr;
#endif
}

int bounds_read_status(int clear) {
#ifdef EMA_BOUNDS_CHECK
    BoundsTable *tb = device_table();
    if (!tb) return 0;
    unsigned v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return 0;
    if (cudaMemcpy(&v, &tb->status, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return 0;
    if (v && clear) cudaMemset(&tb->status, 0, sizeof(v));
    return static_cast<int>(v);
#else
    (void)clear;
    return 0;
#endif
}
}  // namespace ema

using namespace ema;

extern "C" int ema_b200_version(void) { return EMA_B200_VERSION; }

extern "C" int ema_b200_bounds_checked(void) {
#ifdef EMA_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}
extern "C" int ema_b200_bounds_status(int clear) { return bounds_read_status(clear); }
extern "C" int ema_b200_bounds_shrink_next(size_t bytes) {
#ifdef EMA_BOUNDS_CHECK
    g_shrink_next = bytes;
    return EMA_OK;
#else
    (void)bytes;
    return EMA_ERR_UNSUPPORTED;
#endif
}

extern "C" int ema_b200_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" const char *ema_b200_error_string(int code) {
    switch (code) {
        case EMA_OK: return "ok";
        case EMA_ERR_BADARG: return "bad argument (null pointer, negative size or inconsistent shape)";
        case EMA_ERR_ALIGN: return "pointer or stride not aligned for the element type";
        case EMA_ERR_UNSUPPORTED: return "request not supported by this library";
        case EMA_ERR_CUDA: return "a CUDA call failed (see ema_b200_last_cuda_error)";
        case EMA_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case EMA_ERR_WORKSPACE: return "workspace missing or too small";
        case EMA_ERR_SCRATCH_LIMIT:
            return "problem needs more scratch than the library's built-in array holds (8 MiB): "
                   "use ema_b200_bwd with a caller-owned workspace";
        default: return "unknown error code";
    }
}

extern "C" int ema_b200_device_status(int clear) { return read_tc_status(clear); }
extern "C" int ema_b200_set_split(int on) { return tc_set_split(on); }

extern "C" int ema_b200_selftest_wait(int mode, int polls, const void *zero_word, void *stream) {
    if ((mode != 0 && mode != 1) || polls <= 0 || polls > (1 << 20)) return EMA_ERR_BADARG;
    if (mode == 1 && (!zero_word || !aligned(zero_word, 4))) return EMA_ERR_BADARG;
    return launch_selftest_wait(mode, static_cast<unsigned>(polls), static_cast<const unsigned *>(zero_word),
                                static_cast<cudaStream_t>(stream));
}

extern "C" int ema_b200_last_path(void) { return g_last_path; }
extern "C" int ema_b200_last_schedule(void) { return g_last_path == 1 ? tc_last_schedule() : -1; }

extern "C" int ema_b200_set_path(int path) {
    if (path != 0 && path != 1) return EMA_ERR_BADARG;
    g_path.store(path, std::memory_order_relaxed);
    return EMA_OK;
}

extern "C" int ema_b200_tile_steps(const ema_b200_problem *p) {
    if (check_problem(p) != EMA_OK) return 0;
    return kFmaTile;
}

extern "C" size_t ema_b200_tile_states_bytes(const ema_b200_problem *p) {
    if (check_problem(p) != EMA_OK) return 0;
    const int64_t n_tiles = (p->L + kFmaTile - 1) / kFmaTile;
    return static_cast<size_t>(p->b * p->h * n_tiles * p->d) * sizeof(float);
}

// floats of decay-gradient partial sums (the first part of the backward's workspace), rounded to 256 bytes
static size_t bwd_partial_bytes(const ema_b200_problem *p) {
    // sized for the narrowest channel tile (vec = 1) so that it never depends on pointer alignment
    const int64_t n_tiles = (p->L + kFmaTile - 1) / kFmaTile;
    const int64_t n_dtiles = (p->d + kFmaCT - 1) / kFmaCT;
    const int64_t rows = p->b * p->h;
    const int64_t per_step = rows * n_dtiles * n_tiles * kFmaTile;
    const int64_t per_head = kHeadPartialOffset(rows) + rows * n_dtiles * n_tiles * (kFmaThreads / 32);
    const int64_t n = p->decay_mode == EMA_DECAY_PER_STEP ? per_step : per_head;
    return (static_cast<size_t>(n > 0 ? n : 1) * sizeof(float) + 255) / 256 * 256;
}

static size_t sync_bytes(const ema_b200_problem *p) {
    return p->dtype == EMA_BF16 ? tc_sync_bytes(p->b * p->h, p->L, p->d) : 0;
}

extern "C" size_t ema_b200_bwd_workspace_bytes(const ema_b200_problem *p) {
    if (check_problem(p) != EMA_OK) return 0;
    return bwd_partial_bytes(p) + sync_bytes(p);
}

extern "C" size_t ema_b200_fwd_workspace_bytes(const ema_b200_problem *p) {
    if (check_problem(p) != EMA_OK) return 0;
    return sync_bytes(p);
}

static int fwd_impl(const ema_b200_problem *p, const void *x, const float *decay, const float *in_weight,
                    const float *out_weight, void *y, float *chunk_states, float *tile_states,
                    const float *init_state, float *final_state, float *log_decay_sum, float stop_below,
                    void *workspace, size_t workspace_bytes, void *stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    if ((in_weight || out_weight) && p->decay_mode != EMA_DECAY_PER_STEP) return EMA_ERR_UNSUPPORTED;
    if (!aligned(in_weight, 4) || !aligned(out_weight, 4)) return EMA_ERR_ALIGN;
    if (chunk_states && p->chunk <= 0) return EMA_ERR_BADARG;
    if (!(stop_below >= 0.f)) return EMA_ERR_BADARG;
    const size_t es = p->dtype == EMA_F32 ? 4 : 2;
    if (!aligned(x, es) || !aligned(y, es) || !aligned(decay, 4)) return EMA_ERR_ALIGN;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t rows = p->b * p->h;
    if (rows == 0 || p->d == 0) return EMA_OK;  // empty tensors carry null pointers: nothing to do
    if (p->L > 0) {
        if (!x || !decay) return EMA_ERR_BADARG;
        if (!y && !chunk_states && !tile_states && !final_state) return EMA_ERR_BADARG;
    }
    if (p->L == 0) {
        // nothing to scan: the state passes through
        cudaError_t e = cudaSuccess;
        if (final_state) {
            e = init_state ? cudaMemcpyAsync(final_state, init_state, rows * p->d * 4, cudaMemcpyDeviceToDevice, st)
                           : cudaMemsetAsync(final_state, 0, rows * p->d * 4, st);
        }
        if (e == cudaSuccess && log_decay_sum) e = cudaMemsetAsync(log_decay_sum, 0, rows * 4, st);
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
        return EMA_OK;
    }
    const int vec = pick_vec(p, x, y ? y : x, nullptr);
    FusedParams fp;
    fill_params(fp, p, vec);
    fp.x = x; fp.decay = decay; fp.out = y;
    fp.in_weight = in_weight; fp.out_weight = out_weight;
    fp.chunk_states = chunk_states; fp.tile_states = tile_states;
    fp.init_state = init_state; fp.final_state = final_state;
    fp.log_decay_sum = log_decay_sum;
    fp.stop_below = stop_below;
    // optional scratch: without it (or with too little) the kernels simply never cut a work item across CTAs
    const bool ws_ok = workspace && aligned(workspace, 16) && workspace_bytes >= sync_bytes(p);
    fp.sync_ws = ws_ok ? workspace : nullptr;
    fp.sync_ws_bytes = ws_ok ? workspace_bytes : 0;
    if (rows * fp.n_dtiles >= (1ll << 31)) return EMA_ERR_UNSUPPORTED;
    if (ema_b200_bounds_checked()) {
        const size_t state = static_cast<size_t>(rows * p->d) * 4;
        const BoundsRange ranges[] = {
            {y, span4(p, p->y_sb, p->y_sl, p->y_sh, es)},
            {x, span4(p, p->x_sb, p->x_sl, p->x_sh, es)},
            {decay, span_decay(p)}, {in_weight, span_decay(p)}, {out_weight, span_decay(p)},
            {chunk_states, state * static_cast<size_t>(fp.n_chunks)}, {tile_states, ema_b200_tile_states_bytes(p)},
            {init_state, state}, {final_state, state}, {log_decay_sum, static_cast<size_t>(rows) * 4},
            {fp.sync_ws, fp.sync_ws_bytes}};
        fp.bounds = bounds_prepare(ranges, static_cast<int>(sizeof(ranges) / sizeof(ranges[0])), st);
        if (!fp.bounds) return EMA_ERR_CUDA;
    }
    if (p->dtype == EMA_BF16 && y && stop_below == 0.f && tc_enabled() &&
        tc_tensor_ok(x, p->d, p->x_sb, p->x_sl, p->x_sh, p->b, p->L, p->h) &&
        tc_tensor_ok(y, p->d, p->y_sb, p->y_sl, p->y_sh, p->b, p->L, p->h) && aligned(tile_states, 16)) {
        rc = launch_fused_fwd_tc(fp, st);
        if (rc == EMA_OK) g_last_path = 1;
        if (rc != EMA_ERR_UNSUPPORTED) return rc;  // a tensor map the driver refuses falls through to the FMA path
    }
    if (p->dtype == EMA_F32 && vec == 4 && tc_enabled()) {
        rc = launch_fused_fwd_fma_tma(fp, st);
        if (rc == EMA_OK) g_last_path = 2;
        if (rc != EMA_ERR_UNSUPPORTED) return rc;
    }
    g_last_path = 0;
    return launch_fused_fwd_fma(fp, p->dtype, vec, st);
}

extern "C" int ema_b200_fwd(const ema_b200_problem *p, const void *x, const float *decay, void *y,
                            float *chunk_states, float *tile_states, const float *init_state,
                            float *final_state, float *log_decay_sum, float stop_below, void *workspace,
                            size_t workspace_bytes, void *stream) {
    return fwd_impl(p, x, decay, nullptr, nullptr, y, chunk_states, tile_states, init_state, final_state,
                    log_decay_sum, stop_below, workspace, workspace_bytes, stream);
}

extern "C" int ema_b200_fwd_weighted(const ema_b200_problem *p, const void *x, const float *decay,
                                     const float *in_weight, const float *out_weight, void *y,
                                     float *chunk_states, float *tile_states, const float *init_state,
                                     float *final_state, float *log_decay_sum, float stop_below,
                                     void *workspace, size_t workspace_bytes, void *stream) {
    return fwd_impl(p, x, decay, in_weight, out_weight, y, chunk_states, tile_states, init_state, final_state,
                    log_decay_sum, stop_below, workspace, workspace_bytes, stream);
}

extern "C" int ema_b200_bwd(const ema_b200_problem *p, const void *x, const float *decay, const void *dy,
                            const float *tile_states, void *dx, float *ddecay, const float *dfinal_state,
                            float *dinit_state, float stop_below, void *workspace, size_t workspace_bytes,
                            void *stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    const bool empty = p->b * p->h == 0 || p->L == 0 || p->d == 0;
    if (!empty && (!x || !decay || !dy || !dx || !ddecay || !tile_states)) return EMA_ERR_BADARG;
    if (!(stop_below >= 0.f)) return EMA_ERR_BADARG;
    const size_t es = p->dtype == EMA_F32 ? 4 : 2;
    if (!aligned(x, es) || !aligned(dy, es) || !aligned(dx, es) || !aligned(decay, 4) || !aligned(ddecay, 4))
        return EMA_ERR_ALIGN;
    if (!workspace || workspace_bytes < ema_b200_bwd_workspace_bytes(p)) return EMA_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return EMA_ERR_ALIGN;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t rows = p->b * p->h;
    if (rows == 0) return EMA_OK;
    if (p->L == 0 || p->d == 0) {
        cudaError_t e = cudaSuccess;
        if (p->decay_mode == EMA_DECAY_PER_HEAD && ddecay) {
            // ddecay[h] may be strided: clear element by element through a 2-D memset
            e = cudaMemset2DAsync(ddecay, static_cast<size_t>(p->a_sh > 0 ? p->a_sh : 1) * 4, 0, 4,
                                  static_cast<size_t>(p->h), st);
        } else if (p->decay_mode == EMA_DECAY_PER_STEP && ddecay && p->L > 0) {
            // no channels: the gradient of every step's decay is an empty sum (the reduction kernel writes zeros)
            FusedParams fz;
            fill_params(fz, p, 1);
            fz.n_dtiles = 0;
            fz.da_partial = static_cast<float *>(workspace);
            const int rz = launch_da_reduce(fz, ddecay, kFmaTile, st);
            if (rz) return rz;
        }
        if (e == cudaSuccess && dinit_state && p->d > 0) {
            e = dfinal_state ? cudaMemcpyAsync(dinit_state, dfinal_state, rows * p->d * 4, cudaMemcpyDeviceToDevice, st)
                             : cudaMemsetAsync(dinit_state, 0, rows * p->d * 4, st);
        }
        if (e != cudaSuccess) { set_last_cuda_error(e); return EMA_ERR_CUDA; }
        return EMA_OK;
    }
    const int vec = pick_vec(p, x, dx, dy);
    FusedParams fp;
    fill_params(fp, p, vec);
    fp.x = x; fp.decay = decay; fp.dy = dy; fp.out = dx;
    fp.tile_states = const_cast<float *>(tile_states);
    fp.dfinal_state = dfinal_state; fp.dinit_state = dinit_state;
    fp.da_partial = static_cast<float *>(workspace);
    fp.stop_below = stop_below;
    fp.sync_ws = static_cast<uint8_t *>(workspace) + bwd_partial_bytes(p);
    fp.sync_ws_bytes = sync_bytes(p);
    if (rows * fp.n_dtiles >= (1ll << 31)) return EMA_ERR_UNSUPPORTED;
    if (ema_b200_bounds_checked()) {
        const size_t state = static_cast<size_t>(rows * p->d) * 4;
        const BoundsRange ranges[] = {
            {dx, span4(p, p->y_sb, p->y_sl, p->y_sh, es)},
            {x, span4(p, p->x_sb, p->x_sl, p->x_sh, es)}, {dy, span4(p, p->g_sb, p->g_sl, p->g_sh, es)},
            {decay, span_decay(p)}, {ddecay, span_decay(p)},
            {tile_states, ema_b200_tile_states_bytes(p)}, {dfinal_state, state}, {dinit_state, state},
            {workspace, ema_b200_bwd_workspace_bytes(p)}};
        fp.bounds = bounds_prepare(ranges, static_cast<int>(sizeof(ranges) / sizeof(ranges[0])), st);
        if (!fp.bounds) return EMA_ERR_CUDA;
    }
    bool done = false;
    if (p->dtype == EMA_BF16 && stop_below == 0.f && tc_enabled() && vec == 4 &&
        tc_tensor_ok(x, p->d, p->x_sb, p->x_sl, p->x_sh, p->b, p->L, p->h) &&
        tc_tensor_ok(dy, p->d, p->g_sb, p->g_sl, p->g_sh, p->b, p->L, p->h) &&
        tc_tensor_ok(dx, p->d, p->y_sb, p->y_sl, p->y_sh, p->b, p->L, p->h)) {
        // same partial-sum layout as the CUDA-core kernel at vec = 4 (64-channel tiles, 64-step slots)
        rc = launch_fused_bwd_tc(fp, st);
        if (rc && rc != EMA_ERR_UNSUPPORTED) return rc;
        done = rc == EMA_OK;
    }
    g_last_path = done ? 1 : 0;
    if (!done && p->dtype == EMA_F32 && vec == 4 && tc_enabled()) {
        rc = launch_fused_bwd_fma_tma(fp, st);
        if (rc && rc != EMA_ERR_UNSUPPORTED) return rc;
        done = rc == EMA_OK;
        if (done) g_last_path = 2;
    }
    if (!done) {
        rc = launch_fused_bwd_fma(fp, p->dtype, vec, st);
        if (rc) return rc;
    }
    return launch_da_reduce(fp, ddecay, kFmaTile, st);
}


// ---- weighted backward ----------------------------------------------------------------------------------------
extern "C" size_t ema_b200_bwd_weighted_workspace_bytes(const ema_b200_problem *p) {
    if (check_problem(p) != EMA_OK || p->decay_mode != EMA_DECAY_PER_STEP) return 0;
    return 3 * bwd_partial_bytes(p);
}

extern "C" int ema_b200_bwd_weighted(const ema_b200_problem *p, const void *x, const float *decay,
                                     const float *in_weight, const float *out_weight, const void *dy,
                                     const float *tile_states, void *dx, float *ddecay, float *din_weight,
                                     float *dout_weight, const float *dfinal_state, float *dinit_state,
                                     void *workspace, size_t workspace_bytes, void *stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    if (p->decay_mode != EMA_DECAY_PER_STEP) return EMA_ERR_UNSUPPORTED;
    const bool empty = p->b * p->h == 0 || p->L == 0 || p->d == 0;
    if (!empty && (!x || !decay || !dy || !dx || !ddecay || !tile_states)) return EMA_ERR_BADARG;
    if ((in_weight && !din_weight) || (out_weight && !dout_weight)) return EMA_ERR_BADARG;
    const size_t es = p->dtype == EMA_F32 ? 4 : 2;
    if (!aligned(x, es) || !aligned(dy, es) || !aligned(dx, es) || !aligned(decay, 4) || !aligned(ddecay, 4) ||
        !aligned(in_weight, 4) || !aligned(out_weight, 4) || !aligned(din_weight, 4) || !aligned(dout_weight, 4))
        return EMA_ERR_ALIGN;
    if (!workspace || workspace_bytes < ema_b200_bwd_weighted_workspace_bytes(p)) return EMA_ERR_WORKSPACE;
    if (!aligned(workspace, 16)) return EMA_ERR_ALIGN;
    auto st = static_cast<cudaStream_t>(stream);
    const int64_t rows = p->b * p->h;
    if (rows == 0 || p->L == 0) return EMA_OK;
    const int vec = p->d > 0 ? pick_vec(p, x, dx, dy) : 1;
    FusedParams fp;
    fill_params(fp, p, vec);
    fp.x = x; fp.decay = decay; fp.dy = dy; fp.out = dx;
    fp.in_weight = in_weight; fp.out_weight = out_weight;
    fp.tile_states = const_cast<float *>(tile_states);
    fp.dfinal_state = dfinal_state; fp.dinit_state = dinit_state;
    fp.da_partial = static_cast<float *>(workspace);
    fp.weighted_partial_stride = static_cast<int64_t>(bwd_partial_bytes(p) / sizeof(float));
    if (rows * fp.n_dtiles >= (1ll << 31)) return EMA_ERR_UNSUPPORTED;
    if (ema_b200_bounds_checked()) {
        const size_t state = static_cast<size_t>(rows * p->d) * 4;
        const BoundsRange ranges[] = {
            {dx, span4(p, p->y_sb, p->y_sl, p->y_sh, es)},
            {x, span4(p, p->x_sb, p->x_sl, p->x_sh, es)}, {dy, span4(p, p->g_sb, p->g_sl, p->g_sh, es)},
            {decay, span_decay(p)}, {ddecay, span_decay(p)}, {in_weight, span_decay(p)}, {out_weight, span_decay(p)},
            {din_weight, span_decay(p)}, {dout_weight, span_decay(p)},
            {tile_states, ema_b200_tile_states_bytes(p)}, {dfinal_state, state}, {dinit_state, state},
            {workspace, ema_b200_bwd_weighted_workspace_bytes(p)}};
        fp.bounds = bounds_prepare(ranges, static_cast<int>(sizeof(ranges) / sizeof(ranges[0])), st);
        if (!fp.bounds) return EMA_ERR_CUDA;
    }
    if (p->d == 0) {
        fp.n_dtiles = 0;   // no channels: every gradient of a per-step quantity is an empty sum
    } else {
        g_last_path = 0;
        rc = launch_fused_bwd_fma_weighted(fp, p->dtype, vec, st);
        if (rc) return rc;
    }
    // three fixed-order reductions over the channel tiles: decay, input weight, output weight
    rc = launch_da_reduce(fp, ddecay, kFmaTile, st);
    if (rc) return rc;
    FusedParams fq = fp;
    if (din_weight) {
        fq.da_partial = fp.da_partial + fp.weighted_partial_stride;
        rc = launch_da_reduce(fq, din_weight, kFmaTile, st);
        if (rc) return rc;
    }
    if (dout_weight) {
        fq.da_partial = fp.da_partial + 2 * fp.weighted_partial_stride;
        rc = launch_da_reduce(fq, dout_weight, kFmaTile, st);
    }
    return rc;
}
