/*
 * ema_b200.h - C ABI of libema_b200.so: the EMA chunked scan (forward and backward) as
 * hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * The library replaces the GPU side of the reference project's EMA path.  The reference has no
 * FFI of its own: its boundary is a set of Python functions that launch Triton kernels.  Every
 * entry point below names the reference function (file:line inside the reference project) whose
 * device work it performs; the Python drop-ins with the reference's names and signatures call
 * these through ctypes.
 *
 * Conventions for every call
 *   - returns EMA_OK (0) or a negative EMA_ERR_* code; never throws, aborts or traps;
 *   - every pointer is a DEVICE pointer owned by the caller; the library allocates nothing;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*) and the call returns
 *     without synchronising; a bad argument is reported before anything is launched;
 *   - x, y, dy, dx have element type `dtype` (EMA_F32 or EMA_BF16); decay, states, gradients
 *     of the decay and all workspaces are fp32; accumulation is always fp32.
 */
#ifndef EMA_B200_H
#define EMA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EMA_B200_VERSION 100

enum {
    EMA_OK = 0,
    EMA_ERR_BADARG = -1,      /* null pointer, negative size, inconsistent shape             */
    EMA_ERR_ALIGN = -2,       /* pointer or stride not aligned as the dtype requires          */
    EMA_ERR_UNSUPPORTED = -3, /* valid request the library has no kernel for                  */
    EMA_ERR_CUDA = -4,        /* a CUDA call failed; see ema_b200_last_cuda_error()           */
    EMA_ERR_TIMEOUT = -5,     /* a bounded device-side wait ran out                           */
    EMA_ERR_WORKSPACE = -6,   /* workspace pointer null or smaller than _workspace_bytes says */
    EMA_ERR_SCRATCH_LIMIT = -7 /* problem needs more than ema_b200_static_scratch_limit() bytes */
};

enum { EMA_F32 = 0, EMA_BF16 = 1 };

/* decay_mode */
enum {
    EMA_DECAY_PER_STEP = 0, /* decay[b, L, h] with element strides a_sb, a_sl, a_sh            */
    EMA_DECAY_PER_HEAD = 1  /* decay[h] with element stride a_sh (time-invariant)              */
};

/* convention */
enum {
    /* decay holds a in (0,1) and x is the raw input:  y_t = a_t y_{t-1} + (1 - a_t) x_t;
     * the backward returns d/dx and d/da.                                                     */
    EMA_CONV_NORTH_STAR = 0,
    /* decay holds A = log a <= 0 and x is the pre-scaled input u = (1-a) x, the pair
     * (A_ema, X_ema) of the reference's chunked kernels:  y_t = exp(A_t) y_{t-1} + u_t;
     * the backward returns d/du and d/dA.                                                     */
    EMA_CONV_PRESCALED_LOG = 1
};

/* One EMA problem on the strided 4-D view x[b, L, h, d] (d contiguous; rows of the scan are the
 * (b, h) pairs).  The reference's folded layout X[B, L, T] is the case h = 1, b = B, d = T.
 * All strides are in ELEMENTS of the tensor they describe. */
typedef struct ema_b200_problem {
    int64_t b, L, h, d;
    int64_t x_sb, x_sl, x_sh; /* input x                                      */
    int64_t y_sb, y_sl, y_sh; /* output: y in the forward, dx in the backward  */
    int64_t g_sb, g_sl, g_sh; /* upstream gradient dy (backward only)          */
    int64_t a_sb, a_sl, a_sh; /* decay, and its gradient in the backward       */
    int32_t dtype;            /* EMA_F32 | EMA_BF16                            */
    int32_t decay_mode;       /* EMA_DECAY_PER_STEP | EMA_DECAY_PER_HEAD       */
    int32_t convention;       /* EMA_CONV_NORTH_STAR | EMA_CONV_PRESCALED_LOG  */
    int32_t chunk;            /* API-level chunk size Q for chunk_states; 0 = none */
} ema_b200_problem;

/* ---- library info ------------------------------------------------------------------------ */

int ema_b200_version(void);
/* cudaError_t of the most recent failing CUDA call made by this library on this thread. */
int ema_b200_last_cuda_error(void);
const char *ema_b200_error_string(int code);

/* Status word the tensor-core kernels write when a bounded device-side wait runs out: EMA_OK or
 * EMA_ERR_TIMEOUT.  Synchronises the device; clear != 0 resets the word.  Kernels never trap or spin
 * forever: after a timeout they finish their loops without waiting and the call's results are void. */
int ema_b200_device_status(int clear);

/* Self-test of the bounded device-side waits (test support; no counterpart in the reference, whose kernels never
 * wait on one another).  Launches one small thread block that waits - through the same wait functions the
 * tensor-core kernels use, but with a limit of `polls` polls (1 .. 2^20; a thousand polls last a few milliseconds) -
 * for something that never happens: mode 0, an mbarrier nobody arrives on; mode 1, an arrival counter nobody
 * increments (`zero_word`: one 32-bit device word holding 0 that nothing writes).  The wait runs out, the kernel
 * records it in the status word and returns; no copy or tensor memory is in flight, nothing traps or hangs.
 * Afterwards ema_b200_device_status(1) returns EMA_ERR_TIMEOUT once and EMA_OK from then on, and the library keeps
 * working. */
int ema_b200_selftest_wait(int mode, int polls, const void *zero_word, void *stream);

/* Bounds-checking build (test support; no counterpart in the reference).  A library built with -DEMA_BOUNDS_CHECK
 * (build.py --checked -> libema_b200_checked.so) routes every plain global-memory access of its kernels - the fused
 * calls ema_b200_fwd, _fwd_weighted, _bwd, _bwd_weighted, _fold_records and the ten stage calls - through a check against
 * the address ranges of the call's own buffers, which the entry point derives from the shapes, strides and byte counts
 * it was given.  An access outside all of them is recorded (the first one only) and redirected to a sink inside the
 * library's table: nothing outside the buffers is read or written and nothing traps.  TMA copies are clipped by their
 * tensor maps and need no check.  The table is per device and rewritten from host memory before every launch: use one
 * stream at a time with this build, and do not capture its calls in a CUDA graph.
 *   ema_b200_bounds_checked()      1 in that build, 0 in the normal one (where the two calls below do nothing).
 *   ema_b200_bounds_status(clear)  0, or 0x400 | site of the first rejected access since the word was last cleared;
 *                                  synchronises the device.
 *   ema_b200_bounds_shrink_next(n) test hook: the next checked call of this thread registers its output tensor (y or dx)
 *                                  as n bytes shorter than it is, so that the kernel's last stores are rejected although
 *                                  the memory is really there - a self-test of the checker that touches nothing foreign.
 *                                  Returns EMA_ERR_UNSUPPORTED in the normal build. */
int ema_b200_bounds_checked(void);
int ema_b200_bounds_status(int clear);
int ema_b200_bounds_shrink_next(size_t bytes);

/* Which kernels bf16 problems run on: 0 = tensor-core path wherever the layout allows it (default),
 * 1 = plain CUDA-core kernels only (also for fp32, which otherwise uses the TMA-fed variants of the same
 * kernels).  fp32 problems always compute on the CUDA cores (exactness).  Meant for A/B
 * measurements and tests; the environment variable EMA_B200_PATH=fma sets the same switch at load. */
int ema_b200_set_path(int path);
/* How the bf16 kernels spread a problem over the SMs (the environment variable EMA_B200_SPLIT sets the same at load):
 *   0  every work item (scan row x 128 channels) stays on one thread block;
 *   1  (default) items may be cut across thread blocks: when the items do not divide evenly among the SMs, a thread
 *      block hands the carry of a cut item to the next one through the scratch; when there are fewer items than about
 *      two thirds of the SMs (and at least four 128-step tiles), a first pass reduces every tile to its aggregate -
 *      the reference's chunk-state stage, kernels/ema_kernels/ema_state_fwd.py:54, and in the backward its dstates
 *      stage, kernels/ema_kernels_bwd/ema_scan_bwd.py:39 - and every piece of an item starts from the fold of the
 *      aggregates before it (the reference's state passing, kernels/ema_kernels/ema_state_pass.py:100-120), so that no
 *      thread block waits for another;
 *   2  as 1, with the aggregate schedule for every problem that has at least two tiles (tests).
 * Returns the previous setting.  Cutting with carries gives bit-identical results; the aggregate schedule agrees
 * with them to within the rounding of the bf16 decay matrices.  Both need the scratch of
 * ema_b200_fwd_workspace_bytes / ema_b200_bwd_workspace_bytes, whose value depends on this setting. */
int ema_b200_set_split(int on);
/* Schedule of the last tensor-core launch made by ema_b200_fwd / ema_b200_bwd on this thread: 0 whole items,
 * 1 items cut with carries, 2 aggregates; -1 when the last call did not use the tensor-core kernels. */
int ema_b200_last_schedule(void);
/* Kernel family the last ema_b200_fwd / ema_b200_bwd call on this thread launched: 1 = tensor cores,
 * 0 = CUDA cores, 2 = CUDA cores with x (and dy) brought in by TMA (fp32 on 16-byte aligned layouts; same
 * arithmetic and bit-identical results as 0), -1 = none yet.  Lets a test assert which path really ran. */
int ema_b200_last_path(void);

/* Number of time steps one internal tile covers for this problem.  The forward writes one saved
 * state per tile and the backward consumes them, so both report the same value for the same
 * (dtype, d, strides).  n_tiles = ceil(L / tile_steps). */
int ema_b200_tile_steps(const ema_b200_problem *p);

/* Bytes of fp32 storage for the per-tile saved states the forward hands to the backward:
 * [b*h, n_tiles, d]. */
size_t ema_b200_tile_states_bytes(const ema_b200_problem *p);

/* Bytes of scratch the backward needs (partial sums of the decay gradient, one slice per
 * channel tile, reduced by a second kernel in a fixed order: no float atomics). */
size_t ema_b200_bwd_workspace_bytes(const ema_b200_problem *p);

/* ---- fused path -------------------------------------------------------------------------- */

/* Forward scan: one read of x, one write of y (y may be null: only the states are produced).
 * Replaces the four launches of _ema_matmul_scan_combined_fwd
 * (kernels/ema_kernels/ema_combined_fwd.py:12-47) and the three of EMAChunkScanCombinedFn.forward
 * (kernels/ema.py:283-364).
 *   chunk_states  optional [b, h, ceil(L/chunk), d] fp32: state at the START of every API chunk
 *                 (the `states` the reference returns, kernels/ema_kernels/ema_state_pass.py:100-120)
 *   tile_states   optional [b*h, n_tiles, d] fp32 for ema_b200_bwd
 *   init_state    optional [b, h, d] fp32 state before step 0 (zeros when null)
 *   final_state   optional [b, h, d] fp32 state after step L-1
 *   log_decay_sum optional [b, h] fp32: sum of log a over the steps that were processed
 *   stop_below    0 to scan all L steps.  > 0: stop after the first tile at whose end the
 *                 product of decays since step 0 is below this value - used to re-scan only the
 *                 prefix an incoming carry can still influence (sequence-parallel fix-up).
 *   workspace     optional scratch of ema_b200_fwd_workspace_bytes(p) bytes, 16-byte aligned (a few
 *                 hundred KB; for problems with few work items, see ema_b200_set_split, also 4 bytes
 *                 per 128 elements of x for the per-tile aggregates).  With it the bf16 kernels cut
 *                 work items (scan row x 128 channels) across thread blocks so that every SM has
 *                 work; without it each item stays on one thread block.  Two calls that may overlap
 *                 in time must not share a scratch. */
size_t ema_b200_fwd_workspace_bytes(const ema_b200_problem *p);
int ema_b200_fwd(const ema_b200_problem *p, const void *x, const float *decay, void *y,
                 float *chunk_states, float *tile_states, const float *init_state, float *final_state,
                 float *log_decay_sum, float stop_below, void *workspace, size_t workspace_bytes,
                 void *stream);

/* Forward scan with per-step weights folded into the same pass:
 *     s_t = a_t s_{t-1} + in_weight_t x_t ,     y_t = out_weight_t s_t
 * Replaces the elementwise passes over x and over the result that surround the scan in the heads-style entry point
 * ema_chunk_scan_combined (kernels/ema_combined.py:100-128) for state size 1: in_weight = dt' B, out_weight = C,
 * decay = dt' A as a log decay (dt' as in kernels/ema_kernels/ema_chunk_state.py:69-78).
 *   in_weight   optional [b, L, h] fp32 with the decay's strides; null: the convention's weight (1 - a, or 1)
 *   out_weight  optional [b, L, h] fp32 with the decay's strides; null: 1
 * Needs a per-step decay (EMA_ERR_UNSUPPORTED otherwise).  chunk_states, tile_states and final_state receive the
 * states s themselves, not the weighted output.  Everything else as in ema_b200_fwd. */
int ema_b200_fwd_weighted(const ema_b200_problem *p, const void *x, const float *decay, const float *in_weight,
                          const float *out_weight, void *y, float *chunk_states, float *tile_states,
                          const float *init_state, float *final_state, float *log_decay_sum, float stop_below,
                          void *workspace, size_t workspace_bytes, void *stream);

/* Backward scan: reads x, dy and the saved tile states once, writes dx and d(decay).
 * Replaces the nine launches and the torch glue of _ema_chunk_scan_combined_bwd
 * (kernels/ema_kernels_bwd/ema_combined_bwd.py:13-82).
 *   ddecay        [b, L, h] (strides a_s*) or [h]; overwritten, not accumulated
 *   dfinal_state  optional [b, h, d]: gradient flowing into the state after step L-1
 *   dinit_state   optional [b, h, d]: receives the gradient of the state before step 0
 *   stop_below    as in the forward, counted from step L-1 backwards (suffix re-scan)
 *   workspace     ema_b200_bwd_workspace_bytes(p) bytes, 16-byte aligned */
int ema_b200_bwd(const ema_b200_problem *p, const void *x, const float *decay, const void *dy,
                 const float *tile_states, void *dx, float *ddecay, const float *dfinal_state,
                 float *dinit_state, float stop_below, void *workspace, size_t workspace_bytes,
                 void *stream);

/* Backward of ema_b200_fwd_weighted, in one pass over x and dy: with lambda_t = out_weight_t dy_t + a_{t+1} lambda_{t+1}
 *     dx_t = in_weight_t lambda_t,                d decay_t      = sum_d lambda_t s_{t-1}   (times a_t for a log decay),
 *     d in_weight_t = sum_d lambda_t x_t,          d out_weight_t = sum_d dy_t s_t .
 * With gradients the reference's heads-style entry point (kernels/ema_combined.py:100; its own backward is a stub,
 * :89-92) thus needs no elementwise pass over x, dy or the result around the scan: the gradients of dt, A, B, C follow
 * from these three [b, L, h] tensors by the chain rule on [b, L, h]-sized data.
 *   in_weight / out_weight  as in the forward (null: the convention's input weight / 1); per-step decay only
 *   din_weight, dout_weight fp32 [b, L, h] with the decay's strides; required when the weight is given, else null
 *   tile_states             the states s saved by the weighted forward
 *   workspace               ema_b200_bwd_weighted_workspace_bytes(p) bytes, 16-byte aligned
 * Runs on the CUDA cores for both element types (fp32 state, exact fp32 arithmetic). */
size_t ema_b200_bwd_weighted_workspace_bytes(const ema_b200_problem *p);
int ema_b200_bwd_weighted(const ema_b200_problem *p, const void *x, const float *decay, const float *in_weight,
                          const float *out_weight, const void *dy, const float *tile_states, void *dx, float *ddecay,
                          float *din_weight, float *dout_weight, const float *dfinal_state, float *dinit_state,
                          void *workspace, size_t workspace_bytes, void *stream);

/* ---- sequence-parallel carry fold ------------------------------------------------------------
 * (The reference is single-GPU; the recurrence folded here is its chunk-level carry,
 * kernels/ema_kernels/ema_state_pass.py:100-120, h <- exp(cs_last) h + S, applied to whole segments.)
 *
 * records: `world` records in rank order, each [F (rows*d floats) | logP (rows floats)]: the state a
 * rank's segment ends in when scanned from zero and the sum of its log decays - what the ranks
 * all-gather (final_state and log_decay_sum of ema_b200_fwd written into one buffer).
 *   reverse == 0: out[rows, d] = state entering segment `rank`   (fold of records 0 .. rank-1)
 *   reverse != 0: out[rows, d] = adjoint entering segment `rank` from the right (fold of records
 *                 world-1 .. rank+1, F being the dinit_state of ema_b200_bwd)                      */
int ema_b200_fold_records(const float *records, int world, int rank, int64_t rows, int64_t d, int reverse,
                          float *out, void *stream);

/* ---- backward without a workspace ---------------------------------------------------------
 * (No counterpart in the reference: its backward allocates its temporaries with torch.empty.)
 *
 * ema_b200_bwd_static_scratch() is ema_b200_bwd() for callers that can neither hand over a workspace
 * nor allocate one at the time of the call: hosts that gave all device memory to their own arena at
 * start-up, latency-critical loops in which cudaMalloc/cudaFree would stall every stream of the
 * process, and code that runs while the framework's allocator must not be entered.  The partial sums
 * of the decay gradient go to a fixed array in device memory that belongs to the library's image
 * (reserved per device when the image is loaded there); the call itself allocates and frees nothing.
 *
 *  - Limit: ema_b200_bwd_workspace_bytes(p) must not exceed ema_b200_static_scratch_limit()
 *    (8 MiB); otherwise EMA_ERR_SCRATCH_LIMIT is returned and nothing is launched.  Use
 *    ema_b200_bwd() with a caller-owned workspace for larger problems.
 *  - First call on a device: looks up the array's device address (and, like any first launch, makes
 *    the CUDA runtime load the kernels).  Make that first call at start-up, outside any stream
 *    capture; later calls only launch kernels on `stream`.
 *  - One array per device: two calls on the same device whose kernels may overlap (different
 *    streams, or several host threads) race on it and give wrong ddecay.  Order them on one stream or
 *    with events.  Calls on different devices are independent.
 *  - The array needs no clearing: each call writes every partial sum before reading it.
 *  - No dfinal_state / dinit_state / stop_below: the sequence-parallel fix-up passes use
 *    ema_b200_bwd().  Results equal those of ema_b200_bwd() on the same inputs.                  */
size_t ema_b200_static_scratch_limit(void);
int ema_b200_bwd_static_scratch(const ema_b200_problem *p, const void *x, const float *decay, const void *dy,
                                const float *tile_states, void *dx, float *ddecay, void *stream);

/* ---- stage kernels on the reference's folded layouts --------------------------------------
 * X, dout, out, dx: [B, L, T] contiguous, element type `dtype`;  A: [B, L] fp32 with element
 * strides (A_sb, A_sl);  cs: [B, C, Q] fp32 contiguous;  per-chunk states: [B, C, T] fp32
 * contiguous;  C = ceil(L / Q). */

/* ema_chunk_cumsum_fwd, kernels/ema_kernels/ema_cumsum.py:66 (kernel :32). */
int ema_b200_chunk_cumsum(const float *A, int64_t A_sb, int64_t A_sl, float *cs, int64_t B,
                          int64_t L, int Q, void *stream);
/* _ema_chunk_state_fwd, kernels/ema_kernels/ema_state_fwd.py:130 (kernel :54). */
int ema_b200_chunk_state(const void *X, const float *cs, float *S, int dtype, int64_t B, int64_t L,
                         int64_t T, int Q, void *stream);
/* _ema_state_passing_fwd, kernels/ema_kernels/ema_state_pass.py:125 (kernel :57).
 * cs_last has element strides (cl_sb, cl_sc) so that the view cs[..., -1] can be passed as is. */
int ema_b200_state_passing_fwd(const float *S, const float *cs_last, int64_t cl_sb, int64_t cl_sc,
                               float *out, float *final_states, int64_t B, int64_t C, int64_t T,
                               void *stream);
/* _ema_scan_fwd, kernels/ema_kernels/ema_scan_fwd.py:161 (kernel :53). */
int ema_b200_chunk_scan(const void *X, const float *cs, const float *h, void *out, int dtype,
                        int64_t B, int64_t L, int64_t T, int Q, void *stream);
/* _ema_chunk_scan_bwd_dstates, kernels/ema_kernels_bwd/ema_scan_bwd.py:132 (kernel :39). */
int ema_b200_bwd_dstates(const float *cs, const void *dout, float *dh, int dtype, int64_t B,
                         int64_t L, int64_t T, int Q, void *stream);
/* _ema_state_passing_bwd, kernels/ema_kernels_bwd/ema_state_passing_bwd_dstates.py:103 (kernel :20).
 * workspace (optional, ema_b200_state_passing_bwd_workspace_bytes(B, C, T) bytes, 4-byte aligned): per-warp
 * partial dot products [B, C, ceil(T/128)], the counterpart of the partial-sum buffer the reference's wrapper
 * allocates (:134-142).  With it (and T a multiple of 4, 16-byte aligned tensors) a batch row is spread over T / 128
 * thread blocks with 128-bit accesses and the partials are summed in a fixed order by a second kernel; without it
 * one thread block walks a whole row (T <= 16384). */
size_t ema_b200_state_passing_bwd_workspace_bytes(int64_t B, int64_t C, int64_t T);
int ema_b200_state_passing_bwd(const float *h, const float *cs_last, int64_t cl_sb, int64_t cl_sc,
                               const float *dh, float *dS, float *ddA_last, int64_t B, int64_t C,
                               int64_t T, void *workspace, size_t workspace_bytes, void *stream);
/* _chunk_scan_chunk_state_bwd_dx, kernels/ema_kernels_bwd/ema_chunk_scan_chunk_state_bwd_dx.py:208 (kernel :69). */
int ema_b200_bwd_dx(const float *cs, const void *dout, const float *dS, void *dx, int dtype,
                    int64_t B, int64_t L, int64_t T, int Q, void *stream);
/* _ema_chunk_state_bwd_db, kernels/ema_kernels_bwd/ema_chunk_state_bwd_db.py:122 (kernel :28);
 * raw != 0 skips the cumulative sum, like raw_scale_gradient=True. */
int ema_b200_bwd_db(const void *X, const float *cs, const float *dS, float *ddA, int dtype, int raw,
                    int64_t B, int64_t L, int64_t T, int Q, void *stream);
/* _ema_chunk_scan_bwd_dC, kernels/ema_kernels_bwd/ema_chunk_scan_bwd_dc.py:115 (kernel :25). */
int ema_b200_bwd_dc(const float *h, const float *cs, const void *dout, float *ddA, int dtype,
                    int64_t B, int64_t L, int64_t T, int Q, void *stream);
/* _ema_chunk_scan_bwd_ddAcs_stable, kernels/ema_kernels_bwd/ema_scan_da.py:113 (kernel :25). */
int ema_b200_bwd_dacs(const void *X, const float *cs, const void *dout, float *ddA, int dtype,
                      int64_t B, int64_t L, int64_t T, int Q, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* EMA_B200_H */
