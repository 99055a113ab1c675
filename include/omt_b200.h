/* omt_b200.h -- C ABI of libomt_b200.so: the B200 (sm_100a) runtime and kernels under the
 * "omarchy_mac_torch" PyTorch device.
 *
 * This is the boundary the reference's op layer sits on. In the reference the op files (csrc/conv.cpp, nn.cpp,
 * fused.cpp, plans.cpp, optim.cpp) call a wgpu runtime through csrc/omt.h:48-106 (alloc_buf / launch / uniform /
 * sync_all ...) with kernel *names*; here they call these entry points instead. Every function:
 *   - takes plain device pointers, sizes and a stream handle (a cudaStream_t cast to omt_stream_t; NULL = the
 *     legacy default stream); no torch or C++ types cross this boundary;
 *   - returns 0 on success or a negative OMT_E* code; the message is read with omt_last_error();
 *   - never throws, never falls back to the host: there is no CPU path in this library.
 * There are no collective entry points here: the one exchange step of data-parallel training (the gradient all-reduce)
 * is issued by the Python layer through torch.distributed's NCCL backend on the buckets this library's kernels wrote, so
 * the library neither links NCCL nor touches peer memory.
 * All tensors are float32 unless stated. Activations are addressed through OmtAct (pointer + element strides), so
 * the same entry point serves NCHW-contiguous tensors (the reference's only layout, csrc/device.cpp:60-66 base0)
 * and channels-last (NHWC) tensors, which is what the tensor-core kernels prefer.
 */
#ifndef OMT_B200_H
#define OMT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* omt_stream_t; /* cudaStream_t */
typedef void* omt_event_t;  /* cudaEvent_t  */

enum {
  OMT_OK = 0,
  OMT_EINVAL = -1,      /* argument outside what the kernels cover (the op layer's NEED() cases) */
  OMT_ECUDA = -2,       /* a CUDA runtime call failed; omt_last_error() has cudaGetErrorString */
  OMT_ENOMEM = -3,      /* device allocation failed even after releasing the cache */
  OMT_EWORKSPACE = -4,  /* caller-provided workspace too small */
  OMT_ETOOBIG = -5      /* beyond the fixed capacity of a no-allocation entry point */
};

/* ---- geometry ------------------------------------------------------------------------------------------------ */

/* Convolution geometry. Mirrors the reference's `Geo` (csrc/omt.h:224-226) and `conv_geo` (csrc/conv.cpp:19-21):
 * square kernel ks, one stride and one padding for both axes, no dilation. groups is 1 (dense) or ci (depthwise). */
typedef struct OmtConvGeo {
  int32_t n, ci, co, ih, iw, oh, ow, ks, stride, pad, groups;
} OmtConvGeo;

/* An activation tensor [n, c, h, w] given by its base pointer and element strides. */
typedef struct OmtAct {
  float* p;
  int64_t sn, sc, sh, sw;
} OmtAct;

/* epilogue / behaviour flags of the conv entry points */
enum {
  OMT_EPI_BIAS = 1,        /* y += bias[co]          (reference hb bit 0, omarchy_mac_torch/gemm.py:37) */
  OMT_EPI_RELU = 2,        /* y = max(y, 0)          (reference hb bit 1, omarchy_mac_torch/gemm.py:38) */
  OMT_EPI_BNSTATS = 4,     /* omt_conv_fwd: also write batch-norm partial statistics of y (see omt_conv_bnstats_groups) */
  OMT_EPI_ACCUM = 8,       /* omt_conv_dgrad: dx += result (gradient of a tensor with a second consumer, e.g. a residual branch) */
  OMT_PRECISE_ACCUM = 0x400, /* tensor-core path: always keep the 3xTF32 cross terms in their own accumulator (by default 128 x 256
                              * tiles with a reduction of at most 1152 share one, which lets their epilogue overlap the next tile) */
  OMT_FORCE_SIMT = 0x100,  /* skip the tcgen05 path (used by tests to cross-check the two paths) */
  OMT_FORCE_TC = 0x200     /* fail with OMT_EINVAL instead of taking the SIMT path */
};

/* ---- runtime: replaces csrc/runtime.cpp + the allocator/guard half of csrc/device.cpp -------------------------- */

/* Select and initialise a device (creates the context lazily like init_ctx, csrc/runtime.cpp:83-127). */
int omt_init(int device_ordinal);
int omt_device(void);
/* Copies the last error message of the calling thread into buf; returns its length. */
int omt_last_error(char* buf, size_t n);
/* Sticky asynchronous error check (reference check_errors, csrc/runtime.cpp:73-81): returns OMT_ECUDA once a
 * kernel or copy has failed. */
int omt_check_errors(void);
/* Waits for all work on the device (reference sync_all, csrc/runtime.cpp). */
int omt_sync(void);

/* Caching allocator (reference alloc_buf/free_buf/empty_cache, csrc/runtime.cpp:183-240; c10 allocator
 * csrc/device.cpp:18-30). Blocks are rounded to size classes and reused; a block freed while streams other than its
 * allocation stream still use it (omt_record_stream) is parked until their recorded events complete. On
 * cudaErrorMemoryAllocation the cache is released and the allocation retried once (csrc/runtime.cpp:219-225). */
void* omt_malloc(size_t bytes, omt_stream_t stream);
void omt_free(void* p);
int omt_record_stream(void* p, omt_stream_t stream);
void omt_empty_cache(void);
size_t omt_memory_allocated(void);
size_t omt_memory_reserved(void);

/* Streams and events (reference Guard, csrc/device.cpp:120-162, had one in-order queue; here: real streams). */
omt_stream_t omt_stream_create(int high_priority);
int omt_stream_destroy(omt_stream_t s);
int omt_stream_sync(omt_stream_t s);
int omt_stream_query(omt_stream_t s); /* 1 = idle, 0 = busy, <0 error */
omt_event_t omt_event_create(int timing);
int omt_event_destroy(omt_event_t e);
int omt_event_record(omt_event_t e, omt_stream_t s);
int omt_event_query(omt_event_t e); /* 1 = complete */
int omt_event_sync(omt_event_t e);
int omt_stream_wait_event(omt_stream_t s, omt_event_t e);
int omt_event_elapsed_ms(omt_event_t a, omt_event_t b, float* ms);

/* Transfers (reference upload_bytes/download_bytes/record_copy, csrc/runtime.cpp). d2h waits for the copy. */
int omt_memcpy_h2d(void* dst, const void* src, size_t bytes, omt_stream_t s);
int omt_memcpy_d2h(void* dst, const void* src, size_t bytes, omt_stream_t s);
int omt_memcpy_d2d(void* dst, const void* src, size_t bytes, omt_stream_t s);
int omt_memset(void* dst, int byte, size_t bytes, omt_stream_t s);

/* Launch accounting (reference stats().kcount, csrc/runtime.cpp:598-610, bound as kernel_counts in
 * csrc/module.cpp:30-33). omt_launch_count is the number of kernels of this library launched so far. */
uint64_t omt_launch_count(void);
/* Writes "name=count\n" lines for every kernel launched since the last reset; returns bytes needed. */
size_t omt_kernel_counts(char* buf, size_t n, int reset);

/* Per-kernel device timing (reference set_debug_time_kernels / kernel_times, csrc/runtime.cpp:598-610, bound in
 * csrc/module.cpp:30-33). While enabled, every kernel this library launches is bracketed by CUDA events on its stream
 * (the first kernel of an entry point from an event recorded at its start, the following ones from their predecessor).
 * omt_kernel_times waits for the recorded events and writes "name=milliseconds\n" lines, summed per kernel name; it
 * returns the bytes needed. A debugging aid: it creates two events per launch and is not meant for timed runs. */
int omt_kernel_timing(int enable);
size_t omt_kernel_times(char* buf, size_t n, int reset);

/* ---- dense convolution: reference gemm_forward / gemm_grad_input / gemm_grad_weight + csum_nchw ---------------- */

/* Scratch bytes omt_conv_* needs for this geometry (kind: 0 fwd, 1 dgrad, 2 wgrad). When the caller passes
 * workspace == NULL the library takes the scratch from its own caching allocator on `stream`. */
size_t omt_conv_workspace_bytes(int kind, const OmtConvGeo* g, uint32_t flags);

/* Per-geometry plan overrides and the timing pass that finds them. Replaces the reference's tuning cache and autotune
 * (csrc/conv.cpp:29-60 conv_plan / g_conv_cache, :116-155 autotune, :243-272 tune_dump / tune_load). The tensor-core
 * kernels pick their tile width and the weight gradient's split-K slice count from the geometry by fixed rules; an
 * override replaces that choice for one (pass, geometry): pass 0 forward, 1 input gradient, 2 weight gradient; `tile` =
 * tile width in columns (64, 128, 256; 192 for the weight gradient; 0 = the rule), `mult` = factor on the rule's slice
 * count (weight gradient only; 1 = the rule). omt_conv_workspace_bytes and omt_conv_bnstats_groups follow the override.
 * omt_conv_autotune times the rules and every candidate on zero-filled channels-last operands of the geometry
 * (allocated from the library's caching allocator; one warm-up call, then about 15 ms of timed calls per candidate,
 * CUDA events on `stream`, which it synchronises: not inside a stream capture), stores the fastest as the override if it
 * beats the rules by more than 3 % (else removes any override) and reports the choice. Geometries the tensor-core path
 * does not take, or where a width would split the reduction over CTAs, are left to the rules (tile 0).
 * omt_conv_plans_dump writes "pass,n,ci,co,ih,iw,oh,ow,ks,stride,pad=tile,mult\n" lines for all overrides and returns
 * the bytes needed; omt_conv_plans_load reads such lines (skipping those it cannot use) and returns how many it took. */
int omt_conv_plan_set(int kind, const OmtConvGeo* g, int32_t tile, double mult);
int omt_conv_plan_get(int kind, const OmtConvGeo* g, int32_t* tile, double* mult); /* 1 if an override is stored, else 0 */
int omt_conv_autotune(int kind, const OmtConvGeo* g, int32_t* tile, double* mult, float* best_ms, float* rule_ms, omt_stream_t stream);
size_t omt_conv_plans_dump(char* buf, size_t n);
int omt_conv_plans_load(const char* text);

/* y[n,co,oh,ow] = conv(x, w) (+bias)(ReLU). w is [co, ci, ks, ks] contiguous. Replaces gemm_forward
 * (csrc/conv.cpp:70-77) and the kind-0 generated kernel (omarchy_mac_torch/gemm.py:25-42).
 * With OMT_EPI_BNSTATS the epilogue also reduces the values it stores into batch-norm partial statistics, so that the
 * BatchNorm that follows need not read y for its statistics pass (the reference's plans run bn_stats_part over y,
 * csrc/plans.cpp:180-194): for every group of 32 output rows and every channel, `stats` receives the group's sum and its
 * sum of squared deviations from the group's own mean, then the groups' row counts; omt_bn_stats_from_partials merges
 * them. `stats` must hold omt_conv_bnstats_floats(groups, co) floats; nothing needs zeroing; the result is
 * deterministic. Only calls for which omt_conv_bnstats_groups() is non-zero may pass the flag. */
int omt_conv_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y,
                 float* stats, uint32_t flags, void* workspace, size_t workspace_bytes, omt_stream_t stream);
/* Number of 32-row groups omt_conv_fwd(OMT_EPI_BNSTATS) writes partial statistics for with these operands, or 0 when that
 * call cannot produce them (a geometry or layout off the tensor-core path, an output that is not dense channels-last, a
 * reduction split over several CTAs) or would lose by it (a reduction so short that the layer is bound by storing y):
 * the caller then runs omt_bn_stats on y instead. */
int32_t omt_conv_bnstats_groups(const OmtConvGeo* g, const OmtAct* x, const OmtAct* y);
/* Floats of the partial-statistics buffer: groups * (2 * co + 1) values and ceil(co / 32) words the merge uses. */
size_t omt_conv_bnstats_floats(int32_t groups, int32_t co);

/* dx[n,ci,ih,iw] = conv^T(gy, w). Any stride 1..4: strided convs are split into stride^2 phases, each a dense
 * GEMM over the taps that land on it, batched in one launch. Replaces gemm_grad_input (csrc/conv.cpp:78-100) and
 * kinds 1 and 5 (omarchy_mac_torch/gemm.py:43-80). With OMT_EPI_ACCUM the result is added to what dx holds (autograd's
 * accumulation of a second gradient into the same tensor, done in the epilogue); only the tensor-core path does that:
 * other geometries return OMT_EINVAL and the caller adds separately. */
int omt_conv_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, uint32_t flags,
                   void* workspace, size_t workspace_bytes, omt_stream_t stream);

/* dw[co,ci,ks,ks] = sum over (n,oy,ox) of gy * im2col(x); split-K partial slabs in the workspace, then a
 * deterministic slab sum. Replaces gemm_grad_weight (csrc/conv.cpp:102-114), kind 2 (omarchy_mac_torch/gemm.py:81-91)
 * and csrc/kernels/gemm_reduce.wgsl. `scale` multiplies the result (1/world_size pre-scaling for data parallel). */
int omt_conv_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, uint32_t flags,
                   void* workspace, size_t workspace_bytes, omt_stream_t stream);

/* Weight gradient for callers that must not allocate device memory. No counterpart in the reference.
 * Some hosts of this library cannot call cudaMalloc while they run: code replaying a fixed launch sequence inside a
 * real-time loop, or a process whose device memory was handed out in full at start-up and that has no allocator of its
 * own to ask. omt_conv_wgrad needs split-K scratch (from the caller's workspace or the library's allocator); this
 * variant runs the same exact-fp32 kernels with the scratch in a fixed array inside the library image instead, and
 * calls no cudaMalloc, cudaFree or allocating library routine.
 *   - Capacity: omt_conv_wgrad_noalloc_capacity() bytes (16 MiB) of split-K slabs; a geometry that needs more is refused
 *     with OMT_ETOOBIG. Every GPU that loads the library holds that array until the process exits.
 *   - The first call on each device looks up the array's device address (with that device current). With CUDA's lazy
 *     module loading that lookup is also what makes the driver load the library's image and back the 16 MiB array with
 *     device memory, so the FIRST call per device can itself need memory: make it once at start-up, before the process
 *     hands out the rest of the device's memory, and outside any stream capture. Later calls allocate nothing.
 *   - All calls on a device share the array. The slabs are fully overwritten by every call, so nothing needs clearing,
 *     but two calls that overlap on the GPU (different streams) race on it: keep them on one stream or order them. */
size_t omt_conv_wgrad_noalloc_capacity(void);
int omt_conv_wgrad_noalloc(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale,
                           omt_stream_t stream);

/* db[c] = sum over (n,h,w) of gy. Replaces csrc/kernels/csum_nchw.wgsl (csrc/conv.cpp:232-235). */
int omt_conv_bias_grad(const OmtAct* gy, int32_t n, int32_t c, int32_t h, int32_t w, float* db, float scale,
                       omt_stream_t stream);

/* out[M,N] (row-major) = A[M,K] * B[K,N] (+ bias[N]) in float32 on the same tensor-core kernels: a matrix product is the
 * 1x1 case of the implicit GEMM (rows = pixels). Replaces mm_into / mm_ / addmm_ (csrc/linalg.cpp:25-92; the generated
 * kind-4 kernel, omarchy_mac_torch/gemm.py). A and B are given by pointer and element strides (row stride, column stride);
 * three operand layouts map onto the three conv passes and are taken without a copy:
 *   A row-major, B column-major (B = W^T with W [N,K] row-major: nn.Linear forward)          -> the forward kernel (+ bias)
 *   A row-major, B row-major    (grad_output * W: nn.Linear's input gradient)                -> the input-gradient kernel
 *   A column-major, B row-major (A = G^T with G [K,M] row-major: nn.Linear's weight gradient) -> the weight-gradient kernel
 * Any other stride pattern, or a bias outside the first case, returns OMT_EINVAL (the caller copies or adds). */
int omt_gemm(const float* a, int64_t a_row_stride, int64_t a_col_stride, const float* b, int64_t b_row_stride,
             int64_t b_col_stride, const float* bias, float* out, int32_t M, int32_t N, int32_t K, omt_stream_t stream);

/* Per-call device timing of the dense-conv entry points (reference debug_time_kernels / kernel_times,
 * csrc/runtime.cpp:598-610, csrc/module.cpp:30-33). While enabled, omt_conv_fwd/dgrad/wgrad bracket their launches with
 * CUDA events on the caller's stream. omt_conv_timing_read synchronises those events and returns, per pass (index 0 fwd,
 * 1 dgrad, 2 wgrad), the summed algorithmic FLOPs (2*n*co*oh*ow*ci*ks*ks per call, tools/gemm_bench.py:29), the summed
 * milliseconds and the number of calls; `reset` clears the records. */
int omt_conv_timing(int enable);
int omt_conv_timing_read(double flops[3], double ms[3], int64_t calls[3], int reset);
/* The summed algorithmic bytes of the recorded calls per pass: float32 input + output activation + weights of each call
 * (what one pass must move through HBM at least once). Read it before omt_conv_timing_read(..., reset = 1). */
int omt_conv_timing_bytes(double bytes[3]);

/* ---- depthwise convolution: reference dw_fwd/dw_gin/dw_gwt and dwg_* (csrc/conv.cpp:194-229) ------------------- */

int omt_dw_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y,
               uint32_t flags, omt_stream_t stream);
int omt_dw_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, omt_stream_t stream);
int omt_dw_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale,
                 omt_stream_t stream);

/* ---- batch norm: reference batch_norm_ / batch_norm_backward_ (csrc/nn.cpp:25-78), bn_relu_* (csrc/fused.cpp) --- */

enum {
  OMT_BN_RELU = 1,       /* apply / mask ReLU */
  OMT_BN_FUNCTIONAL = 2, /* running stats go to new_rm/new_rv */
  /* ReLU mask as bits. omt_bn_apply(_add) with OMT_BN_RELU also writes, directly behind y (at y.p + n*c*h*w, so y's
   * allocation must extend ceil(n*c*h*w / 32) words further), one bit per element in memory order: word k, bit b =
   * (y[32k + b] > 0). omt_bn_backward(_add) with OMT_BN_RELU then takes the mask from those words and reads none of y's
   * values: 1/8 byte per element and pass instead of 4. The reference's bn_bwd_part / bn_bwd_apply shaders read y
   * (bn_bwd_part.wgsl:25-38, bn_bwd_apply.wgsl:19-23). */
  OMT_BN_MASKBITS = 4
};

/* Per-channel batch statistics. mean[c], var[c] (biased), from shifted sums like bn_stats_part/fin
 * (csrc/kernels/bn_stats_part.wgsl:22-31, bn_stats_fin.wgsl:15-21). Also updates the running statistics:
 * rm += momentum*(mean-rm), rv += momentum*(var*count/(count-1) - rv); with OMT_BN_FUNCTIONAL the updated values
 * are written to new_rm/new_rv instead and rm/rv are left alone (bn_stats_fin_functional.wgsl). rm may be NULL.
 * invstd[c] = rsqrt(var+eps) is written as well. */
int omt_bn_stats(const OmtAct* x, int32_t n, int32_t c, int32_t h, int32_t w, float* mean, float* var,
                 float* invstd, float* rm, float* rv, float* new_rm, float* new_rv, float momentum, float eps,
                 uint32_t flags, omt_stream_t stream);
/* Same outputs as omt_bn_stats, from the partial statistics a conv epilogue wrote (OMT_EPI_BNSTATS; `groups` from
 * omt_conv_bnstats_groups): the groups are merged pairwise with the exact update for mean and squared deviations, in a
 * fixed order, so the variance is accurate for any mean (the property bn_stats_part.wgsl:22-31 gets from its shift). */
int omt_bn_stats_from_partials(const float* partials, int32_t groups, int32_t c, float* mean, float* var, float* invstd,
                               float* rm, float* rv, float* new_rm, float* new_rv, float momentum, float eps,
                               uint32_t flags, omt_stream_t stream);
/* y = (x-mean)*invstd*gamma+beta, ReLU with OMT_BN_RELU (bn_apply.wgsl:17-18, bn_relu.wgsl:17-18). */
int omt_bn_apply(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w, const float* mean,
                 const float* invstd, const float* gamma, const float* beta, uint32_t flags, omt_stream_t stream);
/* y = (x-mean)*invstd*gamma+beta + res, ReLU with OMT_BN_RELU: the tail of a residual block (BatchNorm, add the
 * identity branch, ReLU) in the pass bn_apply makes anyway. `res` has the layout of x; NULL (or res->p NULL) makes it
 * omt_bn_apply. The reference's compile pass 1 (omarchy_mac_torch/compile.py:69-96) fuses BatchNorm+ReLU only; this is
 * the same rewrite carried across the add. */
int omt_bn_apply_add(const OmtAct* x, const OmtAct* res, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w,
                     const float* mean, const float* invstd, const float* gamma, const float* beta, uint32_t flags,
                     omt_stream_t stream);
/* omt_bn_apply followed by the plan's 2x2 stride-2 max pool (omt_pool2_fwd) in one pass over x: z[n,c,h/2,w/2] is the
 * pooled output and idx (strides of z; may be NULL) its argmax in {0..3}; y (full resolution, what the ReLU-masked
 * backward reads; y->p may be NULL) is written on the way. The reference runs bn_relu then pool_fwd as two dispatches
 * (csrc/plans.cpp:180-194, 188-199). Needs even h and w; the three tensors share one layout. */
int omt_bn_apply_pool2(const OmtAct* x, const OmtAct* y, const OmtAct* z, uint8_t* idx, int32_t n, int32_t c, int32_t h,
                       int32_t w, const float* mean, const float* invstd, const float* gamma, const float* beta,
                       uint32_t flags, omt_stream_t stream);
/* Eval mode: invstd = rsqrt(rv+eps) computed on the fly (bn_eval_inv.wgsl, bn_relu_rv.wgsl). */
int omt_bn_eval(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w, const float* rm,
                const float* rv, const float* gamma, const float* beta, float eps, uint32_t flags,
                omt_stream_t stream);
/* Backward (training). dgamma=sum g*xhat, dbeta=sum g, dx=gamma*invstd/m*(m*g-dbeta-xhat*dgamma)
 * (bnb_reduce.wgsl:25-37, bnb_apply.wgsl:19-21). With OMT_BN_RELU, g is first masked by y>0
 * (bn_bwd_part.wgsl:25-38, bn_bwd_apply.wgsl:19-23); y is then required. dx->p may be NULL (mask[0] false).
 * dgb is [2*c]: row 0 dgamma, row 1 dbeta (the layout csrc/nn.cpp:70 uses). scale multiplies dgamma/dbeta only. */
int omt_bn_backward(const OmtAct* gy, const OmtAct* x, const OmtAct* y, const OmtAct* dx, int32_t n, int32_t c,
                    int32_t h, int32_t w, const float* mean, const float* invstd, const float* gamma, float* dgb,
                    float scale, uint32_t flags, omt_stream_t stream);
/* Same with a second output for the backward of omt_bn_apply_add: dres = gy masked by y>0, the gradient of the
 * identity branch, written by the dx pass (needs OMT_BN_RELU and dx). dres NULL makes it omt_bn_backward. */
int omt_bn_backward_add(const OmtAct* gy, const OmtAct* x, const OmtAct* y, const OmtAct* dx, const OmtAct* dres,
                        int32_t n, int32_t c, int32_t h, int32_t w, const float* mean, const float* invstd,
                        const float* gamma, float* dgb, float scale, uint32_t flags, omt_stream_t stream);

/* ---- pooling: plan kernels (pool_fwd/bwd, avgpool_fwd/bwd, gap_fwd/bwd) and general ops (csrc/nn.cpp:137-222) --- */

/* 2x2 stride-2 max pool; idx[n,c,oh,ow] in {0..3} = (dy*2+dx) of the first maximum (strict >), pool_fwd.wgsl:15-21.
 * idx has the strides of y. */
int omt_pool2_fwd(const OmtAct* x, const OmtAct* y, uint8_t* idx, int32_t n, int32_t c, int32_t h, int32_t w,
                  omt_stream_t stream);
int omt_pool2_bwd(const OmtAct* gy, const uint8_t* idx, const OmtAct* gx, int32_t n, int32_t c, int32_t h,
                  int32_t w, omt_stream_t stream);
int omt_avgpool2_fwd(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w,
                     omt_stream_t stream);
int omt_avgpool2_bwd(const OmtAct* gy, const OmtAct* gx, int32_t n, int32_t c, int32_t h, int32_t w,
                     omt_stream_t stream);
/* General max pool with aten semantics: int64 indices = flat iy*iw+ix, NaN propagates
 * (maxpool_gen_fwd.wgsl:16-28). idx has the strides of y. */
typedef struct OmtPool {
  int32_t kh, kw, sh, sw, ph, pw, dh, dw;
} OmtPool;
int omt_maxpool_fwd(const OmtAct* x, const OmtAct* y, int64_t* idx, int32_t n, int32_t c, int32_t ih, int32_t iw,
                    int32_t oh, int32_t ow, const OmtPool* p, omt_stream_t stream);
int omt_maxpool_bwd(const OmtAct* gy, const int64_t* idx, const OmtAct* gx, int32_t n, int32_t c, int32_t ih,
                    int32_t iw, int32_t oh, int32_t ow, const OmtPool* p, omt_stream_t stream);
/* avg pool with aten divisor rules (avgpool_gen_fwd.wgsl); divisor 0 = none. */
int omt_avgpool_fwd(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh,
                    int32_t ow, const OmtPool* p, int32_t count_include_pad, int32_t divisor, omt_stream_t stream);
int omt_avgpool_bwd(const OmtAct* gy, const OmtAct* gx, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh,
                    int32_t ow, const OmtPool* p, int32_t count_include_pad, int32_t divisor, omt_stream_t stream);
/* adaptive average pool (adapool_fwd/bwd.wgsl; gap_fwd/bwd.wgsl are the 1x1 case). */
int omt_adaptive_avgpool_fwd(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t ih, int32_t iw,
                             int32_t oh, int32_t ow, omt_stream_t stream);
int omt_adaptive_avgpool_bwd(const OmtAct* gy, const OmtAct* gx, int32_t n, int32_t c, int32_t ih, int32_t iw,
                             int32_t oh, int32_t ow, omt_stream_t stream);

/* ---- fused optimizers: reference fused_sgd_ / adam_impl (csrc/optim.cpp:12-61), sgd.wgsl, adam.wgsl ------------- */

/* One entry per parameter tensor. The reference issues one dispatch per parameter (csrc/optim.cpp:20-25); here one
 * launch walks the whole table. `step` is the device float32 step counter of that parameter (Adam only). */
typedef struct OmtParam {
  float* p;
  const float* g;
  float* m;          /* SGD momentum buffer (may be NULL) / Adam exp_avg */
  float* v;          /* Adam exp_avg_sq */
  const float* step; /* Adam: device scalar holding the (already incremented) step count */
  int64_t numel;
} OmtParam;

/* g=+-g+wd*p; v=first?g:mom*m+(1-damp)*g; d=nesterov?g+mom*v:v; p-=lr*d  (sgd.wgsl:9-24).
 * `table` is a HOST array of `count` entries. The library keeps device copies of the last few distinct tables (a
 * training loop passes the same one every step), so only the first call with a given table uploads it. */
int omt_sgd(const OmtParam* table, int32_t count, float lr, float momentum, float dampening, float weight_decay,
            int32_t nesterov, int32_t first_step, int32_t maximize, omt_stream_t stream);
/* Adam / AdamW (decoupled=1), adam.wgsl:13-27: bias corrections from the device step counter. */
int omt_adam(const OmtParam* table, int32_t count, float lr, float beta1, float beta2, float eps,
             float weight_decay, int32_t decoupled, int32_t maximize, omt_stream_t stream);

/* ---- fused pointwise chains: reference omt::fused_pointwise (csrc/fused.cpp:139-170) + compile pass 4 ---------------- */

/* A chain of elementwise ops as a straight-line program. The reference generates shader source per chain
 * (omarchy_mac_torch/compile.py:256-336); here the chain is data for one ahead-of-time kernel. Instruction j computes value
 * slot OMT_PW_MAX_INPUTS + j from up to three operands; an operand >= 0 names a value slot (0..n_inputs-1: the inputs;
 * OMT_PW_MAX_INPUTS + i: the result of an earlier instruction i), an operand < 0 names literal[-1 - operand]. The last
 * instruction's value is the output. Op semantics follow the aten ops of the reference's table (compile.py:176-222):
 * ADD/SUB/RSUB take alpha as third operand; THRESHOLD_BWD is (grad, self, threshold); the *_BWD ops are (grad, x or y). */
enum {
  OMT_PW_ADD, OMT_PW_SUB, OMT_PW_RSUB, OMT_PW_MUL, OMT_PW_DIV, OMT_PW_NEG, OMT_PW_RELU, OMT_PW_EXP, OMT_PW_LOG, OMT_PW_SQRT,
  OMT_PW_RSQRT, OMT_PW_RECIP, OMT_PW_ABS, OMT_PW_TANH, OMT_PW_SIGMOID, OMT_PW_SILU, OMT_PW_MAX, OMT_PW_MIN, OMT_PW_POW,
  OMT_PW_THRESHOLD_BWD, OMT_PW_SIGMOID_BWD, OMT_PW_TANH_BWD, OMT_PW_SILU_BWD, OMT_PW_GELU, OMT_PW_GELU_TANH, OMT_PW_GELU_BWD,
  OMT_PW_GELU_TANH_BWD, OMT_PW_CLAMP, OMT_PW_HARDSWISH, OMT_PW_HARDSWISH_BWD, OMT_PW_HARDSIGMOID, OMT_PW_HARDSIGMOID_BWD,
  OMT_PW_OP_COUNT
};
#define OMT_PW_MAX_INPUTS 6
#define OMT_PW_MAX_INSTR 24
#define OMT_PW_MAX_LITERALS 24
typedef struct OmtPwInstr {
  int32_t op, a, b, c;
} OmtPwInstr;
typedef struct OmtPwProgram {
  int32_t n_instr;
  OmtPwInstr instr[OMT_PW_MAX_INSTR];
  float literal[OMT_PW_MAX_LITERALS];
} OmtPwProgram;
/* out = program(inputs) elementwise over `shape` (rank <= 8). in_strides holds 8 element strides per input (0 in a
 * dimension the input broadcasts along), out_strides the output's. One launch. */
int omt_pointwise(const OmtPwProgram* prog, int32_t n_inputs, const float* const* inputs, const int64_t* in_strides,
                  const int64_t* out_strides, const int32_t* shape, int32_t rank, float* out, omt_stream_t stream);

/* ---- classification loss --------------------------------------------------------------------------------------------- */
/* F.cross_entropy on [rows, cols] float32 logits decomposes into log_softmax and nll_loss; the reference runs them as
 * softmax.wgsl (mode 1), nll_fwd.wgsl + two row reductions + a division, nll_bwd.wgsl and softmax_bwd.wgsl
 * (csrc/reduce.cpp:128-201). Matrices are dense row-major; targets are int64 class indices; `weight` ([cols]) may be NULL;
 * rows whose target equals ignore_index contribute nothing; reduction: 0 none (loss is [rows], total_weight 0),
 * 1 mean (sum of -w*logp / sum of w), 2 sum. A target outside [0, cols) makes the loss NaN and gets a zero gradient. */
/* logp = x - logsumexp(x) along each row. */
int omt_log_softmax(const float* x, float* logp, int64_t rows, int32_t cols, omt_stream_t stream);
/* dx = g - exp(logp) * rowsum(g). */
int omt_log_softmax_backward(const float* g, const float* logp, float* dx, int64_t rows, int32_t cols, omt_stream_t stream);
/* loss and total weight from log-probabilities, one launch (rows summed in a fixed order by the last block). */
int omt_nll_loss(const float* logp, const int64_t* target, const float* weight, float* loss, float* total_weight, int64_t rows,
                 int32_t cols, int64_t ignore_index, int32_t reduction, omt_stream_t stream);
/* dlogp: -w[t] * g (/ total_weight for mean) at the target column, 0 elsewhere; g is [rows] for reduction none, else [1]. */
int omt_nll_loss_backward(const float* g, const int64_t* target, const float* weight, const float* total_weight, float* dlogp,
                          int64_t rows, int32_t cols, int64_t ignore_index, int32_t reduction, omt_stream_t stream);
/* Both steps in one launch from the logits: writes logp (what the backward needs), loss and total_weight. */
int omt_softmax_nll(const float* x, const int64_t* target, const float* weight, float* logp, float* loss, float* total_weight,
                    int64_t rows, int32_t cols, int64_t ignore_index, int32_t reduction, omt_stream_t stream);
/* Gradient with respect to the logits in one launch: (exp(logp) - onehot(target)) * w[t] * g (/ total_weight). */
int omt_softmax_nll_backward(const float* g, const float* logp, const int64_t* target, const float* weight,
                             const float* total_weight, float* dx, int64_t rows, int32_t cols, int64_t ignore_index,
                             int32_t reduction, omt_stream_t stream);

/* ---- small helpers used by plans and data parallel ---------------------------------------------------------------- */

/* dst = src * scale over n floats (bucket averaging after all-reduce; icopy.wgsl when scale == 1). */
int omt_scale_copy(float* dst, const float* src, int64_t n, float scale, omt_stream_t stream);
/* strided copy between two activation views (layout change NCHW <-> NHWC). */
int omt_act_copy(const OmtAct* src, const OmtAct* dst, int32_t n, int32_t c, int32_t h, int32_t w,
                 omt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* OMT_B200_H */
