/*
 * vtlb.h -- C ABI of libvtlb200.so: the B200 (sm_100a) device layer for the
 * dense-contraction hot path of vlang/vtl.
 *
 * This is the boundary a V build of vtl binds with `fn C.vtlb_*` declarations in
 * `*_d_b200.v` files.  It takes the place of the calls vtl makes today into the
 * VSL CUDA wrappers; each entry point names the reference interface it replaces
 * (paths inside vlang/vtl).
 *
 * Conventions
 *  - every function returns 0 (VTLB_OK) or a negative VTLB_E* code and never
 *    throws or aborts; vtlb_last_error(ctx) gives the message of the last failure;
 *  - one vtlb_ctx per GPU; calls on one ctx are issued from one thread at a time
 *    (the reference is single-threaded) and are ordered on the ctx's stream;
 *    they are asynchronous unless stated, vtlb_sync() and vtlb_d2h() block;
 *  - `const void* d_*` / `void* d_*` arguments are DEVICE pointers obtained from
 *    vtlb_alloc (offsets into such allocations are fine, 16-byte aligned);
 *    `h_*` arguments are HOST pointers borrowed for the duration of the call;
 *  - matrices are dense row-major with the stated shape; there is no CPU
 *    fallback anywhere: without a usable GPU every call fails with VTLB_ECUDA.
 */
#ifndef VTLB_H
#define VTLB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VTLB_OK 0
#define VTLB_EINVAL (-1)   /* bad argument (shape, alignment, null pointer) */
#define VTLB_ECUDA (-2)    /* a CUDA runtime/driver call failed */
#define VTLB_ENOMEM (-3)   /* device allocation failed */
#define VTLB_ETIMEOUT (-4) /* a bounded device-side wait gave up; see vtlb_check_status */
#define VTLB_ENCCL (-5)    /* NCCL missing or a collective failed */
#define VTLB_ESTATE (-6)   /* call not valid in the ctx's current state */

typedef struct vtlb_ctx vtlb_ctx;

/* ---- context ------------------------------------------------------------
 * Replaces: cuda.get_default_device()/cuda.get_device(id) as used by
 * storage/cuda_d_cuda.v:32-47 and DeviceSession.init_device
 * (autograd_cuda/device_session_d_cuda.v:9-15); the session pointer kept in
 * Context.device_session (autograd/context.v:23). */
int vtlb_device_count(int* count);
int vtlb_ctx_create(int device, vtlb_ctx** out);
int vtlb_ctx_destroy(vtlb_ctx* ctx);
int vtlb_sync(vtlb_ctx* ctx);
const char* vtlb_last_error(vtlb_ctx* ctx); /* ctx may be NULL: process-wide last error */
/* Reads and clears the device status word written by kernels whose bounded
 * waits ran out (0 = none).  Blocks until the stream is idle. */
int vtlb_check_status(vtlb_ctx* ctx, uint32_t* status);
/* Self-test of the bounded device-side waits (no counterpart in the reference, whose GPU calls
 * block on the default stream): launches a one-CTA kernel that waits on an mbarrier for at most
 * limit_ns (1 ns .. 100 ms) with the same wait routine as the tcgen05 kernels.  arrive != 0: a
 * second thread arrives and the wait is satisfied.  arrive == 0: nobody arrives, the wait gives
 * up, the kernel returns normally and sets the status word, so the next vtlb_check_status
 * returns VTLB_ETIMEOUT -- the failure path of a stuck pipeline, without anything being stuck. */
int vtlb_wait_probe(vtlb_ctx* ctx, uint64_t limit_ns, int arrive);
/* Number of kernels this library launched on ctx since creation. */
uint64_t vtlb_launch_count(vtlb_ctx* ctx);
/* cudaStream_t of the ctx (as void*), for callers that time with CUDA events. */
void* vtlb_stream(vtlb_ctx* ctx);

/* Device-side timing with CUDA events on the ctx's compute stream (measurement
 * helper; no counterpart in the reference, which times with time.ticks()). */
int vtlb_event_create(vtlb_ctx* ctx, void** ev_out);
int vtlb_event_record(vtlb_ctx* ctx, void* ev);
int vtlb_event_elapsed_ms(vtlb_ctx* ctx, void* ev_start, void* ev_stop, float* ms); /* blocks */
int vtlb_event_destroy(vtlb_ctx* ctx, void* ev);

/* Optional timing of the tensor-core GEMM launches alone (measurement helper, off by
 * default): while enabled, a CUDA event pair brackets each of the next 2048 GEMM launches on
 * the compute stream; _read blocks, returns their summed duration, their count and their
 * algorithmic work (2*M*N*K each) and resets the counters. */
int vtlb_profile_gemm(vtlb_ctx* ctx, int enable);
int vtlb_profile_gemm_read(vtlb_ctx* ctx, double* total_ms, uint64_t* launches, double* total_ops);
/* While vtlb_profile_gemm is enabled the same ring of event pairs also brackets the other phases
 * of a training step, so that a step's time can be broken down: summed duration and number of
 * spans of one phase since the last vtlb_profile_gemm_read (call this first; _gemm_read resets).
 * VTLB_PHASE_COMM_WAIT is the time the compute stream stood idle in vtlb_comm_wait until the
 * collectives on the communication stream had finished: the exposed, not-overlapped part. */
enum {
  VTLB_PHASE_GEMM = 0,       /* tensor-core GEMM / convolution launches */
  VTLB_PHASE_SPLIT = 1,      /* f32 -> TF32 hi/lo operand planes */
  VTLB_PHASE_OPTIMIZER = 2,  /* Adam / AdamW / SGD / RMSProp step */
  VTLB_PHASE_COMM_WAIT = 3,  /* compute stream waiting for collectives */
  VTLB_PHASE_ELEMENTWISE = 4,/* ReLU backward, bias-gradient column sums, loss kernels */
  VTLB_PHASE_COUNT = 5
};
int vtlb_profile_read_phase(vtlb_ctx* ctx, int phase, double* total_ms, uint64_t* spans);

/* ---- memory ---------------------------------------------------------------
 * Replaces: CpuStorage.cuda()/CudaStorage.cpu()/to_array()/release()
 * (storage/cuda_d_cuda.v:32-107), the raw C.cudaMalloc/cudaMemcpy/cudaFree of
 * autograd_cuda/device_session_gpu_d_cuda.v:24-45,118-152 and
 * compute.GpuBufF64{ensure,upload,download,release}
 * (autograd_cuda/device_session_optimizer_d_cuda.v:7-59).
 * vtlb_alloc / vtlb_free are ordered on the context's compute stream (a freed block may be handed
 * to the next vtlb_alloc at once: whatever is enqueued for the new owner runs after everything that
 * was enqueued for the old one).  Blocks come from the device's stream-ordered pool; blocks of up to
 * 1 MiB are additionally recycled by the context itself (up to 256 MiB of them), because a pool call
 * per small tensor costs more host time than a small kernel takes to run. */
int vtlb_alloc(vtlb_ctx* ctx, size_t bytes, void** d_out);
int vtlb_free(vtlb_ctx* ctx, void* d_ptr);
int vtlb_h2d(vtlb_ctx* ctx, void* d_dst, const void* h_src, size_t bytes);
int vtlb_d2h(vtlb_ctx* ctx, void* h_dst, const void* d_src, size_t bytes); /* blocks */
int vtlb_d2d(vtlb_ctx* ctx, void* d_dst, const void* d_src, size_t bytes);
int vtlb_memset0(vtlb_ctx* ctx, void* d_dst, size_t bytes);
/* Pinned host staging memory for fast h2d/d2h (optional; any host memory works). */
int vtlb_host_alloc(size_t bytes, void** h_out);
int vtlb_host_free(void* h_ptr);
/* Grows the ctx's internal scratch (operand-split buffers, partial sums) to at
 * least `bytes` ahead of time, so that later calls allocate nothing. */
int vtlb_reserve_scratch(vtlb_ctx* ctx, size_t bytes);

/* ---- f32 GEMM -------------------------------------------------------------
 * C[M,N] = op(A).op(B) (+ bias[N]) (ReLU).  op(A) is [M,K]: A is [M,K] row-major
 * when transA == 0, [K,M] when transA != 0; likewise B is [K,N] or, with transB,
 * [N,K].  Computed on tcgen05 tensor cores as a 3-pass TF32 split (hi.hi +
 * hi.lo + lo.hi) with f32 accumulation in tensor memory.
 * Replaces: la.matmul[f32] (la/la.v:38-55), gate_matmul
 * (autograd/gates_blas.v:6-23), compute.gemm_cuda as called from
 * autograd_cuda/device_session_d_cuda.v:43 and tensor_cuda_d_cuda.v:169, and
 * C.cublasDgemm_v2 (autograd_cuda/device_session_gpu_d_cuda.v:143). */
int vtlb_gemm_f32(vtlb_ctx* ctx, int transA, int transB, int M, int N, int K, const void* d_A,
                  const void* d_B, void* d_C, const void* d_bias_or_null, int relu);

/* f32 products of at most `max_flops` (2*M*N*K) run as one FFMA kernel on CUDA cores straight
 * from the caller's operands instead of the tensor-core path: at the size of a 784->256->10
 * MLP on a batch of 64 the call is bound by launch latency, not arithmetic.  Default 1.4e8;
 * 0 sends every product to the tensor cores.  Both paths meet the same error bound. */
int vtlb_set_small_gemm_limit(vtlb_ctx* ctx, double max_flops);

/* ---- Linear layer ---------------------------------------------------------
 * Y[M,N] = X[M,K].W[N,K]^T + b[N]; with relu != 0, Y = relu(.) and, when
 * d_pre_or_null is given, the pre-activation is stored there as well (it is
 * the cache the ReLU gate needs).
 * Replaces: linear_forward_f32 (nn/layers/linear_forward_f32.v:7-18),
 * DeviceSession.linear_forward_f64 (autograd_cuda/device_session_d_cuda.v:17-57)
 * and linear_forward_gpu_chain (device_session_gpu_d_cuda.v:88-181). */
int vtlb_linear_fwd_f32(vtlb_ctx* ctx, const void* d_X, const void* d_W, const void* d_b_or_null,
                        void* d_Y, int M, int N, int K, int relu, void* d_pre_or_null);
/* dX[M,K] = G.W, dW[N,K] = G^T.X, db[N] = column sums of G; any of the three
 * outputs may be NULL.  Outputs are overwritten (the first accumulation onto a
 * zero gradient in Variable.backprop, autograd/variable.v:105).
 * Replaces: LinearGate.backward (nn/gates/layers/linear.v:25-95),
 * linear_backward_f64 (autograd_cuda/linear_backward_cuda_d_cuda.v:9-34),
 * linear_gate_backward_f32_try (nn/gates/layers/linear_gate_backward_f32_try_*.v:6). */
int vtlb_linear_bwd_f32(vtlb_ctx* ctx, const void* d_G, const void* d_X, const void* d_W,
                        void* d_dX_or_null, void* d_dW_or_null, void* d_db_or_null, int M, int N,
                        int K);

/* ---- the same two calls, with the operand planes handed from producer to consumer -----
 * The f32 products run as three TF32 MMAs on hi/lo planes of their operands (x = hi + lo).
 * vtlb_linear_fwd_f32 / _bwd_f32 write those planes in a pass of their own before every
 * product; in a deep network the same activation and gradient matrices are split again and
 * again (each is an operand of up to three products).  Here the GEMM that PRODUCES a matrix
 * also leaves its planes, from its epilogue, in the two layouts the consuming products read:
 *   "rows" planes of a matrix T[R,C]:  hi, lo as [R, vtlb_plane_ld(C)]   (T as the K-major operand)
 *   "cols" planes:                     hi, lo as [C, vtlb_plane_ld(R)]   (T transposed)
 * Each vtlb_planes names two caller-allocated f32 arrays of that size (16-byte aligned; the
 * padding columns are never read).  Every planes argument may be NULL: an input that is NULL is
 * split by the call as before, an output that is NULL is not produced.  Results are the same bit
 * for bit with or without planes.  No counterpart in the reference (its products run in f64 on
 * the host BLAS, la/la.v:38-55).
 *
 * forward:  x_rows = planes of X [M,K] (in); y_rows / y_cols = planes of Y [M,N] and of Y
 *           transposed (out; of the activated output when relu != 0).
 * backward: g_rows / g_cols = planes of G [M,N] and G transposed, x_cols = planes of X
 *           transposed (in).  d_relu_mask_src (the pre-activation [M,K] cached by the ReLU below
 *           this layer, nn/gates/activation/relu.v:21-25) applies that ReLU's backward to dX on
 *           the way out: dX = src < 0 ? 0 : dX.  dx_rows / dx_cols = planes of the (masked) dX
 *           and its transpose (out): the G planes of the layer below.
 * vtlb_f32_planes_worthwhile: 0 for products small enough to run on the CUDA-core route, which
 * reads no planes (callers then skip allocating them).  vtlb_split_planes_f32 writes the planes
 * of a matrix nobody produced through these calls (the network input, the loss gradient). */
typedef struct vtlb_planes {
  void* hi;
  void* lo;
} vtlb_planes;
int vtlb_plane_ld(int kdim);
int vtlb_f32_planes_worthwhile(vtlb_ctx* ctx, int M, int N, int K);
int vtlb_split_planes_f32(vtlb_ctx* ctx, const void* d_src, int R, int C, const vtlb_planes* rows_or_null,
                          const vtlb_planes* cols_or_null);
int vtlb_linear_fwd_f32_planes(vtlb_ctx* ctx, const void* d_X, const void* d_W, const void* d_b_or_null,
                               void* d_Y, int M, int N, int K, int relu, void* d_pre_or_null,
                               const vtlb_planes* x_rows_or_null, const vtlb_planes* y_rows_or_null,
                               const vtlb_planes* y_cols_or_null);
int vtlb_linear_bwd_f32_planes(vtlb_ctx* ctx, const void* d_G, const void* d_X, const void* d_W,
                               void* d_dX_or_null, void* d_dW_or_null, void* d_db_or_null, int M, int N,
                               int K, const vtlb_planes* g_rows_or_null, const vtlb_planes* g_cols_or_null,
                               const vtlb_planes* x_cols_or_null, const void* d_relu_mask_src_or_null,
                               const vtlb_planes* dx_rows_or_null, const vtlb_planes* dx_cols_or_null);

/* db[N] = column sums of G[M,N] (the bias gradient of vtlb_linear_bwd_f32) for callers
 * that cannot let the library allocate device memory: a host that has already given all of
 * HBM to its own pools, or a loop whose latency budget an allocation's implicit
 * synchronisation would break.  No counterpart in the reference.  The partial sums live in
 * a fixed 2 MiB array inside the library image (held on every GPU that loads the library
 * until exit) instead of the ctx scratch, so the call never allocates; the limit is
 * N <= 4096 columns (any M), larger N is refused with VTLB_EINVAL.  The first call on a
 * device looks up the array's device address: make that call before any stream capture.
 * All calls on a GPU share the one array (each call overwrites what it reads, nothing is
 * carried over), so calls that overlap on the same GPU - two contexts, two streams - race;
 * issue them one after the other. */
int vtlb_bias_grad_f32_noalloc(vtlb_ctx* ctx, const void* d_G, int M, int N, void* d_db);

/* ---- ReLU -----------------------------------------------------------------
 * y = x < 0 ? 0 : x;   dx = cached_x < 0 ? 0 : g   (gradient passes at exactly 0).
 * Replaces: relu_forward_f32_try (nn/layers/activation_relu_forward_f32_try_*.v:6),
 * compute.relu_cuda (tensor_cuda_d_cuda.v:208), internal.relu / deriv_relu
 * (nn/internal/activation.v:63-87). */
int vtlb_relu_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, size_t n);
int vtlb_relu_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_cached_x, void* d_dx, size_t n);

/* dst += src (Variable.backprop's parent.grad.add(diff), autograd/variable.v:105) and
 * dst[i] = value (ones_like for the backprop seed, autograd/variable.v:88). */
int vtlb_add_inplace_f32(vtlb_ctx* ctx, void* d_dst, const void* d_src, size_t n);
int vtlb_fill_f32(vtlb_ctx* ctx, void* d_dst, float value, size_t n);

/* ---- parameter initialisers ---------------------------------------------------
 * Random fills behind kaiming_uniform / kaiming_normal / variance_scaled
 * (nn/internal/init.v:35-70), which call vtl.random(-limit, limit, shape) and
 * vtl.normal(shape, mu, sigma) (rand.v:57-79).  The reference's generator is V's global
 * one, seeded from the wall clock; here element i is a pure function of (seed, i):
 *   z = splitmix64(seed + (i+1)*0x9E3779B97F4A7C15)
 *   uniform: u = (z >> 40) * 2^-24;  x = lo + u*(hi - lo)      (f32, two roundings; x in [lo, hi))
 *   normal : Box-Muller in f64 on u1 = ((z>>32)+1)*2^-32, u2 = (z & 0xffffffff)*2^-32,
 *            x = (f32)(mu + sigma*sqrt(-2 ln u1)*cos(2 pi u2))
 * so fills are reproducible and independent of the launch geometry. */
int vtlb_init_uniform_f32(vtlb_ctx* ctx, void* d_out, size_t n, float lo, float hi, uint64_t seed);
int vtlb_init_normal_f32(vtlb_ctx* ctx, void* d_out, size_t n, double mu, double sigma, uint64_t seed);

/* ---- Conv2D / max pooling (NCHW, groups = 1) ------------------------------------
 * y[B,O,OH,OW] = conv(x[B,C,H,W], w[O,C,kh,kw]) + bias[O], OH = (H+2ph-kh)/sh+1; with
 * relu != 0 the output is activated and d_pre_or_null receives the pre-activation.
 * Lowered to the 3xTF32 tcgen05 GEMM with K = C*kh*kw in (ic,kh,kw) order.
 * Backward: d_input, d_weight[O,C,kh,kw], d_bias[O]; any output may be NULL.
 * Replaces: conv2d_forward_f32 / conv2d_backward_f32 (nn/internal/conv2d_forward_f32.v:6,
 * conv2d_backward_f32.v:6, CPU loops conv2d_forward_cpu_f32.v:26-62,
 * conv2d_backward_cpu_f32.v:26-97) and compute.conv2d_cuda / conv2d_backward_cuda
 * (nn/internal/conv2d_cuda_d_cuda.v:28-71, conv2d_backward_cuda_d_cuda.v:9-46). */
int vtlb_conv2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, const void* d_w, const void* d_bias_or_null,
                        void* d_y, int B, int C, int H, int W, int O, int kh, int kw, int ph, int pw,
                        int sh, int sw, int relu, void* d_pre_or_null);
int vtlb_conv2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_x, const void* d_w,
                        void* d_dx_or_null, void* d_dw_or_null, void* d_db_or_null, int B, int C, int H,
                        int W, int O, int kh, int kw, int ph, int pw, int sh, int sw);
/* The same with a dilated window (Conv2DConfig.dilation, nn/layers/conv2d.v:15-21): taps at
 * ih = oh*sh - ph + a*dh, iw = ow*sw - pw + b*dw, OH = (H + 2ph - dh(kh-1) - 1)/sh + 1
 * (conv2d_forward_cpu_f32.v:26-62, conv2d_backward_cpu_f32.v:19,39,65).  dh = dw = 1 is the call
 * above; other dilations run on the lowered route (patch matrix + GEMM). */
int vtlb_conv2d_fwd_f32_dilated(vtlb_ctx* ctx, const void* d_x, const void* d_w, const void* d_bias_or_null,
                                void* d_y, int B, int C, int H, int W, int O, int kh, int kw, int ph, int pw,
                                int sh, int sw, int dh, int dw, int relu, void* d_pre_or_null);
int vtlb_conv2d_bwd_f32_dilated(vtlb_ctx* ctx, const void* d_g, const void* d_x, const void* d_w,
                                void* d_dx_or_null, void* d_dw_or_null, void* d_db_or_null, int B, int C, int H,
                                int W, int O, int kh, int kw, int ph, int pw, int sh, int sw, int dh, int dw);
/* 2-D max pooling with the window geometry of internal.maxpool2d
 * (nn/internal/layers.v:21-66); the first maximum in scan order wins; d_idx (int32) holds
 * the flat index into the whole input.  Backward scatters g onto zeros (layers.v:69-84). */
int vtlb_maxpool2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, void* d_idx, int B, int C, int H,
                           int W, int kh, int kw, int ph, int pw, int sh, int sw);
int vtlb_maxpool2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_idx, void* d_dx, size_t n_out,
                           size_t n_in);
/* The same backward for the 2x2 window with stride 2 and no padding (H % 2 = 0, W % 4 = 0, 16-byte
 * aligned pointers): the windows tile the input, so dX is written directly, without the zero fill
 * and the scatter.  d_relu_cache_or_null = the pre-activation cached by a ReLU whose output the pool
 * read (shaped like dX): when given, that ReLU's backward (nn/internal/activation.v:78-87: zero
 * where the cached value is < 0) is applied in the same pass, and the result is the gradient of the
 * ReLU's input. */
int vtlb_maxpool2x2_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_idx, const void* d_relu_cache_or_null,
                            void* d_dx, int B, int C, int H, int W);

/* ---- losses ---------------------------------------------------------------
 * MSE as the reference computes it: loss = sum((p-t)^2)/n, dP = (p - t) * g with
 * no 2/n factor (nn/internal/activation.v:365-373, nn/internal/loss.v:7-12).
 * d_loss receives one f32 (`loss_scale` multiplies it: pass 1, or 1/ranks ... as
 * needed by the caller); d_dP may be NULL.  `n_div` is the divisor n (the global
 * element count when rows are sharded over ranks). */
int vtlb_mse_fwd_bwd_f32(vtlb_ctx* ctx, const void* d_P, const void* d_T, size_t n, size_t n_div,
                         void* d_loss, void* d_dP_or_null);
/* Softmax cross-entropy over rows of X[B,C] against targets T[B,C]
 * (nn/internal/activation.v:392-420, nn/internal/loss.v:39-65): f64 inside,
 * loss = sum_i(lse_i - t_i.x_i)/batch_div, dX = (softmax - t)/batch_div. */
int vtlb_softmax_ce_fwd_bwd_f32(vtlb_ctx* ctx, const void* d_X, const void* d_T, int B, int C,
                                int batch_div, void* d_loss, void* d_dX_or_null);

/* ---- Adam / AdamW ---------------------------------------------------------
 * One fused multi-tensor launch per call.  Scalars are the f64 values of
 * AdamStepParams (nn/optimizers/adam_step_f64.v:6-12); lr_t is computed by the
 * caller as AdamOptimizer.update does (nn/optimizers/adam.v:88-91).
 * zero_grad != 0 also clears the gradients (adam.v:142).
 * Adam  : f32 arithmetic of adam_step_f32_cpu (nn/optimizers/adam_step_f32.v:6-21).
 * AdamW : f64 arithmetic on f32 state of AdamWOptimizer.update (adamw.v:84-104).
 * Replaces: adam_update_f64_cuda / adam_step_f64 and their 14 BLAS-1 launches
 * (nn/optimizers/adam_f64_d_cuda.v:8-20, adam_step_cuda_d_cuda.v:8-121),
 * try_adam_update_f32_vulkan (adam_f32_vulkan_d_vulkan.v:23). */
typedef struct vtlb_adam_tensor {
  void* d_grad;
  void* d_theta;
  void* d_m;
  void* d_v;
  size_t n;
} vtlb_adam_tensor;
int vtlb_adam_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors, double beta1,
                       double beta2, double lr_t, double epsilon, int zero_grad);
int vtlb_adamw_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors,
                        double beta1, double beta2, double lr_t, double epsilon,
                        double weight_decay, int zero_grad);
/* SGD  : theta -= (f32)lr * g in f32 (internal.sgd_optimize, nn/internal/optimizers.v:6-13, called
 *        by SgdOptimizer.update, nn/optimizers/sgd.v:45-52); d_m and d_v of the tensors are unused.
 * RMSProp: sq = alpha*sq + (1-alpha)*g*g; theta -= lr*(g/(sqrt(sq)+eps) + wd*theta), each element in
 *        f64 and rounded to f32, the update reading the stored sq (RMSPropOptimizer.update,
 *        nn/optimizers/rmsprop.v:70-91); d_v holds sq_avg, d_m is unused. */
int vtlb_sgd_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors, double learning_rate,
                      int zero_grad);
int vtlb_rmsprop_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors, double learning_rate,
                          double alpha, double epsilon, double weight_decay, int zero_grad);

/* ---- INT8 quantised linear ------------------------------------------------
 * No counterpart in the reference (it has no quantisation code); defined here:
 *   amax_r = max_k |a_rk|;  inv = amax_r > 0 ? 127/amax_r : 0;
 *   q_rk = clamp(rint(a_rk * inv), -127, 127);  scale_r = amax_r / 127     (all f32)
 * Code matrices are row-major int8 with leading dimension vtlb_i8_ld(K)
 * (K rounded up to a multiple of 16; the padding bytes are never read).
 * vtlb_quant_rows_i8 serves activations (rows of A[M,K]) and weights (rows of
 * W[N,K], i.e. output channels).  With d_amax_in_or_null the row maxima are
 * taken from there instead of being computed (column-sharded layers). */
int vtlb_i8_ld(int K);
int vtlb_quant_rows_i8(vtlb_ctx* ctx, const void* d_A, int M, int K, void* d_Q, void* d_scale,
                       const void* d_amax_in_or_null);
int vtlb_row_absmax_f32(vtlb_ctx* ctx, const void* d_A, int M, int K, void* d_amax);
/* acc[M,N] (int32) = Aq[M,K].Wq[N,K]^T, exact.  The kernel follows the shape, the result does
 * not: one row of activations streams W through dp4a; up to 128 rows run on tcgen05 kind::i8
 * with the output channels on the M side of the MMA and K cut across a thread-block cluster;
 * larger products run as 128-row tiles, on CTA pairs (cta_group::2) when there are enough. */
int vtlb_gemm_i8_i32(vtlb_ctx* ctx, const void* d_Aq, const void* d_Wq, int M, int N, int K,
                     void* d_acc);
/* Y[M,N] = relu?( (float)acc * (sa[m]*sw[n]) + bias[n] ), the dequantisation
 * fused into the GEMM epilogue; every f32 operation rounds on its own. */
int vtlb_linear_i8_fwd(vtlb_ctx* ctx, const void* d_Aq, const void* d_sa, const void* d_Wq,
                       const void* d_sw, const void* d_bias_or_null, void* d_Y, int M, int N,
                       int K, int relu);

/* Same as vtlb_linear_i8_fwd with the activation codes stored as `shards` column shards one
 * after another: shard s is a dense [M, K/shards] int8 matrix holding columns
 * [s*K/shards, (s+1)*K/shards) - the layout an all-gather of per-rank column slabs of the
 * previous layer leaves behind, read in place through a 3-D tensor map (no re-layout pass).
 * K/shards must be a multiple of 128.  Used by output-column-sharded INT8 inference. */
int vtlb_linear_i8_fwd_sharded_a(vtlb_ctx* ctx, const void* d_Aq_shards, int shards, const void* d_sa,
                                 const void* d_Wq, const void* d_sw, const void* d_bias_or_null,
                                 void* d_Y, int M, int N, int K, int relu);
/* The same (shards >= 1) with the row maxima of |Y| written to d_row_amax[M] by the GEMM's epilogue:
 * what vtlb_row_absmax_f32 would compute from Y, without reading Y again - the next layer's dynamic
 * quantisation (vtlb_quant_rows_i8 with d_amax_in) can start from it.  The maxima are exact (a
 * maximum does not depend on the order it is taken in). */
int vtlb_linear_i8_fwd_amax(vtlb_ctx* ctx, const void* d_Aq_shards, int shards, const void* d_sa,
                            const void* d_Wq, const void* d_sw, const void* d_bias_or_null, void* d_Y,
                            int M, int N, int K, int relu, void* d_row_amax);

/* ---- layers next to the GEMMs -------------------------------------------------
 * Softmax over the last dimension of x[rows, n]: forward in f64 (max, exp(x - max), sum in
 * order, divide; internal.softmax_forward, nn/internal/activation.v:423-457); backward
 * dx_k = s_k (g_k - sum_i g_i s_i) with the softmax recomputed from the cached INPUT in f32
 * (deriv_softmax, :285-332).
 * Average pooling (NCHW): window sum of the in-bounds taps / (kh*kw) in f64
 * (internal.avgpool2d_forward, nn/internal/pool.v:6-45); the backward hands g/(kh*kw) to every
 * tap (the reference's :48-59 returns zeros of the wrong shape; standard rule instead); global
 * average pooling as :62-101.
 * BatchNorm1D on x[B, F]: train = batch mean and biased variance per feature in f64,
 * y = gamma*(x-mean)/sqrt(var+eps)+beta, the f32-rounded statistics returned and blended into
 * the running ones with `momentum` (internal.batchnorm1d_training, nn/internal/batchnorm.v:27-70;
 * nn/layers/batchnorm.v:84-97; running pointers may both be null); infer = the f32 path on the
 * running statistics (:7-24); bwd = the reference's formulas as written (:73-140):
 * dx = gamma*(g - mean_B(g))/std, dgamma = sum g*(x-mean)/std, dbeta = sum g. */
int vtlb_softmax_fwd_f32(vtlb_ctx* ctx, const void* d_x, size_t rows, size_t n, void* d_y);
int vtlb_softmax_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_x, size_t rows, size_t n, void* d_dx);
int vtlb_avgpool2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, int B, int C, int H, int W, int kh, int kw,
                           int ph, int pw, int sh, int sw);
int vtlb_avgpool2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, void* d_dx, int B, int C, int H, int W, int kh, int kw,
                           int ph, int pw, int sh, int sw);
int vtlb_global_avgpool2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, int B, int C, int H, int W);
int vtlb_global_avgpool2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, void* d_dx, int B, int C, int H, int W);
int vtlb_batchnorm1d_train_f32(vtlb_ctx* ctx, const void* d_x, int B, int F, const void* d_gamma, const void* d_beta,
                               double eps, void* d_y, void* d_batch_mean, void* d_batch_var,
                               void* d_running_mean_or_null, void* d_running_var_or_null, double momentum);
int vtlb_batchnorm1d_infer_f32(vtlb_ctx* ctx, const void* d_x, int B, int F, const void* d_gamma, const void* d_beta,
                               const void* d_running_mean, const void* d_running_var, double eps, void* d_y);
int vtlb_batchnorm1d_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_x, int B, int F, const void* d_gamma,
                             const void* d_batch_mean, const void* d_batch_var, double eps, void* d_dx_or_null,
                             void* d_dgamma_or_null, void* d_dbeta_or_null);

/* ---- input pipeline: copies that overlap the compute stream -------------------
 * The reference stages every batch through the host synchronously (cuda_memcpy_host_to_device
 * in storage/cuda_d_cuda.v:32-60 and GpuBufF64.upload, then a blocking download); its loader
 * (datasets/dataloader.v:87-143) builds one batch at a time.  Here the next batch comes in and
 * the last result goes out on copy streams of their own while the current step computes.
 *   vtlb_copy_h2d_async  starts after the compute work enqueued so far (the last reader of
 *                        d_dst) and returns at once; h_src should come from vtlb_host_alloc.
 *   vtlb_copy_d2h_async  starts after the compute work enqueued so far (the producer of d_src).
 *   vtlb_copy_wait       VTLB_COPY_IN_BEFORE_COMPUTE: compute enqueued from now on waits for the
 *                        host->device copies enqueued so far; VTLB_COPY_OUT_BEFORE_COMPUTE: ...
 *                        for the device->host copies (before their source is overwritten);
 *                        VTLB_COPY_OUT_DONE: the host blocks until the device->host copies have
 *                        landed.  Bits may be combined.
 * A double-buffered loop: copy batch 0 in; for each step i: wait(IN_BEFORE_COMPUTE); start the
 * copy of batch i+1 into the other buffer; run step i; copy its result out.  vtlb_sync also waits
 * for both copy streams.  vtlb_free orders a block after the compute (and collective) work
 * enqueued so far, not after copies still running on the copy streams: call vtlb_copy_wait with
 * the matching BEFORE_COMPUTE bit before freeing a buffer such a copy reads or writes. */
#define VTLB_COPY_IN_BEFORE_COMPUTE 1
#define VTLB_COPY_OUT_BEFORE_COMPUTE 2
#define VTLB_COPY_OUT_DONE 4
int vtlb_copy_h2d_async(vtlb_ctx* ctx, void* d_dst, const void* h_src, size_t bytes);
int vtlb_copy_d2h_async(vtlb_ctx* ctx, void* h_dst, const void* d_src, size_t bytes);
int vtlb_copy_wait(vtlb_ctx* ctx, int what);

/* ---- batch assembly for a device-resident dataset ---------------------------
 * vtlb_gather_rows_f32: dst[j, :] = src[indices[j], :] for j < n_rows, rows of row_elems values:
 * what DataLoader.batch / batch_with_labels do element by element on the host
 * (datasets/dataloader.v:41-143).  vtlb_one_hot_f32: out[i, c] = (labels[i] == c), the
 * [N, classes] label tensor the reference's examples build on the host.  An index or label out
 * of range is never dereferenced / leaves a zero row; with check != 0 the call blocks and
 * reports it as VTLB_EINVAL. */
int vtlb_gather_rows_f32(vtlb_ctx* ctx, const void* d_src, int src_rows, size_t row_elems,
                         const void* d_indices_i32, int n_rows, void* d_dst, int check);
int vtlb_one_hot_f32(vtlb_ctx* ctx, const void* d_labels_i32, size_t n, int classes, void* d_out, int check);

/* ---- checkpoint tensor payloads --------------------------------------------
 * The reference writes every tensor of a checkpoint as text: each element widened to f64, its
 * 8 bytes most significant first, the bytes in standard base64 with '=' padding
 * (encode_tensor / decode_tensor, nn/models/serialization.v:421-473; callers save_checkpoint
 * :109-262 and load_weights :279-373).  These two run that byte work on the device, so that only
 * the text crosses to the host: vtlb_ckpt_text_len(n) = 4*ceil(8n/3) characters for n elements.
 * d_text must be 16-byte aligned.  decode converts f64 -> f32 by plain rounding (vtl.cast),
 * refuses a length that does not match n, characters outside the alphabet and malformed
 * padding (VTLB_EINVAL), and blocks until the result is known; encode returns at once. */
size_t vtlb_ckpt_text_len(size_t n);
int vtlb_ckpt_encode_f32(vtlb_ctx* ctx, const void* d_src, size_t n, void* d_text);
int vtlb_ckpt_decode_f32(vtlb_ctx* ctx, const void* d_text, size_t text_len, void* d_dst, size_t n);

/* Measurement helper (no counterpart in the reference): the rate at which this GPU's tensor cores
 * execute INT8 MMAs when nothing has to be loaded -- every CTA pair issues 4 * mma_groups
 * tcgen05.mma.kind::i8 instructions (256 x 256 x 32) on operands resident in shared memory.  The
 * ceiling of any INT8 GEMM at the clocks of the moment, in TOPS; launches two kernels and blocks. */
int vtlb_int8_issue_yardstick(vtlb_ctx* ctx, int mma_groups, double* tops_out);

/* ---- collectives (NCCL over NVLink) ---------------------------------------
 * No counterpart in the reference (single device).  One ctx per rank/process.
 * vtlb_comm_unique_id fills a 128-byte id on one rank; the caller ships it to
 * the others (any host channel) and every rank calls vtlb_comm_init_rank. */
int vtlb_comm_unique_id(void* h_id128);
int vtlb_comm_init_rank(vtlb_ctx* ctx, int nranks, int rank, const void* h_id128);
int vtlb_comm_destroy(vtlb_ctx* ctx);
/* In-place sum over ranks, enqueued on the ctx's communication stream after the
 * work already enqueued on the compute stream; returns at once. */
int vtlb_allreduce_sum_f32_async(vtlb_ctx* ctx, void* d_buf, size_t n);
int vtlb_allreduce_max_f32_async(vtlb_ctx* ctx, void* d_buf, size_t n);
int vtlb_allgather_async(vtlb_ctx* ctx, const void* d_send, void* d_recv, size_t bytes_per_rank);
/* Gives the small collectives of this communicator (vtlb_allreduce_max_f32_async) a communicator and
 * stream of their own, VTLB_COMM_LANE_SMALL; collective, every rank calls it once after
 * vtlb_comm_init_rank.  Without it both lanes are the same stream.  No counterpart in the reference. */
int vtlb_comm_small_lane(vtlb_ctx* ctx);
/* All-gather by the copy engines instead of an NCCL kernel (which occupies 16-32 SMs and slows a
 * persistent GEMM running beside it far more than its share).  Every rank allocates its receive
 * buffer with vtlb_shared_alloc (a plain device allocation plus its 64-byte CUDA IPC handle), ships
 * the handle to the other ranks' processes over any host channel, and opens theirs with
 * vtlb_shared_open.  vtlb_allgather_push_async then copies `bytes` from d_src into every non-null
 * d_peer_dst[r] (the address of this rank's part inside rank r's buffer) on the bulk lane, after the
 * compute work enqueued so far, and appends an all-reduce of one word: once that has completed on a
 * rank (vtlb_comm_mark / vtlb_comm_wait_mark / vtlb_comm_wait) every rank's part has landed in its
 * buffer.  The caller writes its own part itself.  A part may be pushed into a peer's buffer again
 * only after a later collective of this communicator has completed behind the peer's last read of
 * it (the one-word all-reduce of any later push does).  At the end every process closes the buffers
 * it opened (vtlb_shared_close), and only when all have done so does the owner free its own
 * (vtlb_shared_free): an exported buffer must not be freed while another process has it mapped.
 * No counterpart in the reference. */
int vtlb_shared_alloc(vtlb_ctx* ctx, size_t bytes, void** d_out, void* h_handle64);
int vtlb_shared_free(vtlb_ctx* ctx, void* d_ptr);
int vtlb_shared_open(vtlb_ctx* ctx, const void* h_handle64, void** d_peer_out);
int vtlb_shared_close(vtlb_ctx* ctx, void* d_peer);
int vtlb_allgather_push_async(vtlb_ctx* ctx, const void* d_src, void* const* d_peer_dst, int npeers, size_t bytes);
/* Makes the compute stream wait for every collective enqueued so far. */
int vtlb_comm_wait(vtlb_ctx* ctx);
/* Waiting for ONE collective instead of all of them.  Collectives run on two lanes: the bulk lane
 * (all-gather, sum all-reduce) and the small lane (max all-reduce), which has a communicator and
 * a stream of its own where the NCCL at hand can split communicators, so that a few kilobytes of
 * row maxima do not queue behind hundreds of megabytes of codes.  vtlb_comm_mark records mark
 * `slot` (0..63) behind the collectives enqueued so far on `lane`; vtlb_comm_wait_mark makes the
 * compute stream wait for that mark only.  A slot may be marked again once its wait is enqueued. */
#define VTLB_COMM_LANE_BULK 0
#define VTLB_COMM_LANE_SMALL 1
int vtlb_comm_mark(vtlb_ctx* ctx, int lane, int slot);
int vtlb_comm_wait_mark(vtlb_ctx* ctx, int slot);

#ifdef __cplusplus
}
#endif
#endif /* VTLB_H */
