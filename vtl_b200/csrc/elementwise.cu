// Memory-bound kernels that sit between the GEMMs: ReLU forward/backward and the
// two losses, with the reference's exact element-wise semantics
// (nn/internal/activation.v:63-87, 365-373, 392-420; nn/internal/loss.v:7-12, 39-65).
#include "common.cuh"

namespace {

int ew_grid(vtlb_ctx* ctx, size_t items, int per_block) {
  size_t b = (items + per_block - 1) / per_block;
  size_t cap = (size_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

__device__ __forceinline__ float relu1(float x) { return x < 0.0f ? 0.0f : x; }

__global__ void __launch_bounds__(256) relu_fwd_kernel(const float* __restrict__ x,
                                                       float* __restrict__ y, size_t n, int vec) {
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t done = 0;
  if (vec) {
    const size_t n4 = n / 4;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* y4 = reinterpret_cast<float4*>(y);
    for (size_t i = tid; i < n4; i += stride) {
      float4 v = x4[i];
      y4[i] = make_float4(relu1(v.x), relu1(v.y), relu1(v.z), relu1(v.w));
    }
    done = n4 * 4;
  }
  for (size_t i = done + tid; i < n; i += stride) y[i] = relu1(x[i]);
}

__global__ void __launch_bounds__(256) relu_bwd_kernel(const float* __restrict__ g,
                                                       const float* __restrict__ c,
                                                       float* __restrict__ dx, size_t n, int vec) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a small GEMM behind this kernel may start early
  const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t done = 0;
  if (vec) {
    const size_t n4 = n / 4;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    const float4* c4 = reinterpret_cast<const float4*>(c);
    float4* d4 = reinterpret_cast<float4*>(dx);
    for (size_t i = tid; i < n4; i += stride) {
      float4 gv = g4[i], cv = c4[i];
      d4[i] = make_float4(cv.x < 0.f ? 0.f : gv.x, cv.y < 0.f ? 0.f : gv.y,
                          cv.z < 0.f ? 0.f : gv.z, cv.w < 0.f ? 0.f : gv.w);
    }
    done = n4 * 4;
  }
  for (size_t i = done + tid; i < n; i += stride) dx[i] = c[i] < 0.f ? 0.f : g[i];
}

__global__ void __launch_bounds__(256) add_inplace_kernel(float* __restrict__ dst,
                                                          const float* __restrict__ src, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __fadd_rn(dst[i], src[i]);
}
__global__ void __launch_bounds__(256) fill_kernel(float* __restrict__ dst, float value, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    dst[i] = value;
}

__device__ __forceinline__ double block_sum(double v, double* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  if (threadIdx.x < 32) {
    t = threadIdx.x < (blockDim.x >> 5) ? smem[threadIdx.x] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in thread 0
}

// dP = p - t (the reference's g*(p-t)/g.size with g = [1]); per-block partial sums
// of (f32)((f64)d)^2, accumulated in f64.  The reduction is two-stage and has a
// fixed order, so results are reproducible run to run.
__global__ void __launch_bounds__(256) mse_partial_kernel(const float* __restrict__ p,
                                                          const float* __restrict__ t, size_t n,
                                                          float* __restrict__ dp,
                                                          double* __restrict__ partial) {
  __shared__ double sm[8];
  double acc = 0.0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const float d = __fsub_rn(p[i], t[i]);
    if (dp) dp[i] = d;
    const double dd = (double)d;
    acc += (double)(float)(dd * dd);
  }
  const double s = block_sum(acc, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// Short inputs: one CTA does both stages in a single launch.
__global__ void __launch_bounds__(256) mse_short_kernel(const float* __restrict__ p, const float* __restrict__ t,
                                                        size_t n, double divisor, float* __restrict__ dp,
                                                        float* __restrict__ loss) {
  __shared__ double sm[8];
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a small GEMM behind this kernel may start early
  double acc = 0.0;
  for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
    const float d = __fsub_rn(p[i], t[i]);
    if (dp) dp[i] = d;
    const double dd = (double)d;
    acc += (double)(float)(dd * dd);
  }
  const double s = block_sum(acc, sm);
  if (threadIdx.x == 0) *loss = __fdiv_rn((float)s, (float)divisor);
}

__global__ void __launch_bounds__(256) loss_final_kernel(const double* __restrict__ partial,
                                                         int nparts, double divisor,
                                                         int divide_in_f32,
                                                         float* __restrict__ loss) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ double sm[8];
  double acc = 0.0;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partial[i];
  const double s = block_sum(acc, sm);
  if (threadIdx.x == 0)
    *loss = divide_in_f32 ? __fdiv_rn((float)s, (float)divisor) : (float)(s / divisor);
}

// One thread per row: the class count is small (10 in the configurations this
// serves) and everything is f64, as in the reference.
__global__ void __launch_bounds__(128) softmax_ce_kernel(const float* __restrict__ x,
                                                         const float* __restrict__ t, int B, int C,
                                                         double batch_div, float* __restrict__ dx,
                                                         double* __restrict__ partial) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ double sm[8];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  double li = 0.0;
  if (i < B) {
    const float* xi = x + (size_t)i * C;
    const float* ti = t + (size_t)i * C;
    double mx = (double)xi[0];
    for (int c = 1; c < C; ++c) mx = fmax(mx, (double)xi[c]);
    double se = 0.0;
    for (int c = 0; c < C; ++c) se += exp((double)xi[c] - mx);
    double dot = 0.0;
    for (int c = 0; c < C; ++c) dot += (double)ti[c] * (double)xi[c];
    li = log(se) + mx - dot;
    if (dx)
      for (int c = 0; c < C; ++c) {
        const double smx = exp((double)xi[c] - mx) / se;
        dx[(size_t)i * C + c] = (float)((smx - (double)ti[c]) / batch_div);
      }
  }
  const double s = block_sum(li, sm);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

}  // namespace

VTLB_API int vtlb_add_inplace_f32(vtlb_ctx* ctx, void* d_dst, const void* d_src, size_t n) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_dst || !d_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_add_inplace_f32: null pointer");
  add_inplace_kernel<<<ew_grid(ctx, n, 1024), 256, 0, ctx->stream>>>((float*)d_dst, (const float*)d_src, n);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_fill_f32(vtlb_ctx* ctx, void* d_dst, float value, size_t n) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_dst) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_fill_f32: null pointer");
  fill_kernel<<<ew_grid(ctx, n, 1024), 256, 0, ctx->stream>>>((float*)d_dst, value, n);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_relu_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, size_t n) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_x || !d_y) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_relu_fwd_f32: null pointer");
  const int vec = vtlb_aligned16(d_x) && vtlb_aligned16(d_y);
  relu_fwd_kernel<<<ew_grid(ctx, n, 1024), 256, 0, ctx->stream>>>((const float*)d_x, (float*)d_y, n, vec);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_relu_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_cached_x, void* d_dx,
                               size_t n) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_g || !d_cached_x || !d_dx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_relu_bwd_f32: null pointer");
  vtlb_prof_scope prof(ctx, VTLB_PHASE_ELEMENTWISE);
  const int vec = vtlb_aligned16(d_g) && vtlb_aligned16(d_cached_x) && vtlb_aligned16(d_dx);
  VTLB_CUDA(ctx, vtlb_launch_early(relu_bwd_kernel, dim3(ew_grid(ctx, n, 1024)), dim3(256), 0, ctx->stream,
                                   (const float*)d_g, (const float*)d_cached_x, (float*)d_dx, n, vec));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_mse_fwd_bwd_f32(vtlb_ctx* ctx, const void* d_P, const void* d_T, size_t n,
                                  size_t n_div, void* d_loss, void* d_dP_or_null) {
  VTLB_ENTER(ctx);
  if (n == 0 || n_div == 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_mse_fwd_bwd_f32: empty input");
  if (!d_P || !d_T || !d_loss) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_mse_fwd_bwd_f32: null pointer");
  vtlb_prof_scope prof(ctx, VTLB_PHASE_ELEMENTWISE);
  if (n <= 8192) {
    VTLB_CUDA(ctx, vtlb_launch_early(mse_short_kernel, dim3(1), dim3(256), 0, ctx->stream, (const float*)d_P,
                                     (const float*)d_T, n, (double)n_div, (float*)d_dP_or_null, (float*)d_loss));
    VTLB_LAUNCHED(ctx);
    return VTLB_OK;
  }
  const int blocks = ew_grid(ctx, n, 2048);
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, (size_t)blocks * sizeof(double), &scr);
  if (rc) return rc;
  mse_partial_kernel<<<blocks, 256, 0, ctx->stream>>>((const float*)d_P, (const float*)d_T, n,
                                                      (float*)d_dP_or_null, (double*)scr);
  VTLB_LAUNCHED(ctx);
  VTLB_CUDA(ctx, vtlb_launch_early(loss_final_kernel, dim3(1), dim3(256), 0, ctx->stream, (const double*)scr, blocks,
                                   (double)n_div, 1, (float*)d_loss));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_softmax_ce_fwd_bwd_f32(vtlb_ctx* ctx, const void* d_X, const void* d_T, int B,
                                         int C, int batch_div, void* d_loss, void* d_dX_or_null) {
  VTLB_ENTER(ctx);
  if (B <= 0 || C <= 0 || batch_div <= 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_softmax_ce_fwd_bwd_f32: bad shape B=%d C=%d div=%d", B, C, batch_div);
  if (!d_X || !d_T || !d_loss) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_softmax_ce_fwd_bwd_f32: null pointer");
  const int blocks = (B + 127) / 128;
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, (size_t)blocks * sizeof(double), &scr);
  if (rc) return rc;
  VTLB_CUDA(ctx, vtlb_launch_early(softmax_ce_kernel, dim3(blocks), dim3(128), 0, ctx->stream, (const float*)d_X,
                                   (const float*)d_T, B, C, (double)batch_div, (float*)d_dX_or_null, (double*)scr));
  VTLB_LAUNCHED(ctx);
  VTLB_CUDA(ctx, vtlb_launch_early(loss_final_kernel, dim3(1), dim3(256), 0, ctx->stream, (const double*)scr, blocks,
                                   (double)batch_div, 0, (float*)d_loss));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}
