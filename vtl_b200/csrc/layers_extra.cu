// The memory-bound layers that sit next to the GEMMs in the reference's examples: softmax over
// the last dimension, average pooling, 1-D batch normalisation; each with the reference's own
// arithmetic (what is f64 there is f64 here, what is a sequential f32 sum there is one here).
//   softmax     nn/internal/activation.v:423-457 (forward), :285-332 (deriv_softmax)
//   avg-pool    nn/internal/pool.v:6-45, 62-101
//   batchnorm1d nn/internal/batchnorm.v:7-140; running statistics nn/layers/batchnorm.v:84-97
#include "common.cuh"

namespace {

int ex_grid(vtlb_ctx* ctx, size_t items, int per_block) {
  size_t b = (items + per_block - 1) / per_block;
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  return b < 1 ? 1 : (int)b;
}

// ---------------------------------------------------------------- softmax
// One thread per row: the reference sums a row in order, and rows are short (class counts).
__global__ void __launch_bounds__(128) softmax_fwd_kernel(const float* __restrict__ x, size_t rows, size_t n,
                                                          float* __restrict__ y) {
  for (size_t r = blockIdx.x * (size_t)blockDim.x + threadIdx.x; r < rows; r += (size_t)gridDim.x * blockDim.x) {
    const float* xr = x + r * n;
    double mx = (double)xr[0];
    for (size_t c = 1; c < n; ++c) {
      const double v = (double)xr[c];
      if (v > mx) mx = v;
    }
    double sum = 0.0;
    for (size_t c = 0; c < n; ++c) sum = __dadd_rn(sum, exp(__dsub_rn((double)xr[c], mx)));
    for (size_t c = 0; c < n; ++c) y[r * n + c] = (float)__ddiv_rn(exp(__dsub_rn((double)xr[c], mx)), sum);
  }
}

__global__ void __launch_bounds__(128) softmax_bwd_kernel(const float* __restrict__ g, const float* __restrict__ x,
                                                          size_t rows, size_t n, float* __restrict__ dx) {
  for (size_t r = blockIdx.x * (size_t)blockDim.x + threadIdx.x; r < rows; r += (size_t)gridDim.x * blockDim.x) {
    const float* xr = x + r * n;
    const float* gr = g + r * n;
    float mx = xr[0];
    for (size_t c = 1; c < n; ++c)
      if (xr[c] > mx) mx = xr[c];
    float sum = 0.0f;
    for (size_t c = 0; c < n; ++c) sum = __fadd_rn(sum, (float)exp((double)__fsub_rn(xr[c], mx)));
    float ws = 0.0f;
    for (size_t c = 0; c < n; ++c) {
      const float s = __fdiv_rn((float)exp((double)__fsub_rn(xr[c], mx)), sum);
      ws = __fadd_rn(ws, __fmul_rn(gr[c], s));
    }
    for (size_t c = 0; c < n; ++c) {
      const float s = __fdiv_rn((float)exp((double)__fsub_rn(xr[c], mx)), sum);
      dx[r * n + c] = __fmul_rn(s, __fsub_rn(gr[c], ws));
    }
  }
}

// ---------------------------------------------------------------- average pooling
struct PoolDims {
  int B, C, H, W, kh, kw, ph, pw, sh, sw, OH, OW;
};

__global__ void __launch_bounds__(256) avgpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          PoolDims d) {
  const int n = d.B * d.C * d.OH * d.OW;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int ow = i % d.OW, r = i / d.OW, oh = r % d.OH, nc = r / d.OH;
    double sum = 0.0;
    for (int a = 0; a < d.kh; ++a) {
      const int ih = oh * d.sh - d.ph + a;
      if (ih < 0 || ih >= d.H) continue;
      for (int b = 0; b < d.kw; ++b) {
        const int iw = ow * d.sw - d.pw + b;
        if (iw < 0 || iw >= d.W) continue;
        sum = __dadd_rn(sum, (double)x[((size_t)nc * d.H + ih) * d.W + iw]);
      }
    }
    y[i] = (float)__ddiv_rn(sum, (double)(d.kh * d.kw));
  }
}

// gather form of the backward: every input element adds up the windows that cover it, in (oh, ow) order
__global__ void __launch_bounds__(256) avgpool_bwd_kernel(const float* __restrict__ g, float* __restrict__ dx,
                                                          PoolDims d) {
  const int n = d.B * d.C * d.H * d.W;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int iw = i % d.W, r = i / d.W, ih = r % d.H, nc = r / d.H;
    double sum = 0.0;
    for (int oh = 0; oh < d.OH; ++oh) {
      const int a = ih - (oh * d.sh - d.ph);
      if (a < 0 || a >= d.kh) continue;
      for (int ow = 0; ow < d.OW; ++ow) {
        const int b = iw - (ow * d.sw - d.pw);
        if (b < 0 || b >= d.kw) continue;
        sum = __dadd_rn(sum, (double)g[((size_t)nc * d.OH + oh) * d.OW + ow]);
      }
    }
    dx[i] = (float)__ddiv_rn(sum, (double)(d.kh * d.kw));
  }
}

// one warp per (b, c) plane; lane partial sums in f64, combined by shuffles (fixed order)
__global__ void __launch_bounds__(256) global_avgpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                 int planes, int hw) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < planes; p += warps) {
    const float* src = x + (size_t)p * hw;
    double sum = 0.0;
    for (int i = lane; i < hw; i += 32) sum += (double)src[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) y[p] = (float)__ddiv_rn(sum, (double)hw);
  }
}
__global__ void __launch_bounds__(256) global_avgpool_bwd_kernel(const float* __restrict__ g, float* __restrict__ dx,
                                                                 size_t n, int hw) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dx[i] = (float)__ddiv_rn((double)g[i / hw], (double)hw);
}

// ---------------------------------------------------------------- batchnorm1d
// Column sums of x[B, F] (optionally of (x - mean)^2 or of g * (x - mean)) in f64: partial[s][c]
// over the rows of slice s, then a second kernel adds the slices in order.  Threads run along the
// features, so every load instruction reads one contiguous piece of a row.
enum { BN_SUM = 0, BN_SQDIFF = 1, BN_PROD_CENTERED = 2 };
template <int MODE>
__global__ void __launch_bounds__(256) bn_colsum_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                        const double* __restrict__ mean, int B, int F,
                                                        double* __restrict__ partial) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const int S = gridDim.y, s = blockIdx.y;
  const int per = (B + S - 1) / S;
  const int r0 = s * per, r1 = min(B, r0 + per);
  const double mu = MODE == BN_SUM ? 0.0 : mean[c];
  double acc = 0.0;
  for (int r = r0; r < r1; ++r) {
    const double v = (double)a[(size_t)r * F + c];
    if (MODE == BN_SUM) acc = __dadd_rn(acc, v);
    if (MODE == BN_SQDIFF) {
      const double dlt = __dsub_rn(v, mu);
      acc = __dadd_rn(acc, __dmul_rn(dlt, dlt));
    }
    if (MODE == BN_PROD_CENTERED) acc = __dadd_rn(acc, __dmul_rn(v, __dsub_rn((double)b[(size_t)r * F + c], mu)));
  }
  partial[(size_t)s * F + c] = acc;
}
// out[c] = (sum over slices) / divisor
__global__ void bn_colsum_final_kernel(const double* __restrict__ partial, int S, int F, double divisor,
                                       double* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= F) return;
  double t = 0.0;
  for (int s = 0; s < S; ++s) t = __dadd_rn(t, partial[(size_t)s * F + c]);
  out[c] = __ddiv_rn(t, divisor);
}

// y = gamma * (x - mean) / sqrt(var + eps) + beta in f64; also the f32 batch statistics and the
// running statistics (blend of the ROUNDED batch statistics, as the layer does)
__global__ void __launch_bounds__(256) bn_train_apply_kernel(const float* __restrict__ x, int B, int F,
                                                             const float* __restrict__ gamma,
                                                             const float* __restrict__ beta,
                                                             const double* __restrict__ mean,
                                                             const double* __restrict__ var, double eps,
                                                             float* __restrict__ y) {
  const size_t n = (size_t)B * F;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % F);
    const double normalized = __ddiv_rn(__dsub_rn((double)x[i], mean[c]), __dsqrt_rn(__dadd_rn(var[c], eps)));
    y[i] = (float)__dadd_rn(__dmul_rn((double)gamma[c], normalized), (double)beta[c]);
  }
}
__global__ void bn_stats_kernel(const double* __restrict__ mean, const double* __restrict__ var, int F,
                                float* __restrict__ mean_out, float* __restrict__ var_out,
                                float* __restrict__ running_mean, float* __restrict__ running_var,
                                double momentum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= F) return;
  const float m = (float)mean[c], v = (float)var[c];
  mean_out[c] = m;
  var_out[c] = v;
  if (running_mean) {
    const double om = __dsub_rn(1.0, momentum);
    running_mean[c] = (float)__dadd_rn(__dmul_rn(momentum, (double)m), __dmul_rn(om, (double)running_mean[c]));
    running_var[c] = (float)__dadd_rn(__dmul_rn(momentum, (double)v), __dmul_rn(om, (double)running_var[c]));
  }
}

__global__ void __launch_bounds__(256) bn_infer_kernel(const float* __restrict__ x, int B, int F,
                                                       const float* __restrict__ gamma, const float* __restrict__ beta,
                                                       const float* __restrict__ rmean, const float* __restrict__ rvar,
                                                       double eps, float* __restrict__ y) {
  const size_t n = (size_t)B * F;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % F);
    const float stdinv = (float)__ddiv_rn(1.0, __dsqrt_rn(__dadd_rn((double)rvar[c], eps)));
    const float normalized = __fmul_rn(__fsub_rn(x[i], rmean[c]), stdinv);
    y[i] = __fadd_rn(__fmul_rn(normalized, gamma[c]), beta[c]);
  }
}

// dx = gamma * (g - gmean) / std; dgamma = gprod / std; dbeta = gsum  (f64, as written in the reference)
__global__ void __launch_bounds__(256) bn_bwd_apply_kernel(const float* __restrict__ g, int B, int F,
                                                           const float* __restrict__ gamma,
                                                           const float* __restrict__ var, double eps,
                                                           const double* __restrict__ gmean, float* __restrict__ dx) {
  const size_t n = (size_t)B * F;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % F);
    const double std = __dsqrt_rn(__dadd_rn((double)var[c], eps));
    dx[i] = (float)__ddiv_rn(__dmul_rn((double)gamma[c], __dsub_rn((double)g[i], gmean[c])), std);
  }
}
__global__ void bn_bwd_params_kernel(const double* __restrict__ gsum, const double* __restrict__ gprod,
                                     const float* __restrict__ var, double eps, int F, float* __restrict__ dgamma,
                                     float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= F) return;
  if (dgamma) dgamma[c] = (float)__ddiv_rn(gprod[c], __dsqrt_rn(__dadd_rn((double)var[c], eps)));
  if (dbeta) dbeta[c] = (float)gsum[c];
}
// mean as f64 of an f32 vector (the backward receives the rounded batch mean)
__global__ void widen_kernel(const float* __restrict__ a, int n, double* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (double)a[i];
}

int bn_slices(vtlb_ctx* ctx, int B, int F) {
  const int col_blocks = (F + 255) / 256;
  int S = (4 * ctx->sm_count + col_blocks - 1) / col_blocks;
  if (S > (B + 63) / 64) S = (B + 63) / 64;  // at least 64 rows per slice
  return S < 1 ? 1 : S;
}

template <int MODE>
int bn_colsum(vtlb_ctx* ctx, const float* a, const float* b, const double* mean, int B, int F, double divisor,
              double* partial, int S, double* out) {
  bn_colsum_kernel<MODE><<<dim3((F + 255) / 256, S), 256, 0, ctx->stream>>>(a, b, mean, B, F, partial);
  VTLB_LAUNCHED(ctx);
  bn_colsum_final_kernel<<<(F + 255) / 256, 256, 0, ctx->stream>>>(partial, S, F, divisor, out);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

int check_pool(vtlb_ctx* ctx, const char* fn, PoolDims& d) {
  if (d.B <= 0 || d.C <= 0 || d.H <= 0 || d.W <= 0 || d.kh <= 0 || d.kw <= 0 || d.sh <= 0 || d.sw <= 0 ||
      d.ph < 0 || d.pw < 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: bad geometry", fn);
  d.OH = (d.H + 2 * d.ph - d.kh) / d.sh + 1;
  d.OW = (d.W + 2 * d.pw - d.kw) / d.sw + 1;
  if (d.OH <= 0 || d.OW <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "%s: empty output", fn);
  if ((long long)d.B * d.C * d.H * d.W > 0x7fffffffLL || (long long)d.B * d.C * d.OH * d.OW > 0x7fffffffLL)
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: tensor too large for 32-bit indices", fn);
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_softmax_fwd_f32(vtlb_ctx* ctx, const void* d_x, size_t rows, size_t n, void* d_y) {
  VTLB_ENTER(ctx);
  if (rows == 0 || n == 0) return VTLB_OK;
  if (!d_x || !d_y) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_softmax_fwd_f32: null pointer");
  softmax_fwd_kernel<<<ex_grid(ctx, rows, 128), 128, 0, ctx->stream>>>((const float*)d_x, rows, n, (float*)d_y);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_softmax_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_x, size_t rows, size_t n,
                                  void* d_dx) {
  VTLB_ENTER(ctx);
  if (rows == 0 || n == 0) return VTLB_OK;
  if (!d_g || !d_x || !d_dx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_softmax_bwd_f32: null pointer");
  softmax_bwd_kernel<<<ex_grid(ctx, rows, 128), 128, 0, ctx->stream>>>((const float*)d_g, (const float*)d_x, rows, n,
                                                                      (float*)d_dx);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_avgpool2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, int B, int C, int H, int W, int kh,
                                    int kw, int ph, int pw, int sh, int sw) {
  VTLB_ENTER(ctx);
  PoolDims d{B, C, H, W, kh, kw, ph, pw, sh, sw, 0, 0};
  int rc = check_pool(ctx, "vtlb_avgpool2d_fwd_f32", d);
  if (rc) return rc;
  if (!d_x || !d_y) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_avgpool2d_fwd_f32: null pointer");
  avgpool_fwd_kernel<<<ex_grid(ctx, (size_t)B * C * d.OH * d.OW, 256), 256, 0, ctx->stream>>>((const float*)d_x,
                                                                                             (float*)d_y, d);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_avgpool2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, void* d_dx, int B, int C, int H, int W, int kh,
                                    int kw, int ph, int pw, int sh, int sw) {
  VTLB_ENTER(ctx);
  PoolDims d{B, C, H, W, kh, kw, ph, pw, sh, sw, 0, 0};
  int rc = check_pool(ctx, "vtlb_avgpool2d_bwd_f32", d);
  if (rc) return rc;
  if (!d_g || !d_dx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_avgpool2d_bwd_f32: null pointer");
  avgpool_bwd_kernel<<<ex_grid(ctx, (size_t)B * C * H * W, 256), 256, 0, ctx->stream>>>((const float*)d_g,
                                                                                       (float*)d_dx, d);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_global_avgpool2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, int B, int C, int H, int W) {
  VTLB_ENTER(ctx);
  if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || (long long)B * C > 0x7fffffffLL || (long long)H * W > 0x7fffffffLL)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_global_avgpool2d_fwd_f32: bad geometry");
  if (!d_x || !d_y) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_global_avgpool2d_fwd_f32: null pointer");
  global_avgpool_fwd_kernel<<<ex_grid(ctx, (size_t)B * C, 8), 256, 0, ctx->stream>>>((const float*)d_x, (float*)d_y,
                                                                                    B * C, H * W);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_global_avgpool2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, void* d_dx, int B, int C, int H, int W) {
  VTLB_ENTER(ctx);
  if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || (long long)H * W > 0x7fffffffLL)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_global_avgpool2d_bwd_f32: bad geometry");
  if (!d_g || !d_dx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_global_avgpool2d_bwd_f32: null pointer");
  const size_t n = (size_t)B * C * H * W;
  global_avgpool_bwd_kernel<<<ex_grid(ctx, n, 1024), 256, 0, ctx->stream>>>((const float*)d_g, (float*)d_dx, n, H * W);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_batchnorm1d_train_f32(vtlb_ctx* ctx, const void* d_x, int B, int F, const void* d_gamma,
                                        const void* d_beta, double eps, void* d_y, void* d_batch_mean,
                                        void* d_batch_var, void* d_running_mean_or_null,
                                        void* d_running_var_or_null, double momentum) {
  VTLB_ENTER(ctx);
  if (B <= 0 || F <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_batchnorm1d_train_f32: bad shape B=%d F=%d", B, F);
  if (!d_x || !d_gamma || !d_beta || !d_y || !d_batch_mean || !d_batch_var ||
      (!d_running_mean_or_null) != (!d_running_var_or_null))
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_batchnorm1d_train_f32: null pointer");
  const int S = bn_slices(ctx, B, F);
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, ((size_t)S * F + 2 * (size_t)F) * sizeof(double), &scr);
  if (rc) return rc;
  double* partial = (double*)scr;
  double* mean = partial + (size_t)S * F;
  double* var = mean + F;
  const float* x = (const float*)d_x;
  if ((rc = bn_colsum<BN_SUM>(ctx, x, nullptr, nullptr, B, F, (double)B, partial, S, mean))) return rc;
  if ((rc = bn_colsum<BN_SQDIFF>(ctx, x, nullptr, mean, B, F, (double)B, partial, S, var))) return rc;
  bn_train_apply_kernel<<<ex_grid(ctx, (size_t)B * F, 1024), 256, 0, ctx->stream>>>(
      x, B, F, (const float*)d_gamma, (const float*)d_beta, mean, var, eps, (float*)d_y);
  VTLB_LAUNCHED(ctx);
  bn_stats_kernel<<<(F + 255) / 256, 256, 0, ctx->stream>>>(mean, var, F, (float*)d_batch_mean, (float*)d_batch_var,
                                                           (float*)d_running_mean_or_null,
                                                           (float*)d_running_var_or_null, momentum);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_batchnorm1d_infer_f32(vtlb_ctx* ctx, const void* d_x, int B, int F, const void* d_gamma,
                                        const void* d_beta, const void* d_running_mean, const void* d_running_var,
                                        double eps, void* d_y) {
  VTLB_ENTER(ctx);
  if (B <= 0 || F <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_batchnorm1d_infer_f32: bad shape B=%d F=%d", B, F);
  if (!d_x || !d_gamma || !d_beta || !d_running_mean || !d_running_var || !d_y)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_batchnorm1d_infer_f32: null pointer");
  bn_infer_kernel<<<ex_grid(ctx, (size_t)B * F, 1024), 256, 0, ctx->stream>>>(
      (const float*)d_x, B, F, (const float*)d_gamma, (const float*)d_beta, (const float*)d_running_mean,
      (const float*)d_running_var, eps, (float*)d_y);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_batchnorm1d_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_x, int B, int F,
                                      const void* d_gamma, const void* d_batch_mean, const void* d_batch_var,
                                      double eps, void* d_dx_or_null, void* d_dgamma_or_null,
                                      void* d_dbeta_or_null) {
  VTLB_ENTER(ctx);
  if (B <= 0 || F <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_batchnorm1d_bwd_f32: bad shape B=%d F=%d", B, F);
  if (!d_g || !d_x || !d_gamma || !d_batch_mean || !d_batch_var)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_batchnorm1d_bwd_f32: null pointer");
  const int S = bn_slices(ctx, B, F);
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, ((size_t)S * F + 4 * (size_t)F) * sizeof(double), &scr);
  if (rc) return rc;
  double* partial = (double*)scr;
  double* gsum = partial + (size_t)S * F;
  double* gmean = gsum + F;
  double* gprod = gmean + F;
  double* mean64 = gprod + F;
  const float* g = (const float*)d_g;
  if ((rc = bn_colsum<BN_SUM>(ctx, g, nullptr, nullptr, B, F, 1.0, partial, S, gsum))) return rc;
  if ((rc = bn_colsum<BN_SUM>(ctx, g, nullptr, nullptr, B, F, (double)B, partial, S, gmean))) return rc;
  if (d_dx_or_null) {
    bn_bwd_apply_kernel<<<ex_grid(ctx, (size_t)B * F, 1024), 256, 0, ctx->stream>>>(
        g, B, F, (const float*)d_gamma, (const float*)d_batch_var, eps, gmean, (float*)d_dx_or_null);
    VTLB_LAUNCHED(ctx);
  }
  if (d_dgamma_or_null || d_dbeta_or_null) {
    widen_kernel<<<(F + 255) / 256, 256, 0, ctx->stream>>>((const float*)d_batch_mean, F, mean64);
    VTLB_LAUNCHED(ctx);
    if ((rc = bn_colsum<BN_PROD_CENTERED>(ctx, g, (const float*)d_x, mean64, B, F, 1.0, partial, S, gprod))) return rc;
    bn_bwd_params_kernel<<<(F + 255) / 256, 256, 0, ctx->stream>>>(gsum, gprod, (const float*)d_batch_var, eps, F,
                                                                  (float*)d_dgamma_or_null, (float*)d_dbeta_or_null);
    VTLB_LAUNCHED(ctx);
  }
  return VTLB_OK;
}
