// f32 dense contraction: la.matmul / Linear forward and backward of the
// reference (la/la.v:38-55, nn/layers/linear_forward_f32.v:16-18,
// nn/gates/layers/linear.v:69-79) on tcgen05 tensor cores.
//
// The reference multiplies in f64 and rounds once.  Here every f32 operand x is
// split into two TF32 numbers, hi = tf32(x) and lo = tf32(x - hi), by a
// memory-bound pass that also lays the operand out K-major (transposing when
// the caller's layout is the other way round), and the GEMM issues three
// kind::tf32 MMAs per K step (lo.hi + hi.lo + hi.hi).  The dropped lo.lo term
// and the rounding of lo are ~2^-22 relative per product, well inside the
// 1e-5*sqrt(K)*max|A|*max|B| bound.
#include "f32_common.cuh"

namespace {

using f32::split1;

// src [R, C] row-major (C % 4 == 0, 16-byte aligned) -> hi/lo [R, C].  12 bytes/element.
__global__ void __launch_bounds__(256) split_rows_vec_kernel(const float4* __restrict__ src,
                                                             float4* __restrict__ hi,
                                                             float4* __restrict__ lo, size_t n4) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
       i += (size_t)gridDim.x * blockDim.x) {
    float4 x = src[i], h, l;
    split1(x.x, h.x, l.x);
    split1(x.y, h.y, l.y);
    split1(x.z, h.z, l.z);
    split1(x.w, h.w, l.w);
    hi[i] = h;
    lo[i] = l;
  }
}

// General case: src [R, C] -> hi/lo [R, ldo], ldo >= C.
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ src, int R,
                                                         int C, int ldo, float* __restrict__ hi,
                                                         float* __restrict__ lo) {
  const size_t n = (size_t)R * C;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / C, c = i - r * C;
    float h, l;
    split1(src[i], h, l);
    hi[r * ldo + c] = h;
    lo[r * ldo + c] = l;
  }
}

// src [R, C] row-major -> hi/lo [C, ldo] (the transpose), ldo >= R.  32x32 tiles
// through shared memory so that both the reads and the writes are coalesced.
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ src, int R,
                                                              int C, int ldo,
                                                              float* __restrict__ hi,
                                                              float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int tiles_c = (C + 31) / 32, tiles_r = (R + 31) / 32;
  const long long ntiles = (long long)tiles_c * tiles_r;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int r0 = (int)(t / tiles_c) * 32, c0 = (int)(t % tiles_c) * 32;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int r = r0 + ty + j, c = c0 + tx;
      tile[ty + j][tx] = (r < R && c < C) ? src[(size_t)r * C + c] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int c = c0 + ty + j, r = r0 + tx;
      if (c < C && r < R) {
        float h, l;
        split1(tile[tx][ty + j], h, l);
        hi[(size_t)c * ldo + r] = h;
        lo[(size_t)c * ldo + r] = l;
      }
    }
    __syncthreads();
  }
}

// Column sums of G[M,N] in f64: partial[s][n] = sum over rows r == s (mod S).
__global__ void __launch_bounds__(128) colsum_partial_kernel(const float* __restrict__ G, int M,
                                                             int N, double* __restrict__ partial) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  double s = 0.0;
  for (int r = blockIdx.y; r < M; r += gridDim.y) s += (double)G[(size_t)r * N + n];
  partial[(size_t)blockIdx.y * N + n] = s;
}
__global__ void __launch_bounds__(128) colsum_final_kernel(const double* __restrict__ partial,
                                                           int S, int N, float* __restrict__ out) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  double s = 0.0;
  for (int i = 0; i < S; ++i) s += partial[(size_t)i * N + n];
  out[n] = (float)s;
}

// Column sums for short matrices in one launch: 32 columns per CTA, 8 row slices summed in f64
// and combined through shared memory in a fixed order.
__global__ void __launch_bounds__(256) colsum_short_kernel(const float* __restrict__ G, int M, int N,
                                                           float* __restrict__ out) {
  __shared__ double part[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int n = blockIdx.x * 32 + tx;
  double s = 0.0;
  if (n < N)
    for (int r = ty; r < M; r += 8) s += (double)G[(size_t)r * N + n];
  part[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && n < N) {
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += part[i][tx];
    out[n] = (float)t;
  }
}

// out[i] = sum over splits of partial[k][i].  One element per thread; eight running sums per
// element keep eight loads in flight (the order of the additions is fixed: split k goes to sum
// k mod 8, the eight sums are combined pairwise at the end).
__global__ void __launch_bounds__(256) reduce_splits_kernel(const float* __restrict__ partial,
                                                            int splits, size_t n,
                                                            float* __restrict__ out) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    float s[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] = 0.0f;
    int k = 0;
    for (; k + 8 <= splits; k += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = partial[(size_t)(k + j) * n + i];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = __fadd_rn(s[j], v[j]);
    }
    for (int j = 0; k < splits; ++k, ++j) s[j] = __fadd_rn(s[j], partial[(size_t)k * n + i]);
    const float a = __fadd_rn(__fadd_rn(s[0], s[1]), __fadd_rn(s[2], s[3]));
    const float b = __fadd_rn(__fadd_rn(s[4], s[5]), __fadd_rn(s[6], s[7]));
    out[i] = __fadd_rn(a, b);
  }
}

}  // namespace

// Writes op(src) as K-major hi/lo [rows, ld] where rows x kdim is the logical
// operand.  `transposed` says src is stored [kdim, rows].
int f32::split_operand(vtlb_ctx* ctx, const float* src, int rows, int kdim, bool transposed, int ld,
                  float* hi, float* lo) {
  vtlb_prof_scope prof(ctx, VTLB_PHASE_SPLIT);
  if (!transposed) {
    if ((kdim & 3) == 0 && ld == kdim && vtlb_aligned16(src)) {
      const size_t n4 = (size_t)rows * kdim / 4;
      split_rows_vec_kernel<<<f32::grid_for(ctx, n4, 256 * 4), 256, 0, ctx->stream>>>(
          (const float4*)src, (float4*)hi, (float4*)lo, n4);
    } else {
      split_rows_kernel<<<f32::grid_for(ctx, (size_t)rows * kdim, 256 * 4), 256, 0, ctx->stream>>>(
          src, rows, kdim, ld, hi, lo);
    }
  } else {
    const size_t tiles = (size_t)((rows + 31) / 32) * ((kdim + 31) / 32);
    split_transpose_kernel<<<f32::grid_for(ctx, tiles, 1), 256, 0, ctx->stream>>>(src, kdim, rows, ld,
                                                                                 hi, lo);
  }
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

namespace {

using f32::split_operand;

// Optional extras of a product (all null / zero by default):
//   a_planes / b_planes   the operand already split into K-major TF32 planes [rows, ld(K)] by whoever
//                         produced it (then no split pass runs for it)
//   mask                  ReLU backward on the result: C = mask < 0 ? 0 : C, mask laid out like C
//   out_rows / out_cols   receive the TF32 planes of C ([M, ld(N)]) and of C transposed ([N, ld(M)])
// The tensor-core kernels do mask and planes in their epilogue; where they cannot (CUDA-core route,
// unaligned pointers) the same results come from separate passes over the stored C.
struct GemmExtras {
  const vtlb_planes* a_planes = nullptr;
  const vtlb_planes* b_planes = nullptr;
  const float* mask = nullptr;
  const vtlb_planes* out_rows = nullptr;
  const vtlb_planes* out_cols = nullptr;
};

int relu_mask_inplace(vtlb_ctx* ctx, float* C, const float* mask, size_t n) {
  return vtlb_relu_bwd_f32(ctx, C, mask, C, n);
}

int gemm_f32_impl(vtlb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A,
                  const float* B, float* C, const float* bias, int relu, float* pre,
                  const GemmExtras& ex = GemmExtras()) {
  if (!vtlb_aligned16(C) || (pre && !vtlb_aligned16(pre)) || (bias && !vtlb_aligned16(bias)))
    return vtlb_fail(ctx, VTLB_EINVAL, "f32 GEMM: output and bias pointers must be 16-byte aligned");
  const int ld_rows = vtlb_plane_ld(N), ld_cols = vtlb_plane_ld(M);
  int rc, fused = 0;
  if (2.0 * M * N * K <= ctx->small_gemm_flops) {  // launch-latency-bound sizes: CUDA cores, no split passes
    if ((rc = f32::sgemm_small(ctx, transA, transB, M, N, K, A, B, C, bias, relu, pre, nullptr, nullptr, ex.mask)))
      return rc;
    if (ex.mask) fused |= 2;  // the mask is part of that kernel's epilogue
  } else {
    f32::Planes p;
    if ((rc = f32::alloc_planes(ctx, ex.a_planes ? 0 : M, ex.b_planes ? 0 : N, K, 0, &p))) return rc;
    // op(A) is [M,K]: stored [K,M] when transA.  The B operand of the kernel is
    // [N,K] K-major: B stored [K,N] (transB == 0) must be transposed.
    if (ex.a_planes) {
      p.a_hi = (float*)ex.a_planes->hi;
      p.a_lo = (float*)ex.a_planes->lo;
    } else if ((rc = split_operand(ctx, A, M, K, transA != 0, p.ld, p.a_hi, p.a_lo))) {
      return rc;
    }
    if (ex.b_planes) {
      p.b_hi = (float*)ex.b_planes->hi;
      p.b_lo = (float*)ex.b_planes->lo;
    } else if ((rc = split_operand(ctx, B, N, K, transB == 0, p.ld, p.b_hi, p.b_lo))) {
      return rc;
    }
    f32::EpiBiasRelu epi{C, bias, pre, N, relu};
    epi.mask = ex.mask;
    epi.planes = (ex.out_rows ? 1 : 0) | (ex.out_cols ? 2 : 0);
    if (ex.out_rows) {
      epi.rows_hi = (float*)ex.out_rows->hi;
      epi.rows_lo = (float*)ex.out_rows->lo;
      epi.ld_rows = ld_rows;
    }
    if (ex.out_cols) {
      epi.cols_hi = (float*)ex.out_cols->hi;
      epi.cols_lo = (float*)ex.out_cols->lo;
      epi.ld_cols = ld_cols;
    }
    if ((rc = f32::launch_tf32x3(ctx, p, M, N, K, epi, 1, &fused))) return rc;
  }
  if (ex.mask && !(fused & 2) && (rc = relu_mask_inplace(ctx, C, ex.mask, (size_t)M * N))) return rc;
  // planes written by the epilogue are those of the masked result only when it also masked
  const bool planes_ok = (fused & 1) && (!ex.mask || (fused & 2));
  if (!planes_ok) {
    if (ex.out_rows && (rc = split_operand(ctx, C, M, N, false, ld_rows, (float*)ex.out_rows->hi, (float*)ex.out_rows->lo)))
      return rc;
    if (ex.out_cols && (rc = split_operand(ctx, C, N, M, true, ld_cols, (float*)ex.out_cols->hi, (float*)ex.out_cols->lo)))
      return rc;
  }
  return VTLB_OK;
}

int colsum(vtlb_ctx* ctx, const float* G, int M, int N, float* out) {
  vtlb_prof_scope prof(ctx, VTLB_PHASE_ELEMENTWISE);
  if (M <= 1024) {
    colsum_short_kernel<<<(N + 31) / 32, 256, 0, ctx->stream>>>(G, M, N, out);
    VTLB_LAUNCHED(ctx);
    return VTLB_OK;
  }
  int S = (M + 63) / 64;
  if (S > 64) S = 64;
  if (S < 1) S = 1;
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, (size_t)S * N * sizeof(double), &scr);
  if (rc) return rc;
  dim3 grid((N + 127) / 128, S);
  colsum_partial_kernel<<<grid, 128, 0, ctx->stream>>>(G, M, N, (double*)scr);
  VTLB_LAUNCHED(ctx);
  colsum_final_kernel<<<(N + 127) / 128, 128, 0, ctx->stream>>>((const double*)scr, S, N, out);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

int check_f32(vtlb_ctx* ctx, const char* fn, int M, int N, int K) {
  if (M < 0 || N < 0 || K <= 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: bad shape M=%d N=%d K=%d (K must be > 0)", fn, M, N, K);
  return VTLB_OK;
}

}  // namespace

int f32::reduce_splits(vtlb_ctx* ctx, const float* partial, int splits, size_t n, float* out) {
  VTLB_CUDA(ctx, vtlb_launch_early(reduce_splits_kernel, dim3(f32::grid_for(ctx, n, 256)), dim3(256), 0, ctx->stream, partial,
                                   splits, n, out));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_gemm_f32(vtlb_ctx* ctx, int transA, int transB, int M, int N, int K,
                           const void* d_A, const void* d_B, void* d_C,
                           const void* d_bias_or_null, int relu) {
  VTLB_ENTER(ctx);
  int rc = check_f32(ctx, "vtlb_gemm_f32", M, N, K);
  if (rc) return rc;
  if (M == 0 || N == 0) return VTLB_OK;
  if (!d_A || !d_B || !d_C) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_gemm_f32: null pointer");
  return gemm_f32_impl(ctx, transA, transB, M, N, K, (const float*)d_A, (const float*)d_B,
                       (float*)d_C, (const float*)d_bias_or_null, relu, nullptr);
}

namespace {

int check_planes(vtlb_ctx* ctx, const char* fn, const char* what, const vtlb_planes* p) {
  if (p && (!p->hi || !p->lo || !vtlb_aligned16(p->hi) || !vtlb_aligned16(p->lo)))
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: %s planes need two 16-byte-aligned arrays", fn, what);
  return VTLB_OK;
}

int linear_fwd_impl(vtlb_ctx* ctx, const char* fn, const void* d_X, const void* d_W, const void* d_b_or_null,
                    void* d_Y, int M, int N, int K, int relu, void* d_pre_or_null, const vtlb_planes* x_rows,
                    const vtlb_planes* y_rows, const vtlb_planes* y_cols) {
  int rc = check_f32(ctx, fn, M, N, K);
  if (rc) return rc;
  if (M == 0 || N == 0) return VTLB_OK;
  if (!d_X || !d_W || !d_Y) return vtlb_fail(ctx, VTLB_EINVAL, "%s: null pointer", fn);
  if ((rc = check_planes(ctx, fn, "input", x_rows)) || (rc = check_planes(ctx, fn, "output", y_rows)) ||
      (rc = check_planes(ctx, fn, "transposed output", y_cols)))
    return rc;
  if (!x_rows && !y_rows && !y_cols && 2.0 * M * N * K <= ctx->small_gemm_flops &&
      f32::narrow_linear_ok(M, N, K, d_X, d_W, d_X))
    return f32::narrow_linear_fwd(ctx, (const float*)d_X, (const float*)d_W, (const float*)d_b_or_null, (float*)d_Y, M, N,
                                  K, relu, (float*)d_pre_or_null);
  GemmExtras ex;
  ex.a_planes = x_rows;
  ex.out_rows = y_rows;
  ex.out_cols = y_cols;
  return gemm_f32_impl(ctx, 0, 1, M, N, K, (const float*)d_X, (const float*)d_W, (float*)d_Y,
                       (const float*)d_b_or_null, relu, (float*)d_pre_or_null, ex);
}

int linear_bwd_impl(vtlb_ctx* ctx, const char* fn, const void* d_G, const void* d_X, const void* d_W,
                    void* d_dX_or_null, void* d_dW_or_null, void* d_db_or_null, int M, int N, int K,
                    const vtlb_planes* g_rows, const vtlb_planes* g_cols, const vtlb_planes* x_cols,
                    const void* d_relu_mask_src_or_null, const vtlb_planes* dx_rows, const vtlb_planes* dx_cols) {
  if (M <= 0 || N <= 0 || K <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "%s: bad shape M=%d N=%d K=%d", fn, M, N, K);
  if (!d_G) return vtlb_fail(ctx, VTLB_EINVAL, "%s: null gradient", fn);
  int rc;
  if ((rc = check_planes(ctx, fn, "gradient", g_rows)) || (rc = check_planes(ctx, fn, "transposed gradient", g_cols)) ||
      (rc = check_planes(ctx, fn, "transposed input", x_cols)) || (rc = check_planes(ctx, fn, "dX", dx_rows)) ||
      (rc = check_planes(ctx, fn, "transposed dX", dx_cols)))
    return rc;
  if (!d_dX_or_null && (d_relu_mask_src_or_null || dx_rows || dx_cols))
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: a mask or dX planes were given without a dX output", fn);
  // a layer with few output features and many inputs: memory-bound kernels that stream X / dX once
  const bool any_planes = g_rows || g_cols || x_cols || dx_rows || dx_cols;
  const bool narrow = !any_planes && 2.0 * M * N * K <= ctx->small_gemm_flops;
  if (narrow && d_dX_or_null && d_W && f32::narrow_linear_ok(M, N, K, d_dX_or_null, d_W, d_W)) {
    if ((rc = f32::narrow_linear_dx(ctx, (const float*)d_G, (const float*)d_W, (float*)d_dX_or_null, M, N, K))) return rc;
    if (d_relu_mask_src_or_null &&
        (rc = relu_mask_inplace(ctx, (float*)d_dX_or_null, (const float*)d_relu_mask_src_or_null, (size_t)M * K)))
      return rc;
    d_dX_or_null = nullptr;
  }
  if (narrow && d_dW_or_null && d_X && f32::narrow_linear_ok(M, N, K, d_X, d_dW_or_null, d_X)) {
    if ((rc = f32::narrow_linear_dw(ctx, (const float*)d_G, (const float*)d_X, (float*)d_dW_or_null,
                                    (float*)d_db_or_null, M, N, K)))
      return rc;
    d_dW_or_null = nullptr;
    d_db_or_null = nullptr;
  }
  if (d_dX_or_null) {  // dX[M,K] = G[M,N] . W[N,K]   (then, optionally, ReLU backward of the layer below)
    if (!d_W) return vtlb_fail(ctx, VTLB_EINVAL, "%s: dX needs W", fn);
    GemmExtras ex;
    ex.a_planes = g_rows;
    ex.mask = (const float*)d_relu_mask_src_or_null;
    ex.out_rows = dx_rows;
    ex.out_cols = dx_cols;
    if ((rc = gemm_f32_impl(ctx, 0, 0, M, K, N, (const float*)d_G, (const float*)d_W, (float*)d_dX_or_null, nullptr,
                            0, nullptr, ex)))
      return rc;
  }
  bool db_done = false;
  if (d_dW_or_null) {  // dW[N,K] = G^T[N,M] . X[M,K]
    if (!d_X) return vtlb_fail(ctx, VTLB_EINVAL, "%s: dW needs X", fn);
    if (d_db_or_null && 2.0 * M * N * K <= ctx->small_gemm_flops && vtlb_aligned16(d_dW_or_null)) {
      // small product: the CUDA-core kernel sums the rows of G^T (= the bias gradient) on the way
      if ((rc = f32::sgemm_small(ctx, 1, 0, N, K, M, (const float*)d_G, (const float*)d_X, (float*)d_dW_or_null,
                                 nullptr, 0, nullptr, (float*)d_db_or_null, &db_done)))
        return rc;
    } else {
      GemmExtras ex;
      ex.a_planes = g_cols;
      ex.b_planes = x_cols;
      if ((rc = gemm_f32_impl(ctx, 1, 0, N, K, M, (const float*)d_G, (const float*)d_X, (float*)d_dW_or_null,
                              nullptr, 0, nullptr, ex)))
        return rc;
    }
  }
  if (d_db_or_null && !db_done) {
    if ((rc = colsum(ctx, (const float*)d_G, M, N, (float*)d_db_or_null))) return rc;
  }
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_plane_ld(int kdim) { return kdim <= 0 ? 0 : (int)vtlb_round_up((size_t)kdim, 4); }

VTLB_API int vtlb_f32_planes_worthwhile(vtlb_ctx* ctx, int M, int N, int K) {
  // products the CUDA-core route takes never read operand planes
  return ctx && M > 0 && N > 0 && K > 0 && 2.0 * M * N * K > ctx->small_gemm_flops;
}

VTLB_API int vtlb_linear_fwd_f32(vtlb_ctx* ctx, const void* d_X, const void* d_W,
                                 const void* d_b_or_null, void* d_Y, int M, int N, int K, int relu,
                                 void* d_pre_or_null) {
  VTLB_ENTER(ctx);
  return linear_fwd_impl(ctx, "vtlb_linear_fwd_f32", d_X, d_W, d_b_or_null, d_Y, M, N, K, relu, d_pre_or_null,
                         nullptr, nullptr, nullptr);
}

VTLB_API int vtlb_linear_fwd_f32_planes(vtlb_ctx* ctx, const void* d_X, const void* d_W, const void* d_b_or_null,
                                        void* d_Y, int M, int N, int K, int relu, void* d_pre_or_null,
                                        const vtlb_planes* x_rows_or_null, const vtlb_planes* y_rows_or_null,
                                        const vtlb_planes* y_cols_or_null) {
  VTLB_ENTER(ctx);
  return linear_fwd_impl(ctx, "vtlb_linear_fwd_f32_planes", d_X, d_W, d_b_or_null, d_Y, M, N, K, relu,
                         d_pre_or_null, x_rows_or_null, y_rows_or_null, y_cols_or_null);
}

VTLB_API int vtlb_linear_bwd_f32(vtlb_ctx* ctx, const void* d_G, const void* d_X, const void* d_W,
                                 void* d_dX_or_null, void* d_dW_or_null, void* d_db_or_null, int M,
                                 int N, int K) {
  VTLB_ENTER(ctx);
  return linear_bwd_impl(ctx, "vtlb_linear_bwd_f32", d_G, d_X, d_W, d_dX_or_null, d_dW_or_null, d_db_or_null, M, N,
                         K, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
}

VTLB_API int vtlb_linear_bwd_f32_planes(vtlb_ctx* ctx, const void* d_G, const void* d_X, const void* d_W,
                                        void* d_dX_or_null, void* d_dW_or_null, void* d_db_or_null, int M, int N,
                                        int K, const vtlb_planes* g_rows_or_null, const vtlb_planes* g_cols_or_null,
                                        const vtlb_planes* x_cols_or_null, const void* d_relu_mask_src_or_null,
                                        const vtlb_planes* dx_rows_or_null, const vtlb_planes* dx_cols_or_null) {
  VTLB_ENTER(ctx);
  return linear_bwd_impl(ctx, "vtlb_linear_bwd_f32_planes", d_G, d_X, d_W, d_dX_or_null, d_dW_or_null, d_db_or_null,
                         M, N, K, g_rows_or_null, g_cols_or_null, x_cols_or_null, d_relu_mask_src_or_null,
                         dx_rows_or_null, dx_cols_or_null);
}

VTLB_API int vtlb_split_planes_f32(vtlb_ctx* ctx, const void* d_src, int R, int C, const vtlb_planes* rows_or_null,
                                   const vtlb_planes* cols_or_null) {
  VTLB_ENTER(ctx);
  if (R <= 0 || C <= 0 || !d_src) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_split_planes_f32: bad arguments");
  int rc;
  if ((rc = check_planes(ctx, "vtlb_split_planes_f32", "row", rows_or_null)) ||
      (rc = check_planes(ctx, "vtlb_split_planes_f32", "column", cols_or_null)))
    return rc;
  if (rows_or_null && (rc = split_operand(ctx, (const float*)d_src, R, C, false, vtlb_plane_ld(C),
                                          (float*)rows_or_null->hi, (float*)rows_or_null->lo)))
    return rc;
  if (cols_or_null && (rc = split_operand(ctx, (const float*)d_src, C, R, true, vtlb_plane_ld(R),
                                          (float*)cols_or_null->hi, (float*)cols_or_null->lo)))
    return rc;
  return VTLB_OK;
}

// ---------------------------------------------------------------- bias gradient without allocation
// Some hosts cannot let this library allocate device memory while they run: a
// serving process that handed every byte of HBM to its own pools at start-up
// (so a cudaMalloc here would simply fail), or a control loop with a latency
// budget that the implicit synchronisation of an allocation would break.  For
// them the bias gradient (column sums of G) is offered with its partial-sum
// scratch in a fixed array that is part of the library image: every GPU that
// loads the library holds these 2 MiB until the process exits.
constexpr int kNoAllocMaxN = 4096;  // widest G supported by the fixed scratch
constexpr int kNoAllocMaxS = 64;    // row slices (same cap as the allocating path)
static __device__ __align__(256) double g_bias_grad_scratch[(size_t)kNoAllocMaxS * kNoAllocMaxN];

// In host code the array's name is only a handle; the device address has to be
// asked for, once per device, with that device current.
// (Atomic: two host threads may make their first calls on different contexts at the same time;
// both would resolve the same address, so the order of the stores does not matter.)
static std::atomic<double*> g_bias_grad_scratch_addr[64];

VTLB_API int vtlb_bias_grad_f32_noalloc(vtlb_ctx* ctx, const void* d_G, int M, int N, void* d_db) {
  VTLB_ENTER(ctx);
  if (M <= 0 || N <= 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_bias_grad_f32_noalloc: bad shape M=%d N=%d", M, N);
  if (N > kNoAllocMaxN)
    return vtlb_fail(ctx, VTLB_EINVAL,
                     "vtlb_bias_grad_f32_noalloc: N=%d exceeds the fixed scratch (at most %d "
                     "columns); use vtlb_linear_bwd_f32, which allocates",
                     N, kNoAllocMaxN);
  if (!d_G || !d_db) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_bias_grad_f32_noalloc: null pointer");
  if (ctx->device < 0 || ctx->device >= 64)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_bias_grad_f32_noalloc: device index %d not supported", ctx->device);
  double* scratch = g_bias_grad_scratch_addr[ctx->device].load(std::memory_order_relaxed);
  if (!scratch) {  // first call on this device: resolve the array's device address
    void* p = nullptr;
    VTLB_CUDA(ctx, cudaGetSymbolAddress(&p, g_bias_grad_scratch));
    scratch = (double*)p;
    g_bias_grad_scratch_addr[ctx->device].store(scratch, std::memory_order_relaxed);
  }
  int S = (M + 63) / 64;
  if (S > kNoAllocMaxS) S = kNoAllocMaxS;
  // every partial[s][n] with s < S, n < N is written by the first kernel before the second
  // reads it, so nothing left over from an earlier call is ever used and nothing needs clearing
  dim3 grid((N + 127) / 128, S);
  colsum_partial_kernel<<<grid, 128, 0, ctx->stream>>>((const float*)d_G, M, N, scratch);
  VTLB_LAUNCHED(ctx);
  colsum_final_kernel<<<(N + 127) / 128, 128, 0, ctx->stream>>>(scratch, S, N, (float*)d_db);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}
