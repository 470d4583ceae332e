// Linear layers with few output features and many inputs (a classifier head: 16384 -> 10 in baseline
// config 3), forward and backward, as memory-bound CUDA-core kernels.
//
// Such a layer is a few tens of MFLOP over tens of megabytes: Y = X.W^T + b reads X once, dX = G.W
// writes one matrix of X's size, dW = G^T.X reads X once.  The tiled small-GEMM kernel (f32_small.cu)
// cuts it into thousands of tiny tiles and K ranges that meet in clusters and takes 20-45 us per
// product; a 128-row tensor-core tile would be padding in every column but ten.  Here every product
// streams the long operand exactly once with 16-byte accesses, keeps the narrow operand in registers or
// L2, and adds partial sums in a fixed order (no atomics: results are reproducible):
//   forward   CTA = 4 rows x a K chunk of 2048; 4*N running sums per thread, reduced over the CTA,
//             partial[chunk][m][n]; a second launch adds the chunks in order and applies bias / ReLU
//   dX        one thread per four consecutive k: 4*N FMAs from g[m][0..N) and w[n][k..k+3]
//   dW, db    CTA = 16 rows x 1024 k; N*4 running sums per thread; partial[range][n][k]; the second
//             launch adds the ranges in order (and sums the columns of G for db)
// f32 FMA accumulation, like the small-GEMM kernel: sqrt(K) * 2^-24 relative, two orders inside the
// 1e-5 * sqrt(K) * max|A| * max|B| bound.  All kernels wait with griddepcontrol.wait before their
// first access (they are launched early behind the kernel in front).
#include "f32_common.cuh"

namespace {

constexpr int MAXN = 16;          // output features at most
constexpr int FWD_ROWS = 4, FWD_KCHUNK = 2048;
constexpr int DW_ROWS = 16, DW_KCHUNK = 1024;

__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// partial[chunk][m][n] = sum over k in the chunk of x[m][k] * w[n][k]
template <int N>
__global__ void __launch_bounds__(256) narrow_fwd_partial_kernel(const float* __restrict__ X, const float* __restrict__ W,
                                                                 int M, int K, float* __restrict__ partial) {
  pdl_wait();
  __shared__ float red[8][FWD_ROWS * N];
  const int m0 = blockIdx.x * FWD_ROWS, k0 = blockIdx.y * FWD_KCHUNK;
  const int k1 = k0 + FWD_KCHUNK < K ? k0 + FWD_KCHUNK : K;
  float acc[FWD_ROWS][N];
#pragma unroll
  for (int r = 0; r < FWD_ROWS; ++r)
#pragma unroll
    for (int n = 0; n < N; ++n) acc[r][n] = 0.0f;
  for (int k = k0 + threadIdx.x * 4; k < k1; k += 256 * 4) {  // K % 4 == 0: whole float4 pieces
    float4 x[FWD_ROWS];
#pragma unroll
    for (int r = 0; r < FWD_ROWS; ++r)
      x[r] = m0 + r < M ? __ldg(reinterpret_cast<const float4*>(X + (size_t)(m0 + r) * K + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int n = 0; n < N; ++n) {
      const float4 w = __ldg(reinterpret_cast<const float4*>(W + (size_t)n * K + k));
#pragma unroll
      for (int r = 0; r < FWD_ROWS; ++r) {
        acc[r][n] = fmaf(x[r].x, w.x, acc[r][n]);
        acc[r][n] = fmaf(x[r].y, w.y, acc[r][n]);
        acc[r][n] = fmaf(x[r].z, w.z, acc[r][n]);
        acc[r][n] = fmaf(x[r].w, w.w, acc[r][n]);
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < FWD_ROWS; ++r)
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float v = acc[r][n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (lane == 0) red[warp][r * N + n] = v;
    }
  __syncthreads();
  if (threadIdx.x < FWD_ROWS * N) {
    float s = red[0][threadIdx.x];
#pragma unroll
    for (int w = 1; w < 8; ++w) s = __fadd_rn(s, red[w][threadIdx.x]);
    const int r = threadIdx.x / N, n = threadIdx.x - r * N;
    if (m0 + r < M) partial[((size_t)blockIdx.y * M + m0 + r) * N + n] = s;
  }
}

// y[m][n] = sum over chunks (ascending) + bias, pre-activation copy, ReLU
__global__ void __launch_bounds__(256) narrow_fwd_final_kernel(const float* __restrict__ partial, int chunks, int M, int N,
                                                               const float* __restrict__ bias, float* __restrict__ pre,
                                                               int relu, float* __restrict__ Y) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  float s = partial[i];
  for (int c = 1; c < chunks; ++c) s = __fadd_rn(s, partial[(size_t)c * M * N + i]);
  if (bias) s = __fadd_rn(s, bias[i % N]);
  if (pre) pre[i] = s;
  Y[i] = relu && s < 0.f ? 0.f : s;
}

// dx[m][k..k+3] = sum over n of g[m][n] * w[n][k..k+3]
template <int N>
__global__ void __launch_bounds__(256) narrow_dx_kernel(const float* __restrict__ G, const float* __restrict__ W, int M,
                                                        int K, float* __restrict__ dX) {
  pdl_wait();
  const int k = (blockIdx.x * 256 + threadIdx.x) * 4;
  if (k >= K) return;
  float4 w[N];
#pragma unroll
  for (int n = 0; n < N; ++n) w[n] = __ldg(reinterpret_cast<const float4*>(W + (size_t)n * K + k));
  for (int m = blockIdx.y; m < M; m += gridDim.y) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int n = 0; n < N; ++n) {
      const float g = __ldg(G + (size_t)m * N + n);
      o.x = fmaf(g, w[n].x, o.x);
      o.y = fmaf(g, w[n].y, o.y);
      o.z = fmaf(g, w[n].z, o.z);
      o.w = fmaf(g, w[n].w, o.w);
    }
    *reinterpret_cast<float4*>(dX + (size_t)m * K + k) = o;
  }
}

// partial[range][n][k] = sum over the range's rows m of g[m][n] * x[m][k]
template <int N>
__global__ void __launch_bounds__(256) narrow_dw_partial_kernel(const float* __restrict__ G, const float* __restrict__ X,
                                                                int M, int K, float* __restrict__ partial) {
  pdl_wait();
  __shared__ float gs[DW_ROWS][N];
  const int m0 = blockIdx.y * DW_ROWS;
  for (int i = threadIdx.x; i < DW_ROWS * N; i += 256) {
    const int r = i / N, n = i - r * N;
    gs[r][n] = m0 + r < M ? G[(size_t)(m0 + r) * N + n] : 0.0f;
  }
  __syncthreads();
  const int k = blockIdx.x * DW_KCHUNK + threadIdx.x * 4;
  if (k >= K) return;
  float4 acc[N];
#pragma unroll
  for (int n = 0; n < N; ++n) acc[n] = make_float4(0.f, 0.f, 0.f, 0.f);
  const int rows = M - m0 < DW_ROWS ? M - m0 : DW_ROWS;
#pragma unroll 4
  for (int r = 0; r < rows; ++r) {
    const float4 x = __ldg(reinterpret_cast<const float4*>(X + (size_t)(m0 + r) * K + k));
#pragma unroll
    for (int n = 0; n < N; ++n) {
      const float g = gs[r][n];
      acc[n].x = fmaf(g, x.x, acc[n].x);
      acc[n].y = fmaf(g, x.y, acc[n].y);
      acc[n].z = fmaf(g, x.z, acc[n].z);
      acc[n].w = fmaf(g, x.w, acc[n].w);
    }
  }
#pragma unroll
  for (int n = 0; n < N; ++n)
    *reinterpret_cast<float4*>(partial + ((size_t)blockIdx.y * N + n) * K + k) = acc[n];
}

// dW[n][k] = sum over ranges (ascending); the last CTA row also writes db[n] = sum over m of g[m][n]
// (f64, rows in order)
__global__ void __launch_bounds__(256) narrow_dw_final_kernel(const float* __restrict__ partial, int ranges, int N, int K,
                                                              float* __restrict__ dW, const float* __restrict__ G, int M,
                                                              float* __restrict__ db) {
  pdl_wait();
  const size_t n_el = (size_t)N * K;
  const size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 4;
  if (dW && i < n_el) {
    float4 s = *reinterpret_cast<const float4*>(partial + i);
    for (int r = 1; r < ranges; ++r) {
      const float4 p = *reinterpret_cast<const float4*>(partial + (size_t)r * n_el + i);
      s.x = __fadd_rn(s.x, p.x);
      s.y = __fadd_rn(s.y, p.y);
      s.z = __fadd_rn(s.z, p.z);
      s.w = __fadd_rn(s.w, p.w);
    }
    *reinterpret_cast<float4*>(dW + i) = s;
  }
  if (db && blockIdx.x == gridDim.x - 1 && threadIdx.x < N) {
    double s = 0.0;
    for (int m = 0; m < M; ++m) s += (double)G[(size_t)m * N + threadIdx.x];
    db[threadIdx.x] = (float)s;
  }
}

template <int N>
int run_fwd(vtlb_ctx* ctx, const float* X, const float* W, const float* bias, float* Y, int M, int K, int relu,
            float* pre) {
  const int chunks = (K + FWD_KCHUNK - 1) / FWD_KCHUNK;
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, (size_t)chunks * M * N * sizeof(float), &scr);
  if (rc) return rc;
  VTLB_CUDA(ctx, vtlb_launch_early(narrow_fwd_partial_kernel<N>, dim3((M + FWD_ROWS - 1) / FWD_ROWS, chunks), dim3(256), 0,
                                   ctx->stream, X, W, M, K, (float*)scr));
  VTLB_LAUNCHED(ctx);
  VTLB_CUDA(ctx, vtlb_launch_early(narrow_fwd_final_kernel, dim3((M * N + 255) / 256), dim3(256), 0, ctx->stream,
                                   (const float*)scr, chunks, M, N, bias, pre, relu, Y));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

template <int N>
int run_dx(vtlb_ctx* ctx, const float* G, const float* W, float* dX, int M, int K) {
  int gy = M < 64 ? M : 64;
  VTLB_CUDA(ctx, vtlb_launch_early(narrow_dx_kernel<N>, dim3((K / 4 + 255) / 256, gy), dim3(256), 0, ctx->stream, G, W, M,
                                   K, dX));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

template <int N>
int run_dw(vtlb_ctx* ctx, const float* G, const float* X, float* dW, float* db, int M, int K) {
  const int ranges = (M + DW_ROWS - 1) / DW_ROWS;
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, (size_t)ranges * N * K * sizeof(float), &scr);
  if (rc) return rc;
  if (dW) {
    VTLB_CUDA(ctx, vtlb_launch_early(narrow_dw_partial_kernel<N>, dim3((K + DW_KCHUNK - 1) / DW_KCHUNK, ranges), dim3(256),
                                     0, ctx->stream, G, X, M, K, (float*)scr));
    VTLB_LAUNCHED(ctx);
  }
  VTLB_CUDA(ctx, vtlb_launch_early(narrow_dw_final_kernel, dim3((unsigned)(((size_t)N * K / 4 + 255) / 256)), dim3(256), 0,
                                   ctx->stream, (const float*)scr, ranges, N, K, dW, G, M, db));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace

// A Linear layer with at most 16 output features, at least 2048 inputs (a multiple of 4) and
// 16-byte-aligned operands takes these kernels.
bool f32::narrow_linear_ok(int M, int N, int K, const void* a, const void* b, const void* c) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("VTLB_NARROW_LINEAR");
    env = e ? atoi(e) : 1;
  }
  return env && M >= 1 && N >= 1 && N <= MAXN && K >= 2048 && (K & 3) == 0 && vtlb_aligned16(a) && vtlb_aligned16(b) &&
         vtlb_aligned16(c) && (long long)M * K <= 0x7fffffffLL * 4;
}

int f32::narrow_linear_fwd(vtlb_ctx* ctx, const float* X, const float* W, const float* bias, float* Y, int M, int N, int K,
                           int relu, float* pre) {
  switch (N) {
#define VTLB_CASE(n) case n: return run_fwd<n>(ctx, X, W, bias, Y, M, K, relu, pre);
    VTLB_CASE(1) VTLB_CASE(2) VTLB_CASE(3) VTLB_CASE(4) VTLB_CASE(5) VTLB_CASE(6) VTLB_CASE(7) VTLB_CASE(8)
    VTLB_CASE(9) VTLB_CASE(10) VTLB_CASE(11) VTLB_CASE(12) VTLB_CASE(13) VTLB_CASE(14) VTLB_CASE(15) VTLB_CASE(16)
#undef VTLB_CASE
  }
  return vtlb_fail(ctx, VTLB_EINVAL, "narrow_linear_fwd: %d output features", N);
}

int f32::narrow_linear_dx(vtlb_ctx* ctx, const float* G, const float* W, float* dX, int M, int N, int K) {
  switch (N) {
#define VTLB_CASE(n) case n: return run_dx<n>(ctx, G, W, dX, M, K);
    VTLB_CASE(1) VTLB_CASE(2) VTLB_CASE(3) VTLB_CASE(4) VTLB_CASE(5) VTLB_CASE(6) VTLB_CASE(7) VTLB_CASE(8)
    VTLB_CASE(9) VTLB_CASE(10) VTLB_CASE(11) VTLB_CASE(12) VTLB_CASE(13) VTLB_CASE(14) VTLB_CASE(15) VTLB_CASE(16)
#undef VTLB_CASE
  }
  return vtlb_fail(ctx, VTLB_EINVAL, "narrow_linear_dx: %d output features", N);
}

int f32::narrow_linear_dw(vtlb_ctx* ctx, const float* G, const float* X, float* dW, float* db, int M, int N, int K) {
  switch (N) {
#define VTLB_CASE(n) case n: return run_dw<n>(ctx, G, X, dW, db, M, K);
    VTLB_CASE(1) VTLB_CASE(2) VTLB_CASE(3) VTLB_CASE(4) VTLB_CASE(5) VTLB_CASE(6) VTLB_CASE(7) VTLB_CASE(8)
    VTLB_CASE(9) VTLB_CASE(10) VTLB_CASE(11) VTLB_CASE(12) VTLB_CASE(13) VTLB_CASE(14) VTLB_CASE(15) VTLB_CASE(16)
#undef VTLB_CASE
  }
  return vtlb_fail(ctx, VTLB_EINVAL, "narrow_linear_dw: %d output features", N);
}
