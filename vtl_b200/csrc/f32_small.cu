// Small f32 GEMMs on CUDA cores.  A Linear layer of the size of baseline config 1
// (64 x 256 x 784 and smaller) is a few tens of MFLOP: a 128-row tensor-core tile would be
// mostly padding, the operand-split passes would cost more than the product, and the whole
// call is bound by latency, not arithmetic.  Such products run here as a tiled FFMA kernel
// straight from the caller's row-major operands (either may be transposed), with the same
// fused epilogue (bias, pre-activation copy, ReLU).  Because a CTA that walks a long K loop
// pays one global-memory latency per step, K is cut into ranges that run as separate CTAs
// (grid.z) and a second tiny kernel adds the partial sums in a fixed order and applies the
// epilogue.  f32 FMA accumulation differs from the reference's f64 accumulation by
// ~sqrt(K) * 2^-24 relative, two orders inside the 1e-5 * sqrt(K) * max|A| * max|B| bound.
#include "f32_common.cuh"

namespace {

constexpr int TM = 32, TN = 64, TK = 32;

__device__ __forceinline__ void small_epilogue(float o, int m, int n, int N, const float* bias, float* pre,
                                               int relu, float* C) {
  if (bias) o = __fadd_rn(o, bias[n]);
  if (pre) pre[(size_t)m * N + n] = o;
  if (relu && o < 0.f) o = 0.f;
  C[(size_t)m * N + n] = o;
}

// grid = (tiles_n, tiles_m, splits).  With splits == 1 the epilogue is applied here and C is
// written; otherwise the raw partial sums go to partial[z][M][N].
template <bool TA, bool TB>
__global__ void __launch_bounds__(256) sgemm_small_kernel(const float* __restrict__ A,
                                                          const float* __restrict__ B,
                                                          float* __restrict__ C,
                                                          const float* __restrict__ bias,
                                                          float* __restrict__ pre, int M, int N, int K,
                                                          int k_per_split, int relu,
                                                          float* __restrict__ partial) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;  // 16 x 16 threads, 2 x 4 outputs each
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int kbeg = blockIdx.z * k_per_split;
  const int kend = kbeg + k_per_split < K ? kbeg + k_per_split : K;
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  for (int k0 = kbeg; k0 < kend; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // A tile 32 x 32; index order follows the contiguous dimension
      const int e = tid + i * 256;
      const int m = TA ? (e & 31) : (e >> 5), k = TA ? (e >> 5) : (e & 31);
      const int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < kend) v = TA ? A[(size_t)gk * M + gm] : A[(size_t)gm * K + gk];
      As[k][m] = v;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // B tile 32 x 64
      const int e = tid + i * 256;
      const int n = TB ? (e >> 5) : (e & 63), k = TB ? (e & 31) : (e >> 6);
      const int gn = n0 + n, gk = k0 + k;
      float v = 0.f;
      if (gn < N && gk < kend) v = TB ? B[(size_t)gn * K + gk] : B[(size_t)gk * N + gn];
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
      const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      acc[0][0] = fmaf(a0, b.x, acc[0][0]);
      acc[0][1] = fmaf(a0, b.y, acc[0][1]);
      acc[0][2] = fmaf(a0, b.z, acc[0][2]);
      acc[0][3] = fmaf(a0, b.w, acc[0][3]);
      acc[1][0] = fmaf(a1, b.x, acc[1][0]);
      acc[1][1] = fmaf(a1, b.y, acc[1][1]);
      acc[1][2] = fmaf(a1, b.z, acc[1][2]);
      acc[1][3] = fmaf(a1, b.w, acc[1][3]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int m = m0 + ty * 2 + r;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if (partial)
        partial[((size_t)blockIdx.z * M + m) * N + n] = acc[r][j];
      else
        small_epilogue(acc[r][j], m, n, N, bias, pre, relu, C);
    }
  }
}

__global__ void __launch_bounds__(256) small_reduce_kernel(const float* __restrict__ partial, int splits,
                                                           int M, int N, const float* __restrict__ bias,
                                                           float* __restrict__ pre, int relu,
                                                           float* __restrict__ C) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  float s = partial[i];
  for (int z = 1; z < splits; ++z) s = __fadd_rn(s, partial[(size_t)z * M * N + i]);
  small_epilogue(s, i / N, i % N, N, bias, pre, relu, C);
}

}  // namespace

int f32::sgemm_small(vtlb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A,
                     const float* B, float* C, const float* bias, int relu, float* pre) {
  const int tiles = ((N + TN - 1) / TN) * ((M + TM - 1) / TM);
  int splits = (K + 127) / 128;  // at most four 32-wide steps per CTA
  while (splits > 1 && tiles * splits > 4 * ctx->sm_count) --splits;
  int kps = (K + splits - 1) / splits;
  kps = (kps + TK - 1) / TK * TK;
  splits = (K + kps - 1) / kps;
  float* partial = nullptr;
  if (splits > 1) {
    void* scr = nullptr;
    int rc = vtlb_scratch(ctx, (size_t)splits * M * N * sizeof(float), &scr);
    if (rc) return rc;
    partial = (float*)scr;
  }
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, splits);
#define VTLB_SMALL(TA, TB)                                                                              \
  sgemm_small_kernel<TA, TB><<<grid, 256, 0, ctx->stream>>>(A, B, C, bias, pre, M, N, K, kps, relu, partial)
  if (transA && transB) VTLB_SMALL(true, true);
  else if (transA) VTLB_SMALL(true, false);
  else if (transB) VTLB_SMALL(false, true);
  else VTLB_SMALL(false, false);
#undef VTLB_SMALL
  VTLB_LAUNCHED(ctx);
  if (splits > 1) {
    small_reduce_kernel<<<(M * N + 255) / 256, 256, 0, ctx->stream>>>(partial, splits, M, N, bias, pre, relu, C);
    VTLB_LAUNCHED(ctx);
  }
  return VTLB_OK;
}

VTLB_API int vtlb_set_small_gemm_limit(vtlb_ctx* ctx, double max_flops) {
  VTLB_ENTER(ctx);
  if (max_flops < 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_set_small_gemm_limit: negative limit");
  ctx->small_gemm_flops = max_flops;
  return VTLB_OK;
}
