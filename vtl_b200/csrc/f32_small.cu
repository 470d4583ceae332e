// Small f32 GEMMs on CUDA cores.  A Linear layer of the size of baseline config 1
// (64 x 256 x 784 and smaller) is a few tens of MFLOP: a 128-row tensor-core tile would be
// mostly padding, the operand-split passes would cost more than the product, and the whole
// call is bound by latency, not arithmetic.  Such products run here as a tiled FFMA kernel
// straight from the caller's row-major operands (either may be transposed), with the same
// fused epilogue (bias, pre-activation copy, ReLU).  Because a CTA that walks a long K loop
// pays one global-memory latency per step, K is cut into ranges that run as separate CTAs
// (grid.z).  With up to 8 ranges the CTAs of a tile form a thread-block cluster: row m of the
// tile belongs to CTA m % S, every CTA sends its partial rows to their owners' shared memory
// (st.shared::cluster), the cluster meets at a barrier and the owners add the partial sums in
// range order and apply the epilogue -- one launch.  With more ranges the partial sums go
// through global memory and a second tiny kernel adds them, in the same order.
// f32 FMA accumulation differs from the reference's f64 accumulation by
// ~sqrt(K) * 2^-24 relative, two orders inside the 1e-5 * sqrt(K) * max|A| * max|B| bound.
#include <stdlib.h>

#include "f32_common.cuh"

namespace {

constexpr int TM = 32, TN = 64, TK = 32;

// `mask` (shaped like C): the result is zeroed where mask is negative -- the backward of the ReLU
// whose cached input mask is, applied to a dX product on its way out (nn/internal/activation.v:78-87).
__device__ __forceinline__ void small_epilogue(float o, int m, int n, int N, const float* bias, float* pre,
                                               int relu, float* C, const float* mask) {
  if (bias) o = __fadd_rn(o, bias[n]);
  if (pre) pre[(size_t)m * N + n] = o;
  if (relu && o < 0.f) o = 0.f;
  if (mask && __ldg(mask + (size_t)m * N + n) < 0.f) o = 0.f;
  C[(size_t)m * N + n] = o;
}

constexpr int NST = 4;                                           // stages of the operand ring
constexpr int kStageFloats = TK * (TM + 1) + TK * (TN + 4);      // 3232 floats: the B tile starts 16-byte aligned
constexpr int kStageBytes = NST * kStageFloats * (int)sizeof(float);
constexpr int kMaxClusterSplits = 8;
constexpr int kLandRows = 36;  // max over S = 2..8 of S * ceil(TM / S)

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 4-byte asynchronous copy global -> shared; with ok == false nothing is read and zero is written
__device__ __forceinline__ void cp_async_f32(uint32_t dst, const float* src, bool ok) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(ok ? 4 : 0) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// grid = (tiles_n, tiles_m, splits).  With splits == 1 the epilogue is applied here and C is
// written.  With `cluster` set the launch has cluster dimensions (1, 1, splits) and the partial
// sums are exchanged through shared memory; otherwise they go to partial[z][M][N].
template <bool TA, bool TB>
__global__ void __launch_bounds__(256) sgemm_small_kernel(const float* __restrict__ A,
                                                          const float* __restrict__ B,
                                                          float* __restrict__ C,
                                                          const float* __restrict__ bias,
                                                          float* __restrict__ pre, int M, int N, int K,
                                                          int k_per_split, int relu,
                                                          float* __restrict__ partial, int cluster,
                                                          float* __restrict__ a_rowsum,
                                                          const float* __restrict__ mask) {
  // NST stages of (A tile [TK][TM+1], B tile [TK][TN+4]) in dynamic shared memory, filled by
  // cp.async: the loads of up to NST K steps (a whole K range) are in flight at once, so
  // a CTA pays one global-memory latency, not one per step
  extern __shared__ __align__(16) float stage_mem[];
  // landing zone of the cluster exchange: [source CTA][owned row][TN]; written by the peers
  // while this CTA may still be in its K loop, so it shares nothing with the stages
  __shared__ __align__(16) float Land[kLandRows][TN];
  // "this CTA runs": entered here, waited for before the first store into a peer's memory
  if (cluster) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  // Launched with programmatic stream serialisation: the CTAs may be resident before the kernel
  // in front of this one in the stream has finished (its launch latency hidden behind that
  // kernel's tail); nothing of that kernel's output is touched before this wait, which returns
  // once it has completed and its writes are visible.  Then let the next kernel do the same.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;  // 16 x 16 threads, 2 x 4 outputs each
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int kbeg = blockIdx.z * k_per_split;
  const int kend = kbeg + k_per_split < K ? kbeg + k_per_split : K;
  const int nsteps = kend > kbeg ? (kend - kbeg + TK - 1) / TK : 0;
  auto load_stage = [&](int st, int k0) {
    float* as = stage_mem + st * kStageFloats;
    float* bs = as + TK * (TM + 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // A tile 32 x 32; index order follows the contiguous dimension
      const int e = tid + i * 256;
      const int m = TA ? (e & 31) : (e >> 5), k = TA ? (e >> 5) : (e & 31);
      const int gm = m0 + m, gk = k0 + k;
      const bool ok = gm < M && gk < kend;
      const float* src = ok ? (TA ? A + (size_t)gk * M + gm : A + (size_t)gm * K + gk) : A;
      cp_async_f32(smem_addr(as + k * (TM + 1) + m), src, ok);  // zero-filled outside the operand
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // B tile 32 x 64
      const int e = tid + i * 256;
      const int n = TB ? (e >> 5) : (e & 63), k = TB ? (e & 31) : (e >> 6);
      const int gn = n0 + n, gk = k0 + k;
      const bool ok = gn < N && gk < kend;
      const float* src = ok ? (TB ? B + (size_t)gn * K + gk : B + (size_t)gk * N + gn) : B;
      cp_async_f32(smem_addr(bs + k * (TN + 4) + n), src, ok);
    }
  };
  // one commit group per K step, empty ones included, so that "all but the newest NST-1 groups
  // are complete" always means "step s has landed"
#pragma unroll
  for (int st = 0; st < NST; ++st) {
    if (st < nsteps) load_stage(st, kbeg + st * TK);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  // Optional by-product (unsplit launches only): a_rowsum[m] = sum over k of A(m, k), summed in
  // f64 and rounded once.  For dW = G^T . X these are the column sums of G, the bias gradient,
  // which would otherwise cost a launch of its own; the first column of tiles computes them from
  // the A tiles it loads anyway.
  const bool want_sum = a_rowsum != nullptr && blockIdx.x == 0;
  double rsum0 = 0.0, rsum1 = 0.0;
  for (int s = 0; s < nsteps; ++s) {
    asm volatile("cp.async.wait_group %0;" ::"n"(NST - 1) : "memory");
    __syncthreads();
    const float* as = stage_mem + (s % NST) * kStageFloats;
    const float* bs = as + TK * (TM + 1);
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      const float a0 = as[kk * (TM + 1) + ty * 2], a1 = as[kk * (TM + 1) + ty * 2 + 1];
      const float4 b = *reinterpret_cast<const float4*>(bs + kk * (TN + 4) + tx * 4);
      acc[0][0] = fmaf(a0, b.x, acc[0][0]);
      acc[0][1] = fmaf(a0, b.y, acc[0][1]);
      acc[0][2] = fmaf(a0, b.z, acc[0][2]);
      acc[0][3] = fmaf(a0, b.w, acc[0][3]);
      acc[1][0] = fmaf(a1, b.x, acc[1][0]);
      acc[1][1] = fmaf(a1, b.y, acc[1][1]);
      acc[1][2] = fmaf(a1, b.z, acc[1][2]);
      acc[1][3] = fmaf(a1, b.w, acc[1][3]);
      if (want_sum) {
        rsum0 += (double)a0;
        rsum1 += (double)a1;
      }
    }
    __syncthreads();
    if (s + NST < nsteps) load_stage(s % NST, kbeg + (s + NST) * TK);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  if (want_sum && tx == 0) {
    if (m0 + ty * 2 < M) a_rowsum[m0 + ty * 2] = (float)rsum0;
    if (m0 + ty * 2 + 1 < M) a_rowsum[m0 + ty * 2 + 1] = (float)rsum1;
  }
  if (cluster) {
    const int S = gridDim.z;
    const int z = (int)cluster_rank();  // = blockIdx.z: the cluster spans the whole z extent of the grid
    const int rows_per = (TM + S - 1) / S;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every peer has started
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int m = ty * 2 + r;  // row of the tile: owner m % S keeps it as its row m / S
      const uint32_t dst = map_to_rank(smem_addr(&Land[(int)blockIdx.z * rows_per + m / S][tx * 4]), (uint32_t)(m % S));
      st_cluster_v4(dst, acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    // this CTA's rows: partial sums added in range order, like small_reduce_kernel
    for (int e = tid; e < rows_per * TN; e += 256) {
      const int slot = e / TN, nl = e % TN;
      const int ml = slot * S + z;
      const int m = m0 + ml, n = n0 + nl;
      if (ml >= TM || m >= M || n >= N) continue;
      float s0 = Land[slot][nl];
      for (int r = 1; r < S; ++r) s0 = __fadd_rn(s0, Land[r * rows_per + slot][nl]);
      small_epilogue(s0, m, n, N, bias, pre, relu, C, mask);
    }
    return;
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
        small_epilogue(acc[r][j], m, n, N, bias, pre, relu, C, mask);
    }
  }
}

__global__ void __launch_bounds__(256) small_reduce_kernel(const float* __restrict__ partial, int splits,
                                                           int M, int N, const float* __restrict__ bias,
                                                           float* __restrict__ pre, int relu,
                                                           float* __restrict__ C, const float* __restrict__ mask) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a small GEMM behind this one may start early
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  float s = partial[i];
  for (int z = 1; z < splits; ++z) s = __fadd_rn(s, partial[(size_t)z * M * N + i]);
  small_epilogue(s, i / N, i % N, N, bias, pre, relu, C, mask);
}

}  // namespace

int f32::sgemm_small(vtlb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A,
                     const float* B, float* C, const float* bias, int relu, float* pre, float* a_rowsum,
                     bool* rowsum_done, const float* mask) {
  const int tiles = ((N + TN - 1) / TN) * ((M + TM - 1) / TM);
  // K ranges of `kps_want` (VTLB_SMALL_KPS overrides): the product is spread over as many SMs as
  // the cluster limit of 8 ranges allows, since a CTA that walks a long K alone is bound by its own
  // shared-memory reads (measured on config 1: no split 100 us per step, ranges of 256 80 us, of 128 74 us, of 64 67.5 us)
  static int kps_want = -1;
  if (kps_want < 0) {
    const char* e = getenv("VTLB_SMALL_KPS");
    kps_want = e ? atoi(e) : 64;
    if (kps_want < 32) kps_want = 32;
  }
  int splits = (K + kps_want - 1) / kps_want;
  while (splits > 1 && tiles * splits > 4 * ctx->sm_count) --splits;
  int kps = (K + splits - 1) / splits;
  kps = (kps + TK - 1) / TK * TK;
  splits = (K + kps - 1) / kps;
  // A few ranges more than a cluster holds (config 1's first layer: K = 784 = 13 ranges of 64) go
  // through the partial buffer and a second launch.  VTLB_SMALL_CLUSTER_CAP=1 makes the ranges long
  // enough to fit one cluster instead, which saves that launch and measured slower (config 1: 46.6
  // against 46.1 us per step -- the longer K walk costs more than the early-launched reduction).
  static int cap = -1;
  if (cap < 0) {
    const char* e = getenv("VTLB_SMALL_CLUSTER_CAP");
    cap = e ? atoi(e) != 0 : 0;
  }
  if (cap && splits > kMaxClusterSplits && splits <= 2 * kMaxClusterSplits) {
    kps = ((K + kMaxClusterSplits - 1) / kMaxClusterSplits + TK - 1) / TK * TK;
    splits = (K + kps - 1) / kps;
  }
  const bool cluster = splits > 1 && splits <= kMaxClusterSplits;
  if (splits > 1) a_rowsum = nullptr;  // the by-product needs the whole K in one CTA
  if (rowsum_done) *rowsum_done = a_rowsum != nullptr;
  float* partial = nullptr;
  if (splits > 1 && !cluster) {
    void* scr = nullptr;
    int rc = vtlb_scratch(ctx, (size_t)splits * M * N * sizeof(float), &scr);
    if (rc) return rc;
    partial = (float*)scr;
  }
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM, splits);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = kStageBytes;
  cfg.stream = ctx->stream;
  static std::atomic<uint64_t> configured{0};  // one bit per device
  if (!(configured.load(std::memory_order_relaxed) >> (ctx->device & 63) & 1)) {
    VTLB_CUDA(ctx, cudaFuncSetAttribute(sgemm_small_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes));
    VTLB_CUDA(ctx, cudaFuncSetAttribute(sgemm_small_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes));
    VTLB_CUDA(ctx, cudaFuncSetAttribute(sgemm_small_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes));
    VTLB_CUDA(ctx, cudaFuncSetAttribute(sgemm_small_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStageBytes));
    configured.fetch_or(1ull << (ctx->device & 63), std::memory_order_relaxed);
  }
  static int pdl = -1;  // VTLB_SMALL_PDL=0 switches the early launch off (measurements)
  if (pdl < 0) {
    const char* e = getenv("VTLB_SMALL_PDL");
    pdl = e ? atoi(e) != 0 : 1;
  }
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 1;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = (unsigned)(cluster ? splits : 1);
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 2 : 1;
#define VTLB_SMALL(TA, TB)                                                                               \
  VTLB_CUDA(ctx, cudaLaunchKernelEx(&cfg, sgemm_small_kernel<TA, TB>, A, B, C, bias, pre, M, N, K, kps, relu, \
                                    partial, (int)cluster, a_rowsum, mask))
  if (transA && transB) VTLB_SMALL(true, true);
  else if (transA) VTLB_SMALL(true, false);
  else if (transB) VTLB_SMALL(false, true);
  else VTLB_SMALL(false, false);
#undef VTLB_SMALL
  VTLB_LAUNCHED(ctx);
  if (splits > 1 && !cluster) {
    VTLB_CUDA(ctx, vtlb_launch_early(small_reduce_kernel, dim3((M * N + 255) / 256), dim3(256), 0, ctx->stream,
                                     (const float*)partial, splits, M, N, bias, pre, relu, C, mask));
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
