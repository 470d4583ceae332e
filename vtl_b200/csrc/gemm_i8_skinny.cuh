// INT8 GEMM for few activation rows (M <= 128): Y[M,N] = A[M,K] . W[N,K]^T.
//
// The general kernel (gemm_tc.cuh) puts the M rows into a 128-row tile, most of it padding,
// and a tile streams all of K through ONE SM; an SM takes in about 54 bytes per clock, so a
// 4096-deep tile costs 8 us however few rows there are.  Here the operands change places and
// K is cut across a thread-block cluster:
//   * a tile is 128 output channels (rows of W = the M side of the MMA, one TMEM lane each)
//     by MN = 16/32/64/128 activation rows (the N side), so the bytes a CTA pulls are almost
//     all weights, each read once;
//   * the S CTAs of a cluster (1, 2 or 4) take K ranges of the same tile, so S times as many
//     SMs stream the weights; CTA r finishes the rows m = r (mod S), so every CTA sends each
//     row of its int32 partial sums to the landing zone of the row's owner (st.shared::cluster,
//     a warp writing 128 contiguous bytes), the cluster meets at a barrier, and the owner
//     adds the S partials from its own shared memory (integer sums: exact in any order) and
//     applies the epilogue, a warp writing 512 contiguous bytes of a row of Y.  Nobody reads a
//     peer's memory after the barrier, so a CTA may leave as soon as it is done; the barrier
//     that guarantees every peer has started before it is written to is entered at the top
//     and only waited for after the K loop.
// One tile per CTA (grid = tiles * S); warp 0 = TMA producer, warp 1 = MMA issuer and owner
// of the tensor memory, warps 2..5 = epilogue.  Waits are bounded as in gemm_tc.cuh and both
// cluster barriers are reached on every path.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"

namespace skinny {

constexpr int BNCH = 128;                      // output channels per tile = TMEM lanes
constexpr uint32_t W_TILE = BNCH * 128;        // 16 KB of weights per stage
constexpr uint32_t RING_BYTES = 128 * 1024;    // operand ring
constexpr uint32_t LZ_BYTES = 64 * 1024;       // landing zone: [source CTA][owned row][128 channels] int32
constexpr int MAX_STAGES = 8;
constexpr int NUM_THREADS = 192;
constexpr uint32_t BARS_OFF = RING_BYTES + LZ_BYTES;
constexpr uint32_t SMEM_TOTAL = BARS_OFF + 8 * (2 * MAX_STAGES + 1) + 16 + 1024;

struct Params {
  CUtensorMap w;     // W codes [N, K], box 128 rows x 128 bytes
  CUtensorMap a;     // A codes [M, K], box MN rows x 128 bytes
  int M, N, K, MN;
  float* Y;          // fused: f32 output [M, N]
  int32_t* acc;      // raw: int32 output [M, N]
  const float* sa;
  const float* sw;
  const float* bias;  // may be null
  int relu;
  int vec;           // rows of the output may be written 16 bytes at a time
  uint32_t* status;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ int4 ld_shared_v4(uint32_t addr) {
  int4 v;
  asm volatile("ld.shared.v4.s32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ float dequant(int acc, float sa, float sw, float bias, bool has_bias, int relu) {
  const float t = __fmul_rn(sa, sw);
  const float u = __fmul_rn(__int2float_rn(acc), t);
  float y = has_bias ? __fadd_rn(u, bias) : u;
  if (relu && y < 0.0f) y = 0.0f;
  return y;
}

template <bool FUSED, int S>
__global__ void __launch_bounds__(NUM_THREADS, 1) gemm_i8_skinny_kernel(const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // same offset in every CTA of the cluster
  const uint32_t bars = base + BARS_OFF;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  const uint32_t tfull_bar = bars + 8u * (2 * MAX_STAGES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars - raw) + 8u * (2 * MAX_STAGES + 1));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
  const uint32_t lz = base + RING_BYTES;
  const int tile = blockIdx.x / S;
  const int n0 = tile * BNCH;
  const int MN = p.MN;
  const uint32_t a_bytes = (uint32_t)MN * 128u;
  const uint32_t stride = W_TILE + a_bytes;
  const int stages = (int)(RING_BYTES / stride) < MAX_STAGES ? (int)(RING_BYTES / stride) : MAX_STAGES;
  const int total_kb = (p.K + 127) / 128;
  const int per = (total_kb + S - 1) / S;
  const int kb_begin = (int)rank * per;
  const int kb_end = kb_begin + per < total_kb ? kb_begin + per : total_kb;
  const bool has_work = kb_begin < kb_end;
  const uint32_t tmem_cols = MN < 32 ? 32u : (uint32_t)MN;  // 32, 64 or 128: powers of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tmap(&p.w);
    ptx::prefetch_tmap(&p.a);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // launched early (programmatic stream serialisation): the set-up above overlapped the tail of the
  // kernel in front; global memory is first touched after this wait
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // "this CTA runs": waited for (by then for nothing) before the first store into a peer's memory
  if (S > 1) cluster_arrive_relaxed();

  float4 w4 = make_float4(0.f, 0.f, 0.f, 0.f), b4 = w4;  // epilogue warps: weight scales and bias of 4 channels
  float sa_mine = 0.0f;                                   // and the scale of the lane-th row this warp finishes

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, gemm::WAIT_LIMIT_NS)) break;
        ptx::mbar_arrive_expect_tx(full_bar(stage), stride);
        const uint32_t sw = base + (uint32_t)stage * stride;
        ptx::tma_load_2d(sw, &p.w, kb * 128, n0, full_bar(stage));
        ptx::tma_load_2d(sw + W_TILE, &p.a, kb * 128, 0, full_bar(stage));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && has_work) {
      const uint32_t idesc = ptx::umma_idesc(ptx::kCfmtS32, ptx::kFmtS8, BNCH, (uint32_t)MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, gemm::WAIT_LIMIT_NS)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t sw = base + (uint32_t)stage * stride;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint64_t dw = ptx::umma_desc_k_sw128(sw) + 2u * kk;
          const uint64_t da = ptx::umma_desc_k_sw128(sw + W_TILE) + 2u * kk;
          ptx::umma_i8(tmem_base, dw, da, idesc, (kb == kb_begin && kk == 0) ? 0u : 1u);
        }
        ptx::umma_commit(empty_bar(stage));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) ptx::umma_commit(tfull_bar);  // fires once every MMA has read its operands and written TMEM
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue, part 1: park the partial sums
    const int q = warp & 3;  // TMEM lane quarter of this warp = channels q*32 .. q*32+31 of the tile
    // what part 2 needs from global memory is fetched now, behind the K loop
    if (FUSED) {
      const int n = n0 + lane * 4;
      const bool hb = p.bias != nullptr;
      if (p.vec && n + 3 < p.N) {
        w4 = __ldg(reinterpret_cast<const float4*>(p.sw + n));
        if (hb) b4 = __ldg(reinterpret_cast<const float4*>(p.bias + n));
      } else {
        if (n < p.N) { w4.x = __ldg(p.sw + n); if (hb) b4.x = __ldg(p.bias + n); }
        if (n + 1 < p.N) { w4.y = __ldg(p.sw + n + 1); if (hb) b4.y = __ldg(p.bias + n + 1); }
        if (n + 2 < p.N) { w4.z = __ldg(p.sw + n + 2); if (hb) b4.z = __ldg(p.bias + n + 2); }
        if (n + 3 < p.N) { w4.w = __ldg(p.sw + n + 3); if (hb) b4.w = __ldg(p.bias + n + 3); }
      }
      // row scales of the rows this warp finishes, one per lane: row rank + S*(warp-2) + 4*S*lane
      const int mrow = (int)rank + S * (warp - 2) + 4 * S * lane;
      sa_mine = mrow < p.M ? __ldg(p.sa + mrow) : 0.0f;
    }
    bool ok = true;
    if (has_work) {
      ok = ptx::mbar_wait_bounded(tfull_bar, 0, abort_flag, gemm::WAIT_LIMIT_NS);
      ok = __all_sync(0xffffffffu, ok);
      ptx::tc_fence_after();
    }
    // Row m belongs to CTA m % S, which keeps it as its row m / S; this CTA's copy goes to slot
    // [rank][m / S] of the owner's landing zone.  Lane = channel, so a warp's store is 128
    // contiguous bytes.  32 % S == 0: the owner of accumulator column j of a chunk is j % S.
    if (S > 1) cluster_wait();  // every peer has started (entered at the top of the kernel)
    const int rows_per = MN / S;  // slots per source CTA
    uint32_t dst[S];
#pragma unroll
    for (int o = 0; o < S; ++o)
      dst[o] = mapa(lz + (uint32_t)((int)rank * rows_per) * 512u + (uint32_t)(q * 32 + lane) * 4u, (uint32_t)o);
#pragma unroll 1
    for (int c = 0; c * 32 < p.M; ++c) {
      uint32_t v[32];
      if (has_work && ok) {
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c * 32u, v);
        ptx::tmem_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c * 32 + j < p.M) st_cluster_u32(dst[j % S] + (uint32_t)((c * 32 + j) / S) * 512u, v[j]);
    }
    ptx::tc_fence_before();
  }
  if (S > 1 && warp < 2) cluster_wait();  // the producer's and the MMA warp's half of the first barrier

  // every CTA's partial sums have reached their owners
  if (S > 1) cluster_sync_all();
  else __syncthreads();

  if (warp >= 2) {
    // ------------------------------------------------------------ epilogue, part 2: rows m = rank (mod S)
    const int n = n0 + lane * 4;
    const bool hb = p.bias != nullptr;
    auto finish = [&](int m, int4 s, float a) {
      const size_t off = (size_t)m * p.N + n;
      if (FUSED) {
        float4 y;
        y.x = dequant(s.x, a, w4.x, b4.x, hb, p.relu);
        y.y = dequant(s.y, a, w4.y, b4.y, hb, p.relu);
        y.z = dequant(s.z, a, w4.z, b4.z, hb, p.relu);
        y.w = dequant(s.w, a, w4.w, b4.w, hb, p.relu);
        if (p.vec && n + 3 < p.N) {
          *reinterpret_cast<float4*>(p.Y + off) = y;
        } else {
          if (n < p.N) p.Y[off] = y.x;
          if (n + 1 < p.N) p.Y[off + 1] = y.y;
          if (n + 2 < p.N) p.Y[off + 2] = y.z;
          if (n + 3 < p.N) p.Y[off + 3] = y.w;
        }
      } else {
        if (p.vec && n + 3 < p.N) {
          *reinterpret_cast<int4*>(p.acc + off) = s;
        } else {
          if (n < p.N) p.acc[off] = s.x;
          if (n + 1 < p.N) p.acc[off + 1] = s.y;
          if (n + 2 < p.N) p.acc[off + 2] = s.z;
          if (n + 3 < p.N) p.acc[off + 3] = s.w;
        }
      }
    };
    const int rows_per = MN / S;
    int i = 0;
    for (int l = warp - 2; l * S + (int)rank < p.M; l += 4, ++i) {  // l = owned row index
      const int m = l * S + (int)rank;
      const uint32_t mine = lz + (uint32_t)l * 512u + (uint32_t)lane * 16u;
      int4 t[S];
#pragma unroll
      for (int r = 0; r < S; ++r) t[r] = ld_shared_v4(mine + (uint32_t)(r * rows_per) * 512u);
      int4 s = t[0];
#pragma unroll
      for (int r = 1; r < S; ++r) {
        s.x += t[r].x; s.y += t[r].y; s.z += t[r].z; s.w += t[r].w;
      }
      finish(m, s, __shfl_sync(0xffffffffu, sa_mine, i & 31));
    }
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(p.status, VTLB_ST_GEMM_TIMEOUT);
    for (int i = 0; i < 100; ++i) __nanosleep(1000);  // bounded grace period for copies in flight
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------- host side
constexpr int kMaxM = 128;

// One wave of tiles: with more tiles than SMs the general kernel's wider tiles move fewer bytes.
inline bool usable(vtlb_ctx* ctx, int M, int N) {
  return M >= 1 && M <= kMaxM && N >= 1 && (N + BNCH - 1) / BNCH <= ctx->sm_count;
}

template <bool FUSED, int S>
int configure(vtlb_ctx* ctx, int* max_clusters) {
  auto kern = gemm_i8_skinny_kernel<FUSED, S>;
  VTLB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_TOTAL));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(ctx->sm_count / S * S));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_TOTAL;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  VTLB_CUDA(ctx, cudaOccupancyMaxActiveClusters(max_clusters, kern, &cfg));
  return VTLB_OK;
}

template <bool FUSED, int S>
int launch_s(vtlb_ctx* ctx, int tiles, const Params& p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * S));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM_TOTAL;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  VTLB_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemm_i8_skinny_kernel<FUSED, S>, p));
  return VTLB_OK;
}

// `p` arrives with the output pointers, scales, bias and relu filled in.
template <bool FUSED>
int launch(vtlb_ctx* ctx, const void* Aq, const void* Wq, int M, int N, int K, Params p) {
  static int max_clusters[64][3];  // per device: clusters of 1, 2, 4 CTAs resident at a time
  static std::atomic<uint64_t> configured{0};
  const int d = ctx->device & 63;
  if (!(configured.load(std::memory_order_relaxed) >> d & 1)) {
    int rc = configure<FUSED, 1>(ctx, &max_clusters[d][0]);
    if (!rc) rc = configure<FUSED, 2>(ctx, &max_clusters[d][1]);
    if (!rc) rc = configure<FUSED, 4>(ctx, &max_clusters[d][2]);
    if (rc) return rc;
    configured.fetch_or(1ull << d, std::memory_order_relaxed);
  }
  const int ldk = (K + 15) / 16 * 16;
  const int MN = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  const int tiles = (N + BNCH - 1) / BNCH;
  const int total_kb = (K + 127) / 128;
  // as many K ranges as still run in one wave (and leave every CTA at least two K blocks)
  int S = 1;
  for (int i = 2; i >= 1; --i)
    if (tiles <= max_clusters[d][i] && total_kb >= 2 * (1 << i)) {
      S = 1 << i;
      break;
    }
  int rc = gemm::encode_tmap_2d(ctx, &p.w, false, Wq, (uint64_t)K, (uint64_t)N, (uint64_t)ldk, 128, BNCH);
  if (rc) return rc;
  rc = gemm::encode_tmap_2d(ctx, &p.a, false, Aq, (uint64_t)K, (uint64_t)M, (uint64_t)ldk, 128, (uint32_t)MN);
  if (rc) return rc;
  p.M = M; p.N = N; p.K = K; p.MN = MN;
  p.status = ctx->d_status;
  const void* out = FUSED ? (const void*)p.Y : (const void*)p.acc;
  p.vec = (N % 4 == 0) && vtlb_aligned16(out) &&
          (!FUSED || (vtlb_aligned16(p.sw) && (p.bias == nullptr || vtlb_aligned16(p.bias))));
  const bool timed = ctx->prof_on && ctx->prof_ev && ctx->prof_n < vtlb_ctx::kProfSlots;
  if (timed) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
  rc = S == 4 ? launch_s<FUSED, 4>(ctx, tiles, p) : S == 2 ? launch_s<FUSED, 2>(ctx, tiles, p)
                                                          : launch_s<FUSED, 1>(ctx, tiles, p);
  if (rc) return rc;
  if (timed) {
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
    ctx->prof_flops += 2.0 * M * N * K;
  }
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace skinny
