// The tcgen05 GEMM used by both the INT8 path (kind::i8, int32 accumulators) and
// the f32 path (kind::tf32 issued three times per K step on pre-split hi/lo
// operands).  D[M,N] = A[M,K] . B[N,K]^T with both operands K-major.
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer   (one lane): global -> shared, 128-byte-swizzled tiles
//   warp 1      MMA issuer     (one lane): tcgen05.mma into tensor memory; owns the
//                                          tensor-memory allocation
//   warps 2..9  epilogue: tcgen05.ld the finished accumulator, apply the fused
//               epilogue functor, store to global
// Shared-memory stages form a ring guarded by full/empty mbarriers; the
// accumulator is double-buffered in tensor memory so the epilogue of one
// accumulator overlaps the MMAs that fill the other.  Every CTA loads its own
// tiles; there is no cluster and no multicast.
//
// Every mbarrier wait is bounded (ptx::mbar_wait_bounded).  If one runs out the
// CTA raises a shared abort flag, all roles leave their loops, the kernel ORs
// VTLB_ST_GEMM_TIMEOUT into the status word, waits a bounded time for copies
// still in flight, frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "ptx.cuh"

namespace gemm {

constexpr int BM = 128;           // rows of D per tile = TMEM lanes
constexpr int ROW_BYTES = 128;    // bytes of K per shared-memory row (= swizzle span)
constexpr int EPI_WARPS = 8;       // two warps per tensor-memory lane quarter, alternate column chunks
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s per wait

enum Kind { KIND_I8 = 0, KIND_TF32X3 = 1 };

template <int KIND>
struct Traits;
template <>
struct Traits<KIND_I8> {
  static constexpr int ELEM = 1;   // bytes per element
  static constexpr int NOP = 1;    // operand tiles per side per stage
  static constexpr uint32_t CFMT = ptx::kCfmtS32, ABFMT = ptx::kFmtS8;
};
template <>
struct Traits<KIND_TF32X3> {
  static constexpr int ELEM = 4;
  static constexpr int NOP = 2;    // hi and lo
  static constexpr uint32_t CFMT = ptx::kCfmtF32, ABFMT = ptx::kFmtTF32;
};

struct TmapSet {
  CUtensorMap a[2];    // [0] = A (i8) or A_hi, [1] = A_lo
  CUtensorMap b[2];
  // outputs of epilogues that store through TMA: [0] the result, [1] the pre-activation;
  // [2],[3] the result's TF32 hi / lo planes in the result's own layout (epilogues that declare
  // kPlanes: what the next product reads as an operand; the planes of the transpose are written
  // with plain stores)
  CUtensorMap out[4];
};

// One 32-row x 32-column staging tile (128-byte rows, 128-byte swizzle) per epilogue warp.
constexpr uint32_t STAGING_PER_WARP = 32 * 128;
constexpr uint32_t STAGING = EPI_WARPS * STAGING_PER_WARP;

template <int KIND, int BN, int STAGES>
struct Smem {
  static constexpr uint32_t A_TILE = BM * ROW_BYTES;
  static constexpr uint32_t B_TILE = BN * ROW_BYTES;
  static constexpr uint32_t STAGE = Traits<KIND>::NOP * (A_TILE + B_TILE);
  static constexpr uint32_t TILES = STAGES * STAGE;
  static constexpr uint32_t BARS_OFF = TILES + STAGING;
  static constexpr uint32_t BARS = 8 * (2 * STAGES + 4) + 16;
  static constexpr uint32_t TOTAL = BARS_OFF + BARS + 1024;  // + alignment slack
};

// Epilogue of one 32 x 32 chunk held one row per lane in v[32].
//
// Functors that declare kTmaCapable and have `tma` set transform the values in registers and
// hand them to a TMA store: the warp writes its chunk into a swizzled staging tile in shared
// memory and one lane issues cp.async.bulk.tensor, so global memory sees whole 128-byte rows
// instead of 32 scattered 16-byte pieces per store instruction (measured: the scattered stores,
// not the MMAs, bounded the 4096^3 INT8 GEMM).  Edges need no care: the store clips at the
// tensor's extent.  Everything else goes through the functor's own direct stores.

__device__ __forceinline__ void stage_and_store(uint32_t stg, const CUtensorMap* tmap, int lane, int row0,
                                                int col0, const uint32_t (&v)[32], int M, int N) {
  if (lane == 0) ptx::bulk_wait_read_all();  // the previous store has finished reading the tile
  __syncwarp();
  const uint32_t rowaddr = stg + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    ptx::st_shared_v4(rowaddr + (((uint32_t)j ^ ((uint32_t)lane & 7u)) << 4), v[4 * j], v[4 * j + 1],
                      v[4 * j + 2], v[4 * j + 3]);
  ptx::fence_proxy_async();
  __syncwarp();
  if (lane == 0 && row0 < M && col0 < N) {
    ptx::tma_store_2d(tmap, col0, row0, stg);
    ptx::bulk_commit_group();
  }
}

// x = hi + lo + O(2^-22 |x|), both representable in TF32 (the operand split of the 3xTF32 products).
__device__ __forceinline__ uint32_t tf32_hi_bits(uint32_t x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(__uint_as_float(x)));
  return r;
}
__device__ __forceinline__ uint32_t tf32_lo_bits(uint32_t x) {
  const float hi = __uint_as_float(tf32_hi_bits(x));
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(__uint_as_float(x) - hi));
  return r;
}

// The chunk's TF32 hi (LO = false) or lo plane through the staging tile and a TMA store, in the
// chunk's own layout (box at (col0, row0) of a [rows, cols] tensor).
template <bool LO>
__device__ __forceinline__ void stage_and_store_plane(uint32_t stg, const CUtensorMap* tmap, int lane, int row0,
                                                      int col0, const uint32_t (&v)[32], int M, int N) {
  if (lane == 0) ptx::bulk_wait_read_all();
  __syncwarp();
  const uint32_t rowaddr = stg + lane * 128;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) w[e] = LO ? tf32_lo_bits(v[4 * j + e]) : tf32_hi_bits(v[4 * j + e]);
    ptx::st_shared_v4(rowaddr + (((uint32_t)j ^ ((uint32_t)lane & 7u)) << 4), w[0], w[1], w[2], w[3]);
  }
  ptx::fence_proxy_async();
  __syncwarp();
  if (lane == 0 && row0 < M && col0 < N) {
    ptx::tma_store_2d(tmap, col0, row0, stg);
    ptx::bulk_commit_group();
  }
}

// The planes of the chunk transposed, [N, ld] with the chunk's rows along the contiguous dimension:
// lane = row, so every store instruction of the warp writes 32 consecutive words of one row of the
// transposed plane -- whole 128-byte lines straight from the registers, no staging and no wait.
__device__ __forceinline__ void store_planes_transposed(float* __restrict__ hi, float* __restrict__ lo, int ld,
                                                        int row, int col0, const uint32_t (&v)[32], int M, int N) {
  if (row >= M) return;
  uint32_t* ph = reinterpret_cast<uint32_t*>(hi) + (size_t)col0 * ld + row;
  uint32_t* pl = reinterpret_cast<uint32_t*>(lo) + (size_t)col0 * ld + row;
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    if (col0 + c < N) {
      const uint32_t h = tf32_hi_bits(v[c]);
      uint32_t l;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(__uint_as_float(v[c]) - __uint_as_float(h)));
      ph[(size_t)c * ld] = h;
      pl[(size_t)c * ld] = l;
    }
  }
}

template <class Epi>
struct EpiHasPlanes {
  template <class T>
  static constexpr bool test(decltype(T::kPlanes)*) { return T::kPlanes; }
  template <class T>
  static constexpr bool test(...) { return false; }
  static constexpr bool value = test<Epi>(nullptr);
};

template <class Epi>
__device__ __forceinline__ void epilogue_chunk(const Epi& epi, const TmapSet& tm, uint32_t stg, int lane,
                                               int row0, int col0, uint32_t (&v)[32], int M, int N,
                                               int split, bool mask_applied = false) {
  if constexpr (Epi::kTmaCapable) {
    if (epi.tma) {
      bool two;
      if constexpr (EpiHasPlanes<Epi>::value)
        two = epi.transform(row0 + lane, col0, v, M, N, mask_applied);
      else
        two = epi.transform(row0 + lane, col0, v, M, N);
      if (two) {  // true: v now holds the pre-activation
        stage_and_store(stg, &tm.out[1], lane, row0, col0, v, M, N);
        epi.activate(v);
      }
      stage_and_store(stg, &tm.out[0], lane, row0, col0, v, M, N);
      if constexpr (EpiHasPlanes<Epi>::value) {
        // operand planes of the result for the products that consume it next (what a separate
        // split pass over the stored result would write)
        if (epi.planes & 2)
          store_planes_transposed(epi.cols_hi, epi.cols_lo, epi.ld_cols, row0 + lane, col0, v, M, N);
        if (epi.planes & 1) {
          stage_and_store_plane<false>(stg, &tm.out[2], lane, row0, col0, v, M, N);
          stage_and_store_plane<true>(stg, &tm.out[3], lane, row0, col0, v, M, N);
        }
      }
      return;
    }
  }
  epi(row0 + lane, col0, v, M, N, split);
}

// Tile order.  Tiles are walked in groups of `group_m` rows of tiles: inside a group the m
// index runs fastest, then n.  The CTAs resident at one time then share `group_m` blocks of A
// (which stay in L2 for the whole sweep over n) and a few blocks of B, instead of touching
// every block of A for each handful of B blocks.
__device__ __forceinline__ void decode_tile(int mn, int tiles_m, int tiles_n, int group_m, int& tm,
                                            int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = mn / per_group;
  const int first_m = g * group_m;
  const int gsz = tiles_m - first_m < group_m ? tiles_m - first_m : group_m;
  const int r = mn - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}
// Rows of tiles per group such that the group's A blocks take about `budget` bytes of L2.
inline int pick_group_m(int tiles_m, size_t a_bytes_per_tile_row, size_t budget = (size_t)40 << 20) {
  size_t g = budget / (a_bytes_per_tile_row ? a_bytes_per_tile_row : 1);
  if (g < 1) g = 1;
  if (g > (size_t)tiles_m) g = tiles_m;
  return (int)g;
}

template <int KIND, int BN, int STAGES, class Epi>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ TmapSet tm, const Epi epi, int M, int N, int K, int splits,
               int group_m, int a_chunk_k, uint32_t* status) {
  using T = Traits<KIND>;
  using S = Smem<KIND, BN, STAGES>;
  constexpr int NOP = T::NOP;
  constexpr int BK = ROW_BYTES / T::ELEM;   // elements of K per stage
  constexpr int KSTEPS = ROW_BYTES / 32;    // MMAs per operand pair per stage (32 B of K each)
  // Tensor-memory accumulators.  INT8 is exact, so one accumulator per buffer takes the
  // whole K loop.  The f32 accumulator of tcgen05 truncates on every add, a bias that
  // grows with the number of MMAs; the TF32x3 path therefore (a) keeps the small
  // cross terms (lo.hi + hi.lo) in an accumulator of their own, so they never cost
  // the leading sum an ulp, and (b) closes an accumulator every CHUNK_KB stages; the
  // epilogue warps sum the chunks in registers with round-to-nearest adds.
  constexpr int NACC = (KIND == KIND_TF32X3) ? 2 : 1;
  constexpr int CHUNK_KB = (KIND == KIND_TF32X3) ? 4 : 0;  // 0 = the whole K loop
  constexpr uint32_t TMEM_COLS = 2 * NACC * BN;
  static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");
  constexpr uint32_t IDESC = ptx::umma_idesc(T::CFMT, T::ABFMT, BM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + S::BARS_OFF;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars - raw) + 8u * (2 * STAGES + 4));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  // Split-K: the K loop is cut into `splits` ranges and every (m, n, range) is a tile of its
  // own; the epilogue functor receives the range index and stores a partial result.
  const int mn_tiles = tiles_m * tiles_n;
  const int num_tiles = mn_tiles * splits;
  const int total_kb = (K + BK - 1) / BK;
  const int kb_per_split = (total_kb + splits - 1) / splits;
  const int chunk_kb = CHUNK_KB ? CHUNK_KB : kb_per_split;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 32 * EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    for (int i = 0; i < NOP; ++i) {
      ptx::prefetch_tmap(&tm.a[i]);
      ptx::prefetch_tmap(&tm.b[i]);
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mn = tile % mn_tiles, split = tile / mn_tiles;
        int tmi, tni;
      decode_tile(mn, tiles_m, tiles_n, group_m, tmi, tni);
      const int m0 = tmi * BM, n0 = tni * BN;
        const int kb_begin = split * kb_per_split;
        const int kb_end = kb_begin + kb_per_split < total_kb ? kb_begin + kb_per_split : total_kb;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(full_bar(stage), S::STAGE);
          const uint32_t sa = base + stage * S::STAGE;
          const uint32_t sb = sa + NOP * S::A_TILE;
#pragma unroll
          for (int i = 0; i < NOP; ++i)
            if (a_chunk_k)  // A stored as [chunk][M][a_chunk_k] (gathered column shards)
              ptx::tma_load_3d(sa + i * S::A_TILE, &tm.a[i], (kb * BK) % a_chunk_k, m0,
                               (kb * BK) / a_chunk_k, full_bar(stage));
            else
              ptx::tma_load_2d(sa + i * S::A_TILE, &tm.a[i], kb * BK, m0, full_bar(stage));
#pragma unroll
          for (int i = 0; i < NOP; ++i)
            ptx::tma_load_2d(sb + i * S::B_TILE, &tm.b[i], kb * BK, n0, full_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int kb_begin = (tile / mn_tiles) * kb_per_split;
        const int kb_end = kb_begin + kb_per_split < total_kb ? kb_begin + kb_per_split : total_kb;
        for (int kb0 = kb_begin; kb0 < kb_end && ok; kb0 += chunk_kb) {
          const int kb1 = kb0 + chunk_kb < kb_end ? kb0 + chunk_kb : kb_end;
          if (!ptx::mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag,
                                      WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t d_main = tmem_base + acc * BN;
          const uint32_t d_small = tmem_base + (2 + acc) * BN;  // TF32x3 only
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t sa = base + stage * S::STAGE;
            const uint32_t sb = sa + NOP * S::A_TILE;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
              const uint32_t first = (kb == kb0 && kk == 0) ? 0u : 1u;
              // advancing 32 bytes along K inside the swizzled row = +2 in the address field
              if constexpr (KIND == KIND_I8) {
                const uint64_t da = ptx::umma_desc_k_sw128(sa) + 2u * kk;
                const uint64_t db = ptx::umma_desc_k_sw128(sb) + 2u * kk;
                ptx::umma_i8(d_main, da, db, IDESC, first);
              } else {
                const uint64_t a_hi = ptx::umma_desc_k_sw128(sa) + 2u * kk;
                const uint64_t a_lo = ptx::umma_desc_k_sw128(sa + S::A_TILE) + 2u * kk;
                const uint64_t b_hi = ptx::umma_desc_k_sw128(sb) + 2u * kk;
                const uint64_t b_lo = ptx::umma_desc_k_sw128(sb + S::B_TILE) + 2u * kk;
                ptx::umma_tf32(d_small, a_lo, b_hi, IDESC, first);
                ptx::umma_tf32(d_small, a_hi, b_lo, IDESC, 1);
                ptx::umma_tf32(d_main, a_hi, b_hi, IDESC, first);
              }
            }
            ptx::umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!ok) break;
          ptx::umma_commit(tfull_bar(acc));  // this chunk's accumulators are complete
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;  // which of the quarter's two warps: even or odd column chunks
    const uint32_t stg = base + S::TILES + (uint32_t)(warp - 2) * STAGING_PER_WARP;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int mn = tile % mn_tiles, split = tile / mn_tiles;
      int tmi, tni;
      decode_tile(mn, tiles_m, tiles_n, group_m, tmi, tni);
      const int m0 = tmi * BM, n0 = tni * BN;
      const int kb_begin = split * kb_per_split;
      const int kb_end = kb_begin + kb_per_split < total_kb ? kb_begin + kb_per_split : total_kb;
      const int row0 = m0 + q * 32;
      if constexpr (KIND == KIND_I8) {
        ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll 1
        for (int c = half; c < BN / 32; c += 2) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(lane_base + acc * BN + c * 32, v);
          ptx::tmem_wait_ld();
          epilogue_chunk(epi, tm, stg, lane, row0, n0 + c * 32, v, M, N, split);
          __syncwarp();
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(tempty_bar(acc));
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      } else {
        float sum[BN / 2];
#pragma unroll
        for (int j = 0; j < BN / 2; ++j) sum[j] = 0.0f;
        // ReLU-backward mask of the tile's outputs, fetched now as one bit per value
        uint32_t mask_bits[BN / 64];
        if constexpr (EpiHasPlanes<Epi>::value) {
#pragma unroll
          for (int cc = 0; cc < BN / 64; ++cc) {
            mask_bits[cc] = epi.load_mask_bits(row0 + lane, n0 + (2 * cc + half) * 32, M, N);
            asm volatile("" ::: "memory");  // one chunk's eight loads at a time: the running sums own the registers
          }
        }
        for (int kb0 = kb_begin; kb0 < kb_end; kb0 += chunk_kb) {
          ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < BN / 64; ++cc) {
            const int c = 2 * cc + half;
            uint32_t v[32], w[32];
            ptx::tmem_ld_32x32(lane_base + acc * BN + c * 32, v);
            ptx::tmem_ld_32x32(lane_base + (2 + acc) * BN + c * 32, w);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              sum[cc * 32 + j] = __fadd_rn(
                  sum[cc * 32 + j], __fadd_rn(__uint_as_float(v[j]), __uint_as_float(w[j])));
          }
          ptx::tc_fence_before();
          ptx::mbar_arrive(tempty_bar(acc));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
        if (!ok) break;
#pragma unroll
        for (int cc = 0; cc < BN / 64; ++cc) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(sum[cc * 32 + j]);
          if constexpr (EpiHasPlanes<Epi>::value) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (mask_bits[cc] >> j & 1u) v[j] = 0u;
          }
          epilogue_chunk(epi, tm, stg, lane, row0, n0 + (2 * cc + half) * 32, v, M, N, split, true);
          __syncwarp();
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if (warp >= 2 && lane == 0) ptx::bulk_wait_read_all();  // staged TMA stores have left shared memory
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(status, VTLB_ST_GEMM_TIMEOUT);
    // bounded grace period for TMA copies / MMAs still in flight
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side

// cuTensorMapEncodeTiled obtained through the runtime (no link against libcuda).
int encode_tmap_3d_u8(vtlb_ctx* ctx, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows,
                      uint64_t planes, uint64_t row_stride_bytes, uint64_t plane_stride_bytes,
                      uint32_t box_inner, uint32_t box_rows);
int encode_tmap_2d(vtlb_ctx* ctx, CUtensorMap* out, bool f32, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                   uint32_t box_outer);
int encode_tmap_3d_f32_plain(vtlb_ctx* ctx, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows,
                             uint64_t planes, uint32_t box_inner, uint32_t box_rows);

template <int KIND, int BN, int STAGES, class Epi>
int launch(vtlb_ctx* ctx, const TmapSet& tm, const Epi& epi, int M, int N, int K, int splits = 1,
           int a_chunk_k = 0) {
  using S = Smem<KIND, BN, STAGES>;
  static_assert(S::TOTAL <= 232448, "shared memory budget");
  auto kern = gemm_tc_kernel<KIND, BN, STAGES, Epi>;
  static std::atomic<uint64_t> configured{0};  // one bit per device
  if (!(configured.load(std::memory_order_relaxed) >> (ctx->device & 63) & 1)) {
    VTLB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)S::TOTAL));
    configured.fetch_or(1ull << (ctx->device & 63), std::memory_order_relaxed);
  }
  {  // drop ranges that would be empty
    constexpr int BKE = ROW_BYTES / Traits<KIND>::ELEM;
    const int total_kb = (K + BKE - 1) / BKE;
    if (splits < 1) splits = 1;
    if (splits > total_kb) splits = total_kb;
    const int per = (total_kb + splits - 1) / splits;
    splits = (total_kb + per - 1) / per;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * splits;
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  const bool timed = ctx->prof_on && ctx->prof_ev && ctx->prof_n < vtlb_ctx::kProfSlots;
  if (timed) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
  const int group_m = pick_group_m((M + BM - 1) / BM, (size_t)BM * K * Traits<KIND>::ELEM * Traits<KIND>::NOP);
  kern<<<grid, NUM_THREADS, S::TOTAL, ctx->stream>>>(tm, epi, M, N, K, splits, group_m, a_chunk_k,
                                                     ctx->d_status);
  if (timed) {
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
    ctx->prof_flops += 2.0 * M * N * K;
  }
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace gemm
