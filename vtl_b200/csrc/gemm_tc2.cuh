// GEMM on CTA pairs: tcgen05.mma.cta_group::2, one 256 x 256 tile of D per pair; INT8 (kind::i8)
// and f32 as 3xTF32 (kind::tf32 on hi/lo planes).
//
// Why a pair: with one CTA per 128 x 256 tile every SM has to land 48 KB of operands in
// shared memory per 512 tensor-core cycles while the MMA reads 96 B/clk from the same
// shared memory, and the tensor pipe idles waiting for data.  A pair shares the B operand:
// each CTA loads its own 128 rows of A and HALF of the 256 B rows (32 KB per stage), the MMA
// of the leader CTA reads both halves, and each CTA ends up with its own 128 x 256 slice of
// D in its tensor memory.
//
// Roles per CTA (320 threads) as in gemm_tc.cuh: warp 0 TMA producer, warp 1 MMA issuer
// (only in the leader CTA) and tensor-memory owner, warps 2..9 epilogue.  Cross-CTA
// signalling:
//   full[s]    lives in the leader; both CTAs' TMA loads complete their bytes on it
//   empty[s]   one per CTA; the leader's tcgen05.commit multicasts the arrive to both
//   tfull[a]   one per CTA; commit multicast
//   tempty[a]  lives in the leader; the 16 epilogue warps of the pair arrive on it
// No TMA multicast is used: every CTA issues plain loads into its own shared memory.
// All waits are bounded (see gemm_tc.cuh); the two cluster barriers are reached by every
// thread on every path.
#pragma once
#include "gemm_tc.cuh"

namespace gemm2 {

using gemm::BM;
using gemm::NUM_THREADS;
using gemm::ROW_BYTES;
using gemm::WAIT_LIMIT_NS;

constexpr int BN2 = 256;      // columns of D per pair tile
#ifndef VTLB_PAIR_STAGES
#define VTLB_PAIR_STAGES 6  // shared-memory ring depth of the INT8 pair kernel (tuning knob)
#endif

template <int KIND>
struct Cfg {
  static constexpr int NOP = gemm::Traits<KIND>::NOP;                 // operand planes per side
  static constexpr int STAGES = KIND == gemm::KIND_I8 ? VTLB_PAIR_STAGES : 3;
  static constexpr uint32_t A_TILE = BM * ROW_BYTES;                  // this CTA's 128 rows of A
  static constexpr uint32_t B_HALF = (BN2 / 2) * ROW_BYTES;           // this CTA's 128 rows of B
  static constexpr uint32_t STAGE = NOP * (A_TILE + B_HALF);          // 32 KB (INT8) / 64 KB (TF32x3)
  static constexpr uint32_t TILES = STAGES * STAGE;
  static constexpr uint32_t BARS_OFF = TILES + gemm::STAGING;         // epilogue staging tiles in between
  static constexpr uint32_t SMEM_TOTAL = BARS_OFF + 8 * (2 * STAGES + 4) + 16 + 1024;
  // TF32x3 closes its accumulator every CHUNK_KB stages (the f32 accumulate of tcgen05 truncates;
  // see gemm_tc.cuh).  With 256 columns per accumulator and two buffers there is no room in tensor
  // memory for a separate accumulator of the small cross terms: here they share the main one, which
  // costs three truncations per K step instead of one, still two orders inside the error bound.
  static constexpr int CHUNK_KB = KIND == gemm::KIND_TF32X3 ? 4 : 0;
};
constexpr uint32_t TMEM_COLS = 2 * BN2;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank`
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose byte count completes on an mbarrier that may
// live in the peer CTA (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tmap, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* tmap, int x, int y, int z,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the mbarrier at this shared-memory offset in both CTAs of the pair once every
// tcgen05 operation issued so far has completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Scratch of the K-split tiles (see the kernel): flags first, then the parked accumulators.
constexpr int KSPLIT_MAX_TILES = 64;  // at most half of the CTA pairs of a device
constexpr int KSPLIT_FLAG_WORDS = KSPLIT_MAX_TILES * 2 * gemm::EPI_WARPS;  // [tile][rank][warp]
constexpr size_t KSPLIT_BYTES = (size_t)KSPLIT_FLAG_WORDS * 4 + (size_t)KSPLIT_MAX_TILES * 2 * BM * BN2 * 4;
static_assert(KSPLIT_MAX_TILES == vtlb_ctx::kKsplitTiles && KSPLIT_FLAG_WORDS * 4 == vtlb_ctx::kKsplitFlagBytes &&
                  KSPLIT_BYTES == vtlb_ctx::kKsplitBytes,
              "the context allocates the K-split buffer with these sizes");

__device__ __forceinline__ void flag_release(uint32_t* flag, uint32_t value) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}
// Spins until *flag == value; gives up after limit_ns or when the CTA's abort flag is raised
// (and raises it), like the mbarrier waits.
__device__ __forceinline__ bool flag_wait_bounded(const uint32_t* flag, uint32_t value,
                                                  volatile uint32_t* abort_flag, uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    uint32_t seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (seen == value) return true;
    if ((spins & 63u) == 63u) {
      if (*abort_flag) return false;
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
      __nanosleep(64);
    }
  }
}


template <int KIND, class Epi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ gemm::TmapSet tm, const Epi epi, int M, int N, int K,
                 int group_m, int a_chunk_k, int split_tiles, uint32_t* ksplit_buf, uint32_t ksplit_epoch,
                 uint32_t* status) {
  using T = gemm::Traits<KIND>;
  using C = Cfg<KIND>;
  constexpr int NOP = C::NOP, STAGES = C::STAGES;
  constexpr int BK = ROW_BYTES / T::ELEM;  // elements of K per stage
  constexpr int KSTEPS = ROW_BYTES / 32;
  constexpr uint32_t IDESC = ptx::umma_idesc(T::CFMT, T::ABFMT, 2 * BM, BN2);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + C::BARS_OFF;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars - raw) + 8u * (2 * STAGES + 4));
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN2 - 1) / BN2;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int chunk_kb = C::CHUNK_KB ? C::CHUNK_KB : num_kb;
  // Work units.  When the tiles do not fill the last wave of CTA pairs, `split_tiles` tiles (the
  // first ones) are cut along K into two units each, which evens out the work per pair (4096^3:
  // 256 tiles on 74 pairs = 3.46 waves; with 34 tiles cut, 68 pairs run 3.5 tiles' worth and 6
  // pairs run 3).  Pair 2s runs the first K half of cut tile s as its FIRST unit, parks the raw
  // int32 accumulators in `ksplit_buf` and publishes one flag per epilogue warp; pair 2s+1 runs
  // the second half as its SECOND unit (after a full tile), adds the parked values to its own and
  // does the epilogue proper.  By then the parked half has long landed, and the slower epilogue of
  // that one unit hides behind the MMAs of the next.  Integer addition keeps the result
  // bit-identical.  INT8 only.  The first-half unit never waits for anybody and has the lower CTA
  // numbers, which are dispatched first: the second-half unit's (bounded) wait cannot deadlock.
  //
  // Unit `it` of this pair: false when the pair has run out of work.  Full tiles fill every
  // position that is not a half unit, in order of (it, pair).
  auto decode_unit = [&](int it, int& tmi, int& tni, int& k_half, int& slot) -> bool {
    const int S = split_tiles, P = num_pairs, p = pair;
    const bool cut = p < 2 * S;
    k_half = -1;
    slot = 0;
    int f;  // index among the full tiles
    if (it == 0) {
      if (cut && (p & 1) == 0) {
        k_half = 0;
        slot = p >> 1;
      }
      f = cut ? (p >> 1) : p - S;
    } else if (it == 1) {
      if (cut && (p & 1) == 1) {
        k_half = 1;
        slot = p >> 1;
      }
      f = (P - S) + (cut ? (p >> 1) : p - S);
    } else {
      f = 2 * (P - S) + (it - 2) * P + p;
    }
    int tile = slot;
    if (k_half < 0) {
      if (f >= num_tiles - S) return false;
      tile = S + f;
    }
    gemm::decode_tile(tile, tiles_m, tiles_n, group_m, tmi, tni);
    return true;
  };
  auto k_range = [&](int k_half, int& kb_begin, int& kb_end) {
    kb_begin = k_half == 1 ? num_kb / 2 : 0;
    kb_end = k_half == 0 ? num_kb / 2 : num_kb;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);   // the leader's expect_tx arrive; bytes from both CTAs
      ptx::mbar_init(empty_bar(s), 1);  // one multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 2 * gemm::EPI_WARPS);  // the epilogue warps of both CTAs
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
    tmem_alloc2(ptx::smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish2();
  }
  ptx::tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        int tmi, tni, kh, slot, kb_begin, kb_end;
        if (!decode_unit(it, tmi, tni, kh, slot)) break;
        k_range(kh, kb_begin, kb_end);
        const int m0 = tmi * 2 * BM + (int)rank * BM;
        const int n0 = tni * BN2 + (int)rank * (BN2 / 2);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          const uint32_t leader_full = mapa(full_bar(stage), 0);
          if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * C::STAGE);
          const uint32_t sa = base + stage * C::STAGE;
          const uint32_t sb = sa + NOP * C::A_TILE;
#pragma unroll
          for (int i = 0; i < NOP; ++i) {
            if (a_chunk_k)  // A stored as [chunk][M][a_chunk_k] (gathered column shards)
              tma_load_3d_pair(sa + i * C::A_TILE, &tm.a[i], (kb * BK) % a_chunk_k, m0, (kb * BK) / a_chunk_k,
                               leader_full);
            else
              tma_load_2d_pair(sa + i * C::A_TILE, &tm.a[i], kb * BK, m0, leader_full);
          }
#pragma unroll
          for (int i = 0; i < NOP; ++i)
            tma_load_2d_pair(sb + i * C::B_HALF, &tm.b[i], kb * BK, n0, leader_full);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int it = 0; ok; ++it) {
        int tmi, tni, kh, slot, kb_begin, kb_end;
        if (!decode_unit(it, tmi, tni, kh, slot)) break;
        k_range(kh, kb_begin, kb_end);
        for (int kb0 = kb_begin; kb0 < kb_end && ok; kb0 += chunk_kb) {
          const int kb1 = kb0 + chunk_kb < kb_end ? kb0 + chunk_kb : kb_end;
          if (!ptx::mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN2;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t sa = base + stage * C::STAGE;
            const uint32_t sb = sa + NOP * C::A_TILE;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
              const uint32_t first = (kb == kb0 && kk == 0) ? 0u : 1u;
              if constexpr (KIND == gemm::KIND_I8) {
                const uint64_t da = ptx::umma_desc_k_sw128(sa) + 2u * kk;
                const uint64_t db = ptx::umma_desc_k_sw128(sb) + 2u * kk;
                umma_i8_pair(d_tmem, da, db, IDESC, first);
              } else {
                const uint64_t a_hi = ptx::umma_desc_k_sw128(sa) + 2u * kk;
                const uint64_t a_lo = ptx::umma_desc_k_sw128(sa + C::A_TILE) + 2u * kk;
                const uint64_t b_hi = ptx::umma_desc_k_sw128(sb) + 2u * kk;
                const uint64_t b_lo = ptx::umma_desc_k_sw128(sb + C::B_HALF) + 2u * kk;
                umma_tf32_pair(d_tmem, a_lo, b_hi, IDESC, first);  // small terms first
                umma_tf32_pair(d_tmem, a_hi, b_lo, IDESC, 1);
                umma_tf32_pair(d_tmem, a_hi, b_hi, IDESC, 1);
              }
            }
            umma_commit_pair(empty_bar(stage));
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!ok) break;
          umma_commit_pair(tfull_bar(acc));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;  // even or odd 32-column chunks
    const uint32_t stg = base + C::TILES + (uint32_t)(warp - 2) * gemm::STAGING_PER_WARP;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int it = 0; ok; ++it) {
      int tmi, tni, kh, slot;
      if (!decode_unit(it, tmi, tni, kh, slot)) break;
      const int m0 = tmi * 2 * BM + (int)rank * BM;
      const int n0 = tni * BN2;
      const int row0 = m0 + q * 32;
      if constexpr (KIND == gemm::KIND_I8) {
        // Per-row and per-column operands of the epilogue (scales, bias) are fetched before the
        // wait for the accumulator, one column per lane, and handed round by shuffles later:
        // their latency would otherwise sit in front of every 32-column chunk.
        const bool fast = epi.tma != 0;
        typename Epi::Pre pre;
        if (fast) pre = epi.prefetch(row0 + lane, n0 + half * 32 + lane, M, N);
        ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
        // K-split tile: the unit of the first K half parks its accumulators,
        // [slot][rank][warp][chunk][value][lane], and the unit of the second half adds them to its own.
        const int wslot = (slot * 2 + (int)rank) * gemm::EPI_WARPS + (warp - 2);
        uint32_t* park = ksplit_buf + KSPLIT_FLAG_WORDS + (size_t)wslot * (BN2 / 64) * 1024;
        if (kh == 1) {  // wait for the first K half of this tile
          if (lane == 0) ok = flag_wait_bounded(ksplit_buf + wslot, ksplit_epoch, abort_flag, WAIT_LIMIT_NS);
          ok = __all_sync(0xffffffffu, __shfl_sync(0xffffffffu, (int)ok, 0) != 0);
          if (!ok) break;
        }
        float row_amax = 0.0f;
        auto do_chunk = [&](int cc, bool use_pre) {
          const int c = 2 * cc + half;
          uint32_t v[32];
          ptx::tmem_ld_32x32(lane_base + acc * BN2 + c * 32, v);
          ptx::tmem_wait_ld();
          uint32_t* pc = park + cc * 1024 + lane;
          if (kh == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(pc + j * 32, v[j]);
          } else {
            if (kh == 1) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += __ldcg(pc + j * 32);
            }
            if (use_pre) {
              epi.transform_pre(pre, cc, v);
              row_amax = fmaxf(row_amax, epi.chunk_amax(n0 + c * 32, v, N));  // one atomic per warp and tile
              gemm::stage_and_store(stg, &tm.out[0], lane, row0, n0 + c * 32, v, M, N);
            } else {
              gemm::epilogue_chunk(epi, tm, stg, lane, row0, n0 + c * 32, v, M, N, 0);
            }
          }
          __syncwarp();
        };
        if (fast) {
#pragma unroll
          for (int cc = 0; cc < BN2 / 64; ++cc) do_chunk(cc, true);
        } else {
#pragma unroll 1
          for (int cc = 0; cc < BN2 / 64; ++cc) do_chunk(cc, false);
        }
        if (fast && kh != 0) epi.commit_amax(row0 + lane, M, row_amax);
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
        if (kh == 0) {  // publish: every lane's stores, then the flag
          __threadfence();
          __syncwarp();
          if (lane == 0) flag_release(ksplit_buf + wslot, ksplit_epoch);
        }
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      } else {
        float sum[BN2 / 2];  // this warp's four 32-column chunks
#pragma unroll
        for (int j = 0; j < BN2 / 2; ++j) sum[j] = 0.0f;
        // ReLU-backward mask of the tile's outputs, fetched now as one bit per value
        uint32_t mask_bits[BN2 / 64];
        if constexpr (gemm::EpiHasPlanes<Epi>::value) {
#pragma unroll
          for (int cc = 0; cc < BN2 / 64; ++cc) {
            mask_bits[cc] = epi.load_mask_bits(row0 + lane, n0 + (2 * cc + half) * 32, M, N);
            asm volatile("" ::: "memory");  // one chunk's eight loads at a time: the running sums own the registers
          }
        }
        for (int kb0 = 0; kb0 < num_kb; kb0 += chunk_kb) {
          ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < BN2 / 64; ++cc) {
            uint32_t v[32];
            ptx::tmem_ld_32x32(lane_base + acc * BN2 + (2 * cc + half) * 32, v);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[cc * 32 + j] = __fadd_rn(sum[cc * 32 + j], __uint_as_float(v[j]));
          }
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
        if (!ok) break;
#pragma unroll
        for (int cc = 0; cc < BN2 / 64; ++cc) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(sum[cc * 32 + j]);
          if constexpr (gemm::EpiHasPlanes<Epi>::value) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (mask_bits[cc] >> j & 1u) v[j] = 0u;
          }
          gemm::epilogue_chunk(epi, tm, stg, lane, row0, n0 + (2 * cc + half) * 32, v, M, N, 0, true);
          __syncwarp();
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if (warp >= 2 && lane == 0) ptx::bulk_wait_read_all();  // staged TMA stores have left shared memory
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(status, VTLB_ST_GEMM_TIMEOUT);
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // the peer may still signal this CTA's barriers until it gets here
  ptx::tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

// True when the problem has enough 256 x 256 tiles for the CTA pairs to pay off.
inline bool pair_worthwhile(vtlb_ctx* ctx, int M, int N) {
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  return M >= 512 && N >= 256 && tiles >= ctx->sm_count / 4;
}

template <int KIND, class Epi>
int launch_pair(vtlb_ctx* ctx, const gemm::TmapSet& tm, const Epi& epi, int M, int N, int K,
                int a_chunk_k = 0, bool k_split = false) {
  using C = Cfg<KIND>;
  static_assert(C::SMEM_TOTAL <= 232448, "shared memory budget");
  auto kern = gemm_pair_kernel<KIND, Epi>;
  static std::atomic<uint64_t> configured{0};
  if (!(configured.load(std::memory_order_relaxed) >> (ctx->device & 63) & 1)) {
    VTLB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM_TOTAL));
    configured.fetch_or(1ull << (ctx->device & 63), std::memory_order_relaxed);
  }
  const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN2 - 1) / BN2);
  int pairs = ctx->sm_count / 2;
  if (tiles < pairs) pairs = tiles;
  const bool timed = ctx->prof_on && ctx->prof_ev && ctx->prof_n < vtlb_ctx::kProfSlots;
  if (timed) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
  const int group_m = gemm::pick_group_m((M + 2 * BM - 1) / (2 * BM),
                                         (size_t)2 * BM * K * gemm::Traits<KIND>::ELEM * C::NOP);
  // When the final wave would fill at most half of the pairs, cut that many tiles into two half-K
  // units each (INT8 only: integer partial sums add up exactly); they all fit in the first wave.
  int split_tiles = 0;
  if (KIND == gemm::KIND_I8 && k_split) {
    const int rem = tiles % pairs;
    const int num_kb = (K + 127) / 128;
    if (tiles > pairs && rem > 0 && 2 * rem <= pairs && rem <= KSPLIT_MAX_TILES && num_kb >= 8) split_tiles = rem;
  }
  if (split_tiles && ++ctx->ksplit_epoch == 0) ctx->ksplit_epoch = 1;  // flags hold the epoch of their launch
  kern<<<2 * pairs, NUM_THREADS, C::SMEM_TOTAL, ctx->stream>>>(tm, epi, M, N, K, group_m, a_chunk_k, split_tiles,
                                                               (uint32_t*)ctx->ksplit_buf, ctx->ksplit_epoch,
                                                               ctx->d_status);
  if (timed) {
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
    ctx->prof_flops += 2.0 * M * N * K;
  }
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace gemm2
