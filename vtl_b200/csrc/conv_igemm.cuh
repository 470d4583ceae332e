// Convolution as an implicit GEMM on tcgen05 (f32 as 3xTF32): D[m, n] = sum_k A[m, k] . B[n, k]
// where the rows m are pixels (b, y, x) of an output grid, the columns k are (channel, tap) pairs
// and A[m, k] = src[b][ch(k)][y*sy + dy(k)][x*sx + dx(k)] (zero outside the image) is never
// stored: eight warps of the CTA gather it straight from the NCHW tensor, split every value into
// its TF32 hi/lo parts and write both into the 128-byte-swizzled shared-memory tiles the MMAs
// read.  B (the weights, a few KB) comes in by TMA from pre-split planes as in gemm_tc.cuh.
//   forward        src = x, rows = output pixels, k = (kh, kw, ic), dy = kh - ph, dx = kw - pw,
//                  B = the weights regrouped as [oc][(kh, kw, ic)]
//   input gradient src = g, rows = input pixels,  k = (kh, kw, oc), dy = ph - kh, dx = pw - kw
//                  (unit stride), B = the weights regrouped as [ic][(kh, kw, oc)]
// The channel runs fastest in k: when the channel count is a multiple of 32, a K block of 32
// columns is one tap of 32 consecutive channels, so a gather thread tests its pixel's tap once and
// then loads at a fixed stride (one plane apart) - about five times fewer instructions per element
// than looking every column up in the table, which remains the general path.
// Replaces the im2col / col2im passes of the lowered path for these two products.
//
// One persistent CTA per SM, 448 threads: warp 0 = TMA producer for B (one lane), warp 1 = MMA
// issuer and tensor-memory owner, warps 2..5 = epilogue (one per tensor-memory lane quarter),
// warps 6..13 = gather (two threads per tile row, half a K block each).  full[s] collects the
// producer's expect_tx arrive, the TMA bytes and one arrive per gather warp (after
// fence.proxy.async: the tensor core reads shared memory through the async proxy); empty[s] is the
// MMA commit.  All waits are bounded as in gemm_tc.cuh.
#pragma once
#include "f32_common.cuh"
#include "gemm_tc.cuh"

namespace igemm {

using gemm::BM;
using gemm::ROW_BYTES;
using gemm::WAIT_LIMIT_NS;

constexpr int BN = 64;
constexpr int STAGES = 3;
constexpr int EPI_WARPS = 4, GATHER_WARPS = 8;  // two gather threads per tile row: half a K block each
constexpr int NUM_THREADS = 64 + 32 * (EPI_WARPS + GATHER_WARPS);
// The gather warps are the ones with work to do; everybody else sleeps between polls of a barrier
// (measured: polling warps executed two thirds of the kernel's instructions).
constexpr uint32_t POLL_SLEEP_NS = 40;
constexpr int MAX_K = 2048;  // (channel, tap) pairs whose offsets fit the shared-memory table
constexpr uint32_t A_TILE = BM * ROW_BYTES, B_TILE = BN * ROW_BYTES;
constexpr uint32_t STAGE = 2 * (A_TILE + B_TILE);
constexpr uint32_t TILES = STAGES * STAGE;
constexpr uint32_t TABLE_OFF = TILES;                 // int2 per k: {offset, bit of its tap (0 for k >= K)}
// Output staging, per epilogue warp: [half of the channels][output, pre-activation][32 channels][32
// pixels] f32, 4 KB each.  One TMA store per piece writes it as 32 runs of 128 bytes into the NCHW
// tensor; the two halves alternate, so a warp fills one while the other drains.
constexpr uint32_t OUT_PIECE = 32 * 32 * 4;
constexpr uint32_t OUT_WARP = 4 * OUT_PIECE;
constexpr uint32_t OUT_OFF = TABLE_OFF + MAX_K * 8;
constexpr uint32_t BARS_OFF = OUT_OFF + 4 * OUT_WARP;
constexpr uint32_t SMEM_TOTAL = BARS_OFF + 8 * (2 * STAGES + 4) + 16 + 1024;

struct Geometry {
  int B, Cs, Hs, Ws;   // source tensor [B, Cs, Hs, Ws]
  int Ho, Wo;          // grid of the GEMM rows: m = (b, y, x), y < Ho, x < Wo
  int sy, sx;          // source row/column of a grid point = y*sy + dy, x*sx + dx
  int kh, kw;          // taps; k = (a * kw + b) * Cs + ch
  int dy0, dx0, dsign; // dy = dy0 + dsign * a, dx = dx0 + dsign * b
  int K;               // Cs * kh * kw
};


template <class Epi>
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_igemm_kernel(const float* __restrict__ src, const Geometry g, const __grid_constant__ gemm::TmapSet tm,
                  const Epi epi, int M, int N, int staged_out, uint32_t* status) {
  constexpr int BK = 32, KSTEPS = 4, CHUNK_KB = 4;
  constexpr int HB = BK * BM / (32 * GATHER_WARPS);  // elements of a row's K block per gather thread
  constexpr uint32_t TMEM_COLS = 4 * BN;  // two buffers x (main + small cross-term accumulator)
  constexpr uint32_t IDESC = ptx::umma_idesc(ptx::kCfmtF32, ptx::kFmtTF32, BM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + BARS_OFF;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars - raw) + 8u * (2 * STAGES + 4));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int2* ktab = reinterpret_cast<int2*>(smem_raw + (base - raw) + TABLE_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (g.K + BK - 1) / BK;

  // (channel, tap) -> offset inside an image and the tap's index (whether a tap falls inside the
  // image depends on the pixel only: every gather thread keeps one validity bit per tap)
  const int taps = g.kh * g.kw;
  for (int k = threadIdx.x; k < num_kb * BK; k += NUM_THREADS) {
    int2 e = make_int2(0, 0);  // k >= K: no tap
    if (k < g.K) {
      const int r = k / g.Cs, ch = k - r * g.Cs;
      const int a = r / g.kw, b = r - a * g.kw;
      const int dy = g.dy0 + g.dsign * a, dx = g.dx0 + g.dsign * b;
      e.x = (ch * g.Hs + dy) * g.Ws + dx;
      e.y = (int)(1u << r);
    }
    ktab[k] = e;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1 + GATHER_WARPS);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 32 * EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tmap(&tm.b[0]);
    ptx::prefetch_tmap(&tm.b[1]);
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
    // ------------------------------------------------------------ TMA producer (B planes)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * B_TILE);
          const uint32_t sb = base + stage * STAGE + 2 * A_TILE;
          ptx::tma_load_2d(sb, &tm.b[0], kb * BK, n0, full_bar(stage));
          ptx::tma_load_2d(sb + B_TILE, &tm.b[1], kb * BK, n0, full_bar(stage));
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
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += CHUNK_KB) {
          const int kb1 = kb0 + CHUNK_KB < num_kb ? kb0 + CHUNK_KB : num_kb;
          if (!ptx::mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t d_main = tmem_base + acc * BN;
          const uint32_t d_small = tmem_base + (2 + acc) * BN;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!ptx::mbar_wait_bounded(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t sa = base + stage * STAGE;
            const uint32_t sb = sa + 2 * A_TILE;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
              const uint32_t first = (kb == kb0 && kk == 0) ? 0u : 1u;
              const uint64_t a_hi = ptx::umma_desc_k_sw128(sa) + 2u * kk;
              const uint64_t a_lo = ptx::umma_desc_k_sw128(sa + A_TILE) + 2u * kk;
              const uint64_t b_hi = ptx::umma_desc_k_sw128(sb) + 2u * kk;
              const uint64_t b_lo = ptx::umma_desc_k_sw128(sb + B_TILE) + 2u * kk;
              ptx::umma_tf32(d_small, a_lo, b_hi, IDESC, first);
              ptx::umma_tf32(d_small, a_hi, b_lo, IDESC, 1);
              ptx::umma_tf32(d_main, a_hi, b_hi, IDESC, first);
            }
            ptx::umma_commit(empty_bar(stage));
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!ok) break;
          ptx::umma_commit(tfull_bar(acc));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const uint32_t stg = base + OUT_OFF + (uint32_t)q * OUT_WARP;
    const bool even_n = (N % BN) == 0;  // every tile stores two halves: one may drain while the other fills
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      const int row0 = m0 + q * 32;
      // lane j holds the bias of channels n0 + j and n0 + 32 + j (handed round by shuffles below)
      float bias0 = 0.0f, bias1 = 0.0f;
      if (staged_out) {
        bias0 = epi.bias_at(n0 + lane, N);
        bias1 = epi.bias_at(n0 + 32 + lane, N);
      }
      float sum[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) sum[j] = 0.0f;
      for (int kb0 = 0; kb0 < num_kb; kb0 += CHUNK_KB) {
        ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS, 4 * POLL_SLEEP_NS);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32], w[32];
          ptx::tmem_ld_32x32(lane_base + acc * BN + c * 32, v);
          ptx::tmem_ld_32x32(lane_base + (2 + acc) * BN + c * 32, w);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            sum[c * 32 + j] = __fadd_rn(sum[c * 32 + j], __fadd_rn(__uint_as_float(v[j]), __uint_as_float(w[j])));
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(tempty_bar(acc));
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) break;
      if (staged_out) {
        // The 32 rows of this warp are one run of pixels of one image (the host checked that the
        // pixels of an image are a multiple of 32): write them channel-major into this warp's
        // staging pieces and let TMA stores put them into the NCHW output as runs of 128 bytes.
        // (Storing from registers, one 128-byte piece per instruction 4 KB apart, took 14 k cycles
        // per tile and made the epilogue the bound of the whole kernel.)  No warp waits for another.
        if (row0 < M) {
          const int img = row0 / epi.P, p0 = row0 - img * epi.P;
#pragma unroll
          for (int h = 0; h < BN / 32; ++h) {
            if (n0 + 32 * h >= N) break;
            const uint32_t s_y = stg + (uint32_t)h * (2 * OUT_PIECE) + (uint32_t)lane * 4u, s_pre = s_y + OUT_PIECE;
            if (lane == 0) {  // the stores that last read this half have finished reading
              if (even_n)
                ptx::bulk_wait_read<1>();
              else
                ptx::bulk_wait_read<0>();
            }
            __syncwarp();
            const float bh = h ? bias1 : bias0;
            // (flags copied out of the parameter struct: each store below is an asm statement that
            // clobbers memory, after which the compiler reloads whatever it reads from epi)
            const bool has_pre = epi.pre != nullptr, relu = epi.relu != 0, has_bias = epi.bias != nullptr;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float bj = __shfl_sync(0xffffffffu, bh, j);
              const float o = has_bias ? __fadd_rn(sum[h * 32 + j], bj) : sum[h * 32 + j];
              if (has_pre) ptx::st_shared_f32(s_pre + (uint32_t)j * 128u, o);
              ptx::st_shared_f32(s_y + (uint32_t)j * 128u, relu && o < 0.f ? 0.f : o);
            }
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
              const uint32_t piece = stg + (uint32_t)h * (2 * OUT_PIECE);
              if (epi.pre) ptx::tma_store_3d(&tm.out[1], p0, n0 + 32 * h, img, piece + OUT_PIECE);
              ptx::tma_store_3d(&tm.out[0], p0, n0 + 32 * h, img, piece);
              ptx::bulk_commit_group();
            }
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(sum[c * 32 + j]);
          epi(row0 + lane, n0 + c * 32, v, M, N, 0);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ gather (A planes)
    const int gt = threadIdx.x - 32 * (2 + EPI_WARPS);
    const int r = gt & (BM - 1);   // tile row of this thread, 0..127
    const int kh0 = (gt / BM) * HB;  // its half of the K block: elements kh0 .. kh0 + HB - 1
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    // The (tile, K block) pairs of this CTA form one sequence, and the loads run two items ahead of
    // the stores across tile boundaries as well (restarting the pipeline at every tile left two
    // load latencies exposed per tile: most of the time of a layer with one K block per tile).
    const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int total = my_tiles * num_kb;
    int l_tile = blockIdx.x, l_kb = 0;  // the item the next load belongs to
    uint32_t valid = 0u;                // bit t: tap t of this row's pixel lies inside the image (at most 32 taps)
    int img = 0;                        // element index of (b, channel 0, y0, x0); the tensor has < 2^31 elements
    auto locate = [&](int tile) {       // position of this thread's row in `tile`; rows past M produce zeros
      const int m = (tile % tiles_m) * BM + r;
      valid = 0u;
      img = 0;
      if (m < M) {
        const int per = g.Ho * g.Wo;
        const int b = m / per, p = m - b * per;
        const int y = p / g.Wo, x = p - y * g.Wo;
        const int y0 = y * g.sy, x0 = x * g.sx;
        img = (b * g.Cs * g.Hs + y0) * g.Ws + x0;
        for (int t = 0; t < taps; ++t) {
          const int a = t / g.kw, bb = t - a * g.kw;
          const int yy = y0 + g.dy0 + g.dsign * a, xx = x0 + g.dx0 + g.dsign * bb;
          if ((unsigned)yy < (unsigned)g.Hs && (unsigned)xx < (unsigned)g.Ws) valid |= 1u << t;
        }
      }
    };
    if (total > 0) locate(l_tile);
    {
      // the 32 values of this row for K block kb: all loads are issued before anything waits on
      // them, and the next block's loads are in flight while this one is split and stored
      const bool one_tap = (g.Cs % BK) == 0;  // every K block lies inside one tap
      const int plane = g.Hs * g.Ws;
      auto load_kb = [&](int kb, float (&v)[HB]) {
        if (one_tap) {
          const int2 e = ktab[kb * BK + kh0];  // this thread's first column: its channel's offset, the tap's bit
          if (valid & (uint32_t)e.y) {
            const float* p = src + (img + e.x);
#pragma unroll
            for (int j = 0; j < HB; ++j) v[j] = __ldg(p + (size_t)j * plane);
          } else {
#pragma unroll
            for (int j = 0; j < HB; ++j) v[j] = 0.0f;
          }
          return;
        }
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const int2 e = ktab[kb * BK + kh0 + j];
          v[j] = 0.0f;
          if (valid & (uint32_t)e.y) v[j] = __ldg(src + (img + e.x));  // skipping the load beat loading a dummy
        }
      };
      // splits one K block held in v and stores it into the current stage
      auto store_kb = [&](const float (&v)[HB]) -> bool {
        bool good = ptx::mbar_wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS);
        good = __all_sync(0xffffffffu, good);
        if (!good) return false;
        const uint32_t row_hi = base + stage * STAGE + (uint32_t)r * ROW_BYTES;
        const uint32_t row_lo = row_hi + A_TILE;
#pragma unroll
        for (int q4 = 0; q4 < HB / 4; ++q4) {
          float hi[4], lo[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) f32::split1(v[q4 * 4 + j], hi[j], lo[j]);
          const uint32_t c4 = (uint32_t)(kh0 / 4 + q4);
          const uint32_t off = (c4 ^ ((uint32_t)r & 7u)) << 4;  // 128-byte swizzle of the 16-byte piece
          ptx::st_shared_v4(row_hi + off, __float_as_uint(hi[0]), __float_as_uint(hi[1]), __float_as_uint(hi[2]),
                            __float_as_uint(hi[3]));
          ptx::st_shared_v4(row_lo + off, __float_as_uint(lo[0]), __float_as_uint(lo[1]), __float_as_uint(lo[2]),
                            __float_as_uint(lo[3]));
        }
        ptx::fence_proxy_async();  // this thread's tile rows become visible to the tensor core
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(full_bar(stage));
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
        return true;
      };
      // Three register buffers rotate: the loads of the next two K blocks are in flight while one is
      // split and stored.  (Copying buffers over instead of rotating them made every iteration wait
      // for the loads it had just issued.)
      auto load_next = [&](float (&v)[HB]) {
        load_kb(l_kb, v);
        if (++l_kb == num_kb) {
          l_kb = 0;
          l_tile += gridDim.x;
          if (l_tile < num_tiles) locate(l_tile);
        }
      };
      float va[HB], vb[HB], vc[HB];
      if (total > 0) load_next(va);
      if (total > 1) load_next(vb);
      for (int i = 0; i < total && ok; i += 3) {
        if (i + 2 < total) load_next(vc);
        ok = store_kb(va);
        if (!ok || i + 1 >= total) break;
        if (i + 3 < total) load_next(va);
        ok = store_kb(vb);
        if (!ok || i + 2 >= total) break;
        if (i + 4 < total) load_next(vb);
        ok = store_kb(vc);
      }
    }
  }

  // ------------------------------------------------------------ teardown
  if (warp >= 2 && warp < 2 + EPI_WARPS && lane == 0) ptx::bulk_wait_read_all();  // staged stores have left shared memory
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(status, VTLB_ST_GEMM_TIMEOUT);
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// B planes: [N rows, ld >= K] hi and lo, K-major (as f32::split_operand writes them)
template <class Epi>
int launch(vtlb_ctx* ctx, const float* src, const Geometry& g, const float* b_hi, const float* b_lo, int ldb,
           const Epi& epi, int M, int N) {
  static_assert(SMEM_TOTAL <= 232448, "shared memory budget");
  gemm::TmapSet tm;
  int rc;
  // outputs go through staged TMA stores when every tile lies inside one image
  const int staged = (epi.P % 32 == 0) && vtlb_aligned16(epi.Y) && (!epi.pre || vtlb_aligned16(epi.pre));
  if (staged) {
    const uint64_t images = (uint64_t)M / epi.P;
    if ((rc = gemm::encode_tmap_3d_f32_plain(ctx, &tm.out[0], epi.Y, epi.P, epi.O, images, 32, 32))) return rc;
    tm.out[1] = tm.out[0];
    if (epi.pre && (rc = gemm::encode_tmap_3d_f32_plain(ctx, &tm.out[1], epi.pre, epi.P, epi.O, images, 32, 32)))
      return rc;
  }
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[0], true, b_hi, g.K, N, (uint64_t)ldb * 4, 32, BN))) return rc;
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[1], true, b_lo, g.K, N, (uint64_t)ldb * 4, 32, BN))) return rc;
  auto kern = conv_igemm_kernel<Epi>;
  static std::atomic<uint64_t> configured{0};
  if (!(configured.load(std::memory_order_relaxed) >> (ctx->device & 63) & 1)) {
    VTLB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_TOTAL));
    configured.fetch_or(1ull << (ctx->device & 63), std::memory_order_relaxed);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  const bool timed = ctx->prof_on && ctx->prof_ev && ctx->prof_n < vtlb_ctx::kProfSlots;
  if (timed) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
  kern<<<grid, NUM_THREADS, SMEM_TOTAL, ctx->stream>>>(src, g, tm, epi, M, N, staged, ctx->d_status);
  if (timed) {
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
    ctx->prof_flops += 2.0 * M * N * g.K;
  }
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace igemm
