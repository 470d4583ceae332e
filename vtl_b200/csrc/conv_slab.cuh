// Unit-stride convolution on tcgen05 (f32 as 3xTF32) from a shared-memory slab of the source.
//
// conv_igemm.cuh gathers every A element once per tap: nine loads, splits and stores per source
// value of a 3x3 window.  Here a tile stages its piece of the source ONCE, as rows of 32 channels:
//   slab row p  <->  position q0 + p of the zero-padded source grid, row-major with pitch
//                    Wp = Wo + kw - 1 (a pixel's 32 channels are one 128-byte row, written with
//                    the 128-byte swizzle the MMA expects)
// and the output positions of the tile are 128 consecutive positions q0 .. q0 + 127 of the same
// grid.  The A operand of tap (a, b) is then the same slab read from row (dy - dy_min) * Wp +
// (dx - dx_min) on: only the start address of the shared-memory descriptor moves, by whole rows.
// (The swizzle is a function of the shared-memory address bits, so a descriptor may start at any
// row of a 1024-byte aligned slab.)  Positions in the kw - 1 padding columns of a grid row
// produce accumulator rows nobody reads; a tile is R = 128 / Wp whole output rows, whose pixels are
// one contiguous run of every channel plane of the NCHW output.
//
// k runs (channel group of 32, tap, channel): K block kb of the regrouped weight planes
// (k = tap * Cs + channel) is tap * G + group.  A source with Cs = 32 G channels takes G slabs per
// tile, one after the other into the same accumulators.
//
// One persistent CTA per SM, 448 threads: warp 0 = TMA producer for the weights, warp 1 = MMA
// issuer and tensor-memory owner, warps 2..5 = epilogue, warps 6..13 = slab fill (lane = slab row,
// so a load instruction reads consecutive pixels of an image row; the next slab's loads are in
// flight while the current one is split and stored).  Two slabs alternate.  All waits are bounded.
#pragma once
#include "conv_igemm.cuh"

namespace cslab {

using gemm::BM;
using gemm::ROW_BYTES;
using gemm::WAIT_LIMIT_NS;
using igemm::Geometry;

constexpr int BN = 64;
constexpr int MAX_B_STAGES = 6;  // as many weight stages as the shared memory left by the staging tiles holds
constexpr int EPI_WARPS = 4, FILL_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * (EPI_WARPS + FILL_WARPS);
constexpr uint32_t POLL_SLEEP_NS = 40;
constexpr int SLAB_ROWS = 200;  // 128 positions + the largest tap shift: (kh - 1) * Wp + kw - 1 <= 72
constexpr uint32_t SLAB_PLANE = SLAB_ROWS * ROW_BYTES;  // hi or lo part: 25 x 1024 bytes
constexpr uint32_t SLAB = 2 * SLAB_PLANE;
constexpr uint32_t B_TILE = BN * ROW_BYTES, B_STAGE = 2 * B_TILE;
// Layout: two slabs | one or two staging tiles [BN channels][R * Wo pixels] f32 (output, pre-activation)
// | weight stages | barriers, tensor-memory slot, tap table.
constexpr uint32_t OUT_OFF = 2 * SLAB;
constexpr int NUM_BARS = 2 * MAX_B_STAGES + 4 + 4 + 1;  // weights full/empty, slab full/empty, tfull/tempty, epilogue
constexpr int MAX_TAPS = 32;
constexpr uint32_t TAIL_BYTES = 8 * NUM_BARS + 16 + 4 * MAX_TAPS;
constexpr uint32_t SMEM_MAX = 232448;
static_assert(SLAB_PLANE % 1024 == 0, "slab planes must keep the swizzle phase");

struct Tiling {
  int Wp;             // pitch of the padded grid
  int R;              // output rows per tile
  int tiles_per_img;  // ceil(Ho / R)
  int dy_min, dx_min;
  int G;              // channel groups of 32
  int b_stages;       // weight stages (launch() fills these three in)
  uint32_t out_tile;  // bytes of one staging tile, a multiple of 1024
  uint32_t b_off;     // offset of the weight stages
};

inline bool usable(const Geometry& g, Tiling* t) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("VTLB_CONV_SLAB");
    env = e ? atoi(e) : 1;
  }
  if (!env || g.sy != 1 || g.sx != 1 || g.Cs % 32 != 0 || g.Wo % 4 != 0) return false;
  t->Wp = g.Wo + g.kw - 1;
  if (t->Wp > BM) return false;
  if (BM + (g.kh - 1) * t->Wp + g.kw - 1 > SLAB_ROWS || g.kh * g.kw > MAX_TAPS) return false;
  t->R = BM / t->Wp;
  t->tiles_per_img = (g.Ho + t->R - 1) / t->R;
  const int dy_end = g.dy0 + g.dsign * (g.kh - 1), dx_end = g.dx0 + g.dsign * (g.kw - 1);
  t->dy_min = g.dy0 < dy_end ? g.dy0 : dy_end;
  t->dx_min = g.dx0 < dx_end ? g.dx0 : dx_end;
  t->G = g.Cs / 32;
  return true;
}

template <class Epi>
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_slab_kernel(const float* __restrict__ src, const Geometry g, const Tiling tl,
                 const __grid_constant__ gemm::TmapSet tm, const Epi epi, int N, uint32_t* status) {
  constexpr int BK = 32, KSTEPS = 4, CHUNK_KB = 4;
  // Two buffers of three accumulators each: a_hi.b_hi | a_hi.b_lo (one MMA writes both) and a_lo.b_hi.
  constexpr uint32_t ACC_COLS = 3 * BN;
  constexpr uint32_t TMEM_COLS = 512;  // 2 * ACC_COLS rounded up to a power of two
  constexpr uint32_t IDESC = ptx::umma_idesc(ptx::kCfmtF32, ptx::kFmtTF32, BM, BN);
  constexpr uint32_t IDESC2 = ptx::umma_idesc(ptx::kCfmtF32, ptx::kFmtTF32, BM, 2 * BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t B_STAGES = (uint32_t)tl.b_stages, B_OFF = tl.b_off;
  const uint32_t bars = base + B_OFF + B_STAGES * B_STAGE;
  auto bfull_bar = [&](int s) { return bars + 8u * s; };
  auto bempty_bar = [&](int s) { return bars + 8u * (MAX_B_STAGES + s); };
  auto sfull_bar = [&](int s) { return bars + 8u * (2 * MAX_B_STAGES + s); };
  auto sempty_bar = [&](int s) { return bars + 8u * (2 * MAX_B_STAGES + 2 + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * MAX_B_STAGES + 4 + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * MAX_B_STAGES + 6 + a); };
  const uint32_t epi_bar = bars + 8u * (2 * MAX_B_STAGES + 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars - raw) + 8u * NUM_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint32_t* shift_tab = tmem_slot + 4;  // per tap: its row shift in the slab, in descriptor units (16 bytes)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = g.kh * g.kw;
  const int tiles_m = g.B * tl.tiles_per_img, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kb_per_tile = tl.G * taps;  // K blocks of 32 accumulated into one tile

  if (threadIdx.x < taps) {
    const int a = threadIdx.x / g.kw, b = threadIdx.x - a * g.kw;
    const int shift = (g.dy0 + g.dsign * a - tl.dy_min) * tl.Wp + (g.dx0 + g.dsign * b - tl.dx_min);
    shift_tab[threadIdx.x] = (uint32_t)shift * (ROW_BYTES >> 4);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < (int)B_STAGES; ++s) {
      ptx::mbar_init(bfull_bar(s), 1);
      ptx::mbar_init(bempty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(sfull_bar(s), FILL_WARPS);
      ptx::mbar_init(sempty_bar(s), 1);
      ptx::mbar_init(tfull_bar(s), 1);
      ptx::mbar_init(tempty_bar(s), 32 * EPI_WARPS);
    }
    ptx::mbar_init(epi_bar, 32 * EPI_WARPS);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
    ptx::prefetch_tmap(&tm.b[0]);
    ptx::prefetch_tmap(&tm.b[1]);
    ptx::prefetch_tmap(&tm.out[0]);
    ptx::prefetch_tmap(&tm.out[1]);
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
    // ------------------------------------------------------------ TMA producer (weight planes)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int n0 = (tile / tiles_m) * BN;
        for (int i = 0; i < kb_per_tile; ++i) {
          const int grp = i / taps, tap = i - grp * taps;
          const int kb = tap * tl.G + grp;
          if (!ptx::mbar_wait_bounded(bempty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(bfull_bar(stage), B_STAGE);
          const uint32_t sb = base + B_OFF + stage * B_STAGE;
          ptx::tma_load_2d(sb, &tm.b[0], kb * BK, n0, bfull_bar(stage));
          ptx::tma_load_2d(sb + B_TILE, &tm.b[1], kb * BK, n0, bfull_bar(stage));
          if (++stage == B_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0, slab = 0, slab_phase = 0;
      bool ok = true;
      // Two MMAs per K step: the hi and lo planes of the weights lie back to back in a stage, so
      // a_hi . [b_hi; b_lo] is one MMA of 2 BN columns (main term | a_hi . b_lo) and a_lo . b_hi goes
      // to the third accumulator.  At BN = 64 an MMA is bound by fetching its operands from shared
      // memory (the 4 KB of A above all): this reads 14 KB per K step instead of 18.
      const uint64_t desc0 = ptx::umma_desc_k_sw128(base);  // + (byte offset >> 4) selects a tile and a row
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        uint32_t d_main = 0;
        int i = 0;  // K block of this tile
        for (int grp = 0; grp < tl.G && ok; ++grp) {
          // the slab of this channel group
          if (!ptx::mbar_wait_bounded(sfull_bar(slab), slab_phase, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
            ok = false;
            break;
          }
          const uint64_t slab_desc = desc0 + ((slab * SLAB) >> 4);
          for (int tap = 0; tap < taps; ++tap, ++i) {
            const bool chunk_start = (i % CHUNK_KB) == 0;
            if (chunk_start) {  // a new accumulator chunk
              if (!ptx::mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
                ok = false;
                break;
              }
              d_main = tmem_base + acc * ACC_COLS;
            }
            if (!ptx::mbar_wait_bounded(bfull_bar(stage), phase, abort_flag, WAIT_LIMIT_NS, POLL_SLEEP_NS)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint64_t a_hi = slab_desc + shift_tab[tap];  // rows shifted by the tap: ROW_BYTES >> 4 per row
            const uint64_t a_lo = a_hi + (SLAB_PLANE >> 4);
            const uint64_t b_hl = desc0 + ((B_OFF + stage * B_STAGE) >> 4);  // 2 BN rows: b_hi, then b_lo
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
              const uint32_t accumulate = (chunk_start && kk == 0) ? 0u : 1u;
              ptx::umma_tf32(d_main, a_hi + 2u * kk, b_hl + 2u * kk, IDESC2, accumulate);
              ptx::umma_tf32(d_main + 2 * BN, a_lo + 2u * kk, b_hl + 2u * kk, IDESC, accumulate);
            }
            ptx::umma_commit(bempty_bar(stage));
            if (++stage == B_STAGES) {
              stage = 0;
              phase ^= 1u;
            }
            if (i % CHUNK_KB == CHUNK_KB - 1 || i == kb_per_tile - 1) {
              ptx::umma_commit(tfull_bar(acc));
              acc ^= 1u;
              if (acc == 0) acc_phase ^= 1u;
            }
          }
          if (!ok) break;
          ptx::umma_commit(sempty_bar(slab));  // the slab may be refilled once these MMAs have read it
          slab ^= 1u;
          if (slab == 0) slab_phase ^= 1u;
        }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint32_t acc = 0, acc_phase = 0, epi_phase = 0;
    bool ok = true;
    const int m = q * 32 + lane;                 // this thread's position inside a tile
    const int pr = m / tl.Wp, pc = m - pr * tl.Wp;  // row of the tile, column of the padded grid
    const int rw = tl.R * g.Wo;                  // pixels of a full tile = pitch of the staging tile
    const uint32_t stg_y = base + OUT_OFF, stg_pre = stg_y + tl.out_tile;
    auto meet = [&]() -> bool {  // bounded rendezvous of the 128 epilogue threads
      ptx::mbar_arrive(epi_bar);
      const bool good = ptx::mbar_wait_bounded(epi_bar, epi_phase, abort_flag, WAIT_LIMIT_NS);
      epi_phase ^= 1u;
      return __all_sync(0xffffffffu, good);
    };
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tm_i = tile % tiles_m, n0 = (tile / tiles_m) * BN;
      const int img = tm_i / tl.tiles_per_img, y0 = (tm_i - img * tl.tiles_per_img) * tl.R;
      const float bias0 = epi.bias_at(n0 + lane, N), bias1 = epi.bias_at(n0 + 32 + lane, N);
      float sum[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) sum[j] = 0.0f;
      for (int c0 = 0; c0 < kb_per_tile; c0 += CHUNK_KB) {
        ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS, 4 * POLL_SLEEP_NS);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < BN / 16; ++c) {
          uint32_t v[16], w1[16], w2[16];
          ptx::tmem_ld_32x16(lane_base + acc * ACC_COLS + c * 16, v);
          ptx::tmem_ld_32x16(lane_base + acc * ACC_COLS + BN + c * 16, w1);
          ptx::tmem_ld_32x16(lane_base + acc * ACC_COLS + 2 * BN + c * 16, w2);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float small = __fadd_rn(__uint_as_float(w1[j]), __uint_as_float(w2[j]));
            sum[c * 16 + j] = __fadd_rn(sum[c * 16 + j], __fadd_rn(__uint_as_float(v[j]), small));
          }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(tempty_bar(acc));
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) break;
      // The tile's pixels are one run of every channel plane: write them channel-major and compact
      // (padding columns dropped) into the staging tiles; one TMA store per tensor writes the runs.
      // Rows past the image are clipped by the store (the innermost extent of the map is Ho * Wo).
      if (warp == 2 && lane == 0) ptx::bulk_wait_read_all();  // the previous tile's stores have read the staging tiles
      if (!(ok = meet())) break;
      // (the flags are copied out of the parameter struct first: every shared-memory store below is an
      // asm statement that clobbers memory, after which the compiler reloads whatever it reads from epi)
      const bool keep = pc < g.Wo && pr < tl.R;
      const bool keep_pre = keep && epi.pre != nullptr, relu = epi.relu != 0, has_bias = epi.bias != nullptr;
      const uint32_t to_pre = tl.out_tile;
      const uint32_t pitch = (uint32_t)rw * 4u;
      uint32_t at = stg_y + (uint32_t)(pr * g.Wo + pc) * 4u;  // a running address: one add per channel
#pragma unroll
      for (int j = 0; j < BN; ++j) {
        const float bj = __shfl_sync(0xffffffffu, j < 32 ? bias0 : bias1, j & 31);
        const float o = has_bias ? __fadd_rn(sum[j], bj) : sum[j];
        if (keep_pre) ptx::st_shared_f32(at + to_pre, o);
        if (keep) ptx::st_shared_f32(at, relu && o < 0.f ? 0.f : o);
        at += pitch;
      }
      ptx::fence_proxy_async();
      if (!(ok = meet())) break;
      if (warp == 2 && lane == 0) {
        if (epi.pre) ptx::tma_store_3d(&tm.out[1], y0 * g.Wo, n0, img, stg_pre);
        ptx::tma_store_3d(&tm.out[0], y0 * g.Wo, n0, img, stg_y);
        ptx::bulk_commit_group();
      }
    }
  } else {
    // ------------------------------------------------------------ slab fill
    // Work items of a slab: (row p, half of the 32 channels), 2 * SLAB_ROWS of them for 256 threads:
    // every thread owns item ft, the first 2 * SLAB_ROWS - 256 threads also item ft + 256.
    const int ft = threadIdx.x - 32 * (2 + EPI_WARPS);
    constexpr int HB = 16;
    constexpr int ITEMS = 2 * SLAB_ROWS;
    const bool two = ft + 256 < ITEMS;
    const int p0 = ft % SLAB_ROWS, h0 = ft / SLAB_ROWS;
    const int p1 = (ft + 256) % SLAB_ROWS, h1 = (ft + 256) / SLAB_ROWS;
    const int r0 = p0 / tl.Wp, c0 = p0 - r0 * tl.Wp, r1 = p1 / tl.Wp, c1 = p1 - r1 * tl.Wp;
    const int plane = g.Hs * g.Ws;
    const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int total = my_tiles * tl.G;  // slabs this CTA fills
    int l_tile = blockIdx.x, l_grp = 0;
    uint32_t slab = 0, slab_phase = 0;
    bool ok = true;

    // loads of one item: 16 channels of one source pixel (zeros outside the image)
    auto load_item = [&](int img, int y0, int grp, int r, int c, int h, float (&v)[HB]) {
      const int ys = y0 + r + tl.dy_min, xs = c + tl.dx_min;
      if ((unsigned)ys < (unsigned)g.Hs && (unsigned)xs < (unsigned)g.Ws) {
        const float* s = src + ((size_t)(img * g.Cs + grp * 32 + h * HB) * g.Hs + ys) * g.Ws + xs;
#pragma unroll
        for (int j = 0; j < HB; ++j) v[j] = __ldg(s + (size_t)j * plane);
      } else {
#pragma unroll
        for (int j = 0; j < HB; ++j) v[j] = 0.0f;
      }
    };
    auto load_next = [&](float (&va)[HB], float (&vb)[HB]) {
      const int tm_i = l_tile % tiles_m;
      const int img = tm_i / tl.tiles_per_img, y0 = (tm_i - img * tl.tiles_per_img) * tl.R;
      load_item(img, y0, l_grp, r0, c0, h0, va);
      if (two) load_item(img, y0, l_grp, r1, c1, h1, vb);
      if (++l_grp == tl.G) {
        l_grp = 0;
        l_tile += gridDim.x;
      }
    };
    auto store_item = [&](uint32_t slab_addr, int p, int h, const float (&v)[HB]) {
      const uint32_t row_hi = slab_addr + (uint32_t)p * ROW_BYTES;
      const uint32_t row_lo = row_hi + SLAB_PLANE;
#pragma unroll
      for (int q4 = 0; q4 < HB / 4; ++q4) {
        float hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) f32::split1(v[q4 * 4 + j], hi[j], lo[j]);
        const uint32_t c4 = (uint32_t)(h * (HB / 4) + q4);
        const uint32_t off = (c4 ^ ((uint32_t)p & 7u)) << 4;  // 128-byte swizzle of the 16-byte piece
        ptx::st_shared_v4(row_hi + off, __float_as_uint(hi[0]), __float_as_uint(hi[1]), __float_as_uint(hi[2]),
                          __float_as_uint(hi[3]));
        ptx::st_shared_v4(row_lo + off, __float_as_uint(lo[0]), __float_as_uint(lo[1]), __float_as_uint(lo[2]),
                          __float_as_uint(lo[3]));
      }
    };
    auto store_slab = [&](const float (&va)[HB], const float (&vb)[HB]) -> bool {
      bool good = ptx::mbar_wait_bounded(sempty_bar(slab), slab_phase ^ 1u, abort_flag, WAIT_LIMIT_NS);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      const uint32_t slab_addr = base + slab * SLAB;
      store_item(slab_addr, p0, h0, va);
      if (two) store_item(slab_addr, p1, h1, vb);
      ptx::fence_proxy_async();  // this thread's rows become visible to the tensor core
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(sfull_bar(slab));
      slab ^= 1u;
      if (slab == 0) slab_phase ^= 1u;
      return true;
    };
    float a0[HB], a1[HB], b0[HB], b1[HB];
    if (total > 0) load_next(a0, a1);
    for (int i = 0; i < total && ok; i += 2) {
      if (i + 1 < total) load_next(b0, b1);
      ok = store_slab(a0, a1);
      if (!ok || i + 1 >= total) break;
      if (i + 2 < total) load_next(a0, a1);
      ok = store_slab(b0, b1);
    }
  }

  // ------------------------------------------------------------ teardown
  if (warp == 2 && lane == 0) ptx::bulk_wait_read_all();  // staged stores have left shared memory
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

// B planes: [N rows, ld >= K] hi and lo, k = tap * Cs + channel (regroup_weights_split_kernel)
template <class Epi>
int launch(vtlb_ctx* ctx, const float* src, const Geometry& g, Tiling tl, const float* b_hi, const float* b_lo,
           int ldb, const Epi& epi, int N) {
  gemm::TmapSet tm;
  int rc;
  const int box_px = tl.R * g.Wo;  // a multiple of 4 pixels (16 bytes), at most 128
  tl.out_tile = (uint32_t)vtlb_round_up((size_t)BN * box_px * 4, 1024);
  tl.b_off = OUT_OFF + (epi.pre ? 2u : 1u) * tl.out_tile;
  tl.b_stages = (int)((SMEM_MAX - 1024 - TAIL_BYTES - tl.b_off) / B_STAGE);
  if (tl.b_stages > MAX_B_STAGES) tl.b_stages = MAX_B_STAGES;
  const uint32_t smem_total = tl.b_off + tl.b_stages * B_STAGE + TAIL_BYTES + 1024;
  if ((rc = gemm::encode_tmap_3d_f32_plain(ctx, &tm.out[0], epi.Y, epi.P, epi.O, g.B, box_px, BN))) return rc;
  tm.out[1] = tm.out[0];
  if (epi.pre && (rc = gemm::encode_tmap_3d_f32_plain(ctx, &tm.out[1], epi.pre, epi.P, epi.O, g.B, box_px, BN)))
    return rc;
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[0], true, b_hi, g.K, N, (uint64_t)ldb * 4, 32, BN))) return rc;
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[1], true, b_lo, g.K, N, (uint64_t)ldb * 4, 32, BN))) return rc;
  auto kern = conv_slab_kernel<Epi>;
  static std::atomic<uint64_t> configured{0};
  if (!(configured.load(std::memory_order_relaxed) >> (ctx->device & 63) & 1)) {
    VTLB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX));
    configured.fetch_or(1ull << (ctx->device & 63), std::memory_order_relaxed);
  }
  const int tiles = g.B * tl.tiles_per_img * ((N + BN - 1) / BN);
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  const bool timed = ctx->prof_on && ctx->prof_ev && ctx->prof_n < vtlb_ctx::kProfSlots;
  if (timed) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
  kern<<<grid, NUM_THREADS, smem_total, ctx->stream>>>(src, g, tl, tm, epi, N, ctx->d_status);
  if (timed) {
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
    ctx->prof_flops += 2.0 * g.B * g.Ho * g.Wo * (double)N * g.K;
  }
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace cslab
