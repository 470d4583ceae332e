// Weight gradient of a unit-stride convolution as an implicit GEMM on tcgen05 (f32 as 3xTF32):
//   dW[o][c][a][b] = sum over (image, y, x) of g[image][o][y][x] * xin[image][c][y + a - ph][x + b - pw]
// (nn/internal/conv2d_backward_cpu_f32.v:56-82).  The contraction runs over pixels, which NCHW
// stores contiguously for both operands, so both are K-major as they lie and nothing is lowered to a
// patch matrix: one K block is one output row (up to 32 pixels) of one image.
//
//   A (M side)  for tap row a: the source row y + a - ph, 32 channels, in kw copies shifted by
//               b - pw pixels: kw tiles of [32 channels][32 pixels], 96 useful of the 128 MMA rows
//   B (N side)  the gradient row: [64 output channels][32 pixels]
//   D           kh accumulators [128 lanes = (b, c)][64 columns = o] in tensor memory
//
// A CTA owns a run of consecutive output rows (of consecutive images) for one group of 32 source
// channels and one block of 64 output channels, keeps the source rows of the last kh output rows in
// a ring of kh + 3 shared-memory slots (each source row is loaded, split into TF32 hi/lo and stored
// once, although kh output rows use it), and writes its sums as one partial dW; a second launch
// adds the partials of all CTAs in a fixed order.  Accumulators are closed every four rows and summed
// in registers, like in the other 3xTF32 kernels (the f32 accumulate of tcgen05 truncates).
//
// 13 warps: warp 0 = MMA issuer and tensor-memory owner; warps 1,2,3,7 fill the source-row window;
// warps 11,12 fill the gradient stages; warps 4,5,6 and 8,9,10 are the epilogue (tensor-memory lane
// quarters 0..2 = the kw shifted copies; the two sets take 32 output channels each).  All waits are
// bounded; a wait that runs out raises the abort flag and the kernel sets the status word.
#pragma once
#include "f32_common.cuh"

namespace cwgrad {

using gemm::ROW_BYTES;
using gemm::WAIT_LIMIT_NS;

constexpr int BO = 64;                 // output channels per CTA
constexpr int MAX_KH = 3, MAX_KW = 3;
constexpr int MAX_SLOTS = MAX_KH + 3;  // source-row window: the kh rows in use and three rows of lead for the fill
constexpr int GS = 4;                  // gradient stages
constexpr int CHUNK_ROWS = 4;          // output rows per accumulator chunk (128 pixels of the contraction)
constexpr int NUM_WARPS = 13, NUM_THREADS = 32 * NUM_WARPS;
constexpr int XFILL_WARPS = 4, GFILL_WARPS = 2, EPI_WARPS = 6;
constexpr uint32_t TILE = 32 * ROW_BYTES;               // one [32 rows][32 pixels] tile: 4 KB
constexpr uint32_t SLOT_PLANE = MAX_KW * TILE;           // hi or lo part of a slot
constexpr uint32_t SLOT = 2 * SLOT_PLANE;                // 24 KB
constexpr uint32_t G_PLANE = BO * ROW_BYTES, G_STAGE = 2 * G_PLANE;  // 16 KB
constexpr uint32_t WINDOW = MAX_SLOTS * SLOT;            // the lo operand of the last slot reads 4 KB past it: into G
constexpr uint32_t G_OFF = WINDOW;
constexpr uint32_t BARS_OFF = G_OFF + GS * G_STAGE;
constexpr int NUM_BARS = 2 * MAX_SLOTS + 2 * GS + 2 + 2;  // xfull, xempty, gfull, gempty, tfull, tempty
constexpr uint32_t SMEM_TOTAL = BARS_OFF + 8 * NUM_BARS + 16 + 1024;
constexpr uint32_t ACC_COLS = MAX_KH * BO;               // one buffer: kh accumulators of 64 columns
constexpr uint32_t TMEM_COLS = 512;                      // two buffers (384) rounded up to a power of two
static_assert(SLOT % 1024 == 0 && G_STAGE % 1024 == 0, "tiles must keep the swizzle phase");

struct Params {
  const float* x;    // [B, C, H, W]
  const float* g;    // [B, O, Ho, Wo]
  float* partial;    // [parts][O][C][kh][kw]
  int B, C, H, W, O, Ho, Wo, kh, kw, ph, pw;
  int rows_total, rows_per_part;
  uint32_t* status;
};

inline bool usable(int sh, int sw, int kh, int kw, int Wo, int dil) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("VTLB_CONV_WGRAD");
    env = e ? atoi(e) : 1;
  }
  return env && dil == 1 && sh == 1 && sw == 1 && kh <= MAX_KH && kw <= MAX_KW && Wo <= 32;
}

__global__ void __launch_bounds__(NUM_THREADS, 1) conv_wgrad_kernel(const Params p) {
  constexpr uint32_t IDESC = ptx::umma_idesc(ptx::kCfmtF32, ptx::kFmtTF32, 128, BO);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + BARS_OFF;
  auto xfull_bar = [&](int s) { return bars + 8u * s; };
  auto xempty_bar = [&](int s) { return bars + 8u * (MAX_SLOTS + s); };
  auto gfull_bar = [&](int s) { return bars + 8u * (2 * MAX_SLOTS + s); };
  auto gempty_bar = [&](int s) { return bars + 8u * (2 * MAX_SLOTS + GS + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * MAX_SLOTS + 2 * GS + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * MAX_SLOTS + 2 * GS + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bars - raw) + 8u * NUM_BARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kh = p.kh, kw = p.kw, nslots = kh + 3;
  const int grp = blockIdx.y, ob = blockIdx.z;
  const int row_begin = blockIdx.x * p.rows_per_part;
  const int row_end = row_begin + p.rows_per_part < p.rows_total ? row_begin + p.rows_per_part : p.rows_total;
  const int R = row_end - row_begin;  // > 0 by construction of the grid

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_SLOTS; ++s) {
      ptx::mbar_init(xfull_bar(s), XFILL_WARPS);
      ptx::mbar_init(xempty_bar(s), 1);
    }
    for (int s = 0; s < GS; ++s) {
      ptx::mbar_init(gfull_bar(s), GFILL_WARPS);
      ptx::mbar_init(gempty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 32 * EPI_WARPS);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 0) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early: the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Output row i of this CTA (i = 0 .. R-1) is row y of image img; the first row of the CTA and the
  // first row of every image start a new window (kh source rows to fill), every other row adds one.
  // Source rows are numbered in the order they are filled ("count"); count n lives in slot n % nslots.
  auto row_of = [&](int i, int& img, int& y) {
    const int gr = row_begin + i;
    img = gr / p.Ho;
    y = gr - img * p.Ho;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // One thread issues everything: no divisions (slots, stages and rows advance by counters), and the
      // waits for the NEXT row's operands sit between the tap rows of the current one, while MMAs are
      // queued.  (Measured: the kernel is bound by the tensor core fetching its operands from shared
      // memory, 36 MMAs of 4 KB + 2 KB per output row at about 70 bytes per clock; issuing the commits
      // later, behind the next row's first MMAs, changed nothing.)
      const uint64_t desc0 = ptx::umma_desc_k_sw128(base);
      uint32_t acc = 0, acc_phase = 0;
      uint32_t xs = 0, xph = 0;    // slot and parity of the next source row to wait for
      uint32_t gs = 0, gph = 0;    // stage and parity of the next gradient row to wait for
      bool ok = true;
      auto wait_operands = [&](bool first) -> bool {  // of the row that is issued next
        const int need = first ? kh : 1;
        for (int k = 0; k < need; ++k) {
          if (!ptx::mbar_wait_bounded(xfull_bar((int)xs), xph, abort_flag, WAIT_LIMIT_NS)) return false;
          if (++xs == (uint32_t)nslots) {
            xs = 0;
            xph ^= 1u;
          }
        }
        if (!ptx::mbar_wait_bounded(gfull_bar((int)gs), gph, abort_flag, WAIT_LIMIT_NS)) return false;
        if (++gs == (uint32_t)GS) {
          gs = 0;
          gph ^= 1u;
        }
        return true;
      };
      auto issue_tap = [&](uint32_t slot, uint32_t d, uint64_t b_hi, uint64_t b_lo, bool fresh) {
        const uint64_t a_hi = desc0 + ((slot * SLOT) >> 4);
        const uint64_t a_lo = a_hi + (SLOT_PLANE >> 4);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          ptx::umma_tf32(d, a_lo + 2u * kk, b_hi + 2u * kk, IDESC, (fresh && kk == 0) ? 0u : 1u);  // small terms first
          ptx::umma_tf32(d, a_hi + 2u * kk, b_lo + 2u * kk, IDESC, 1u);
          ptx::umma_tf32(d, a_hi + 2u * kk, b_hi + 2u * kk, IDESC, 1u);
        }
      };
      auto wrap = [&](uint32_t s_) { return s_ >= (uint32_t)nslots ? s_ - (uint32_t)nslots : s_; };
      int y = row_begin - (row_begin / p.Ho) * p.Ho;
      uint32_t slot0 = 0, gcur = 0;  // window slot of tap row 0 and gradient stage of the current row
      int in_chunk = 0;
      ok = wait_operands(true);
      for (int i = 0; i < R && ok; ++i) {
        const bool chunk_start = in_chunk == 0;
        if (chunk_start && !ptx::mbar_wait_bounded(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint64_t b_hi = desc0 + ((G_OFF + gcur * G_STAGE) >> 4);
        const uint64_t b_lo = b_hi + (G_PLANE >> 4);
        const uint32_t d0 = tmem_base + acc * ACC_COLS;
        for (int a = 0; a + 1 < kh; ++a) issue_tap(wrap(slot0 + (uint32_t)a), d0 + (uint32_t)a * BO, b_hi, b_lo, chunk_start);
        // the next row: where its window starts, and its operands (normally long there)
        const bool has_next = i + 1 < R;
        const int y_next = y + 1 == p.Ho ? 0 : y + 1;
        const bool first_next = y_next == 0;
        const uint32_t slot0_next = first_next ? xs : wrap(slot0 + 1u);
        const uint32_t g_next = gs;
        if (has_next && !wait_operands(first_next)) {
          ok = false;
          break;
        }
        issue_tap(wrap(slot0 + (uint32_t)(kh - 1)), d0 + (uint32_t)(kh - 1) * BO, b_hi, b_lo, chunk_start);
        // once these MMAs have read their operands the gradient stage is free, and so are the window
        // slots no later row reads: the oldest source row, or all kh when the next output row starts a
        // new window (first row of the next image) or there is none
        ptx::umma_commit(gempty_bar((int)gcur));
        const int freed = (!has_next || first_next) ? kh : 1;
        for (int a = 0; a < freed; ++a) ptx::umma_commit(xempty_bar((int)wrap(slot0 + (uint32_t)a)));
        if (++in_chunk == CHUNK_ROWS || !has_next) {
          in_chunk = 0;
          ptx::umma_commit(tfull_bar(acc));
          acc ^= 1u;
          if (acc == 0) acc_phase ^= 1u;
        }
        y = y_next;
        slot0 = slot0_next;
        gcur = g_next;
      }
    }
  } else if (warp == 1 || warp == 2 || warp == 3 || warp == 7) {
    // ------------------------------------------------------------ source-row window
    // 128 threads: thread = (channel c, eight pixels 8j .. 8j+7).  It loads the 8 + kw - 1 source pixels
    // its eight positions see through the kw horizontal taps and writes them, split into hi / lo, as two
    // 16-byte pieces of row c of each of the kw shifted tiles.
    const int ft = (warp == 7 ? 3 : warp - 1) * 32 + lane;
    const int c = ft >> 2, j = ft & 3;
    const int cg = grp * 32 + c;
    constexpr int NV = 8 + MAX_KW - 1;
    auto load_row = [&](int img, int r, float (&v)[NV]) {
      const bool row_ok = cg < p.C && (unsigned)r < (unsigned)p.H;
      const float* s = p.x + ((size_t)(img * p.C + (row_ok ? cg : 0)) * p.H + (row_ok ? r : 0)) * p.W;
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        const int px = 8 * j - p.pw + e;
        v[e] = (row_ok && e < 8 + kw - 1 && (unsigned)px < (unsigned)p.W) ? __ldg(s + px) : 0.0f;
      }
    };
    auto store_row = [&](uint32_t slot_addr, const float (&v)[NV]) {
      for (int b = 0; b < kw; ++b) {
        const uint32_t row_hi = slot_addr + (uint32_t)b * TILE + (uint32_t)c * ROW_BYTES;
        const uint32_t row_lo = row_hi + SLOT_PLANE;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float val = v[0];
#pragma unroll
            for (int t = 0; t < MAX_KW; ++t)  // v[4h + e + b] without a run-time register index
              if (t == b) val = v[4 * h + e + t];
            f32::split1(val, hi[e], lo[e]);
          }
          const uint32_t off = (((uint32_t)(2 * j + h)) ^ ((uint32_t)c & 7u)) << 4;
          ptx::st_shared_v4(row_hi + off, __float_as_uint(hi[0]), __float_as_uint(hi[1]), __float_as_uint(hi[2]),
                            __float_as_uint(hi[3]));
          ptx::st_shared_v4(row_lo + off, __float_as_uint(lo[0]), __float_as_uint(lo[1]), __float_as_uint(lo[2]),
                            __float_as_uint(lo[3]));
        }
      }
    };
    // the source rows in the order they are filled: (image, source row)
    int it_i = 0, it_a = 0;  // next item: output row it_i, tap row it_a
    auto next_item = [&](int& img, int& r) -> bool {
      if (it_i >= R) return false;
      int y;
      row_of(it_i, img, y);
      const bool first = it_i == 0 || y == 0;
      if (it_a == 0 && !first) it_a = kh - 1;
      r = y - p.ph + it_a;
      if (++it_a == kh) {
        it_a = 0;
        ++it_i;
      }
      return true;
    };
    // Three rows in registers: the loads of the two rows after the one being stored are in flight
    // (a row period is about the latency of one load from HBM).  The buffers rotate by name, not by
    // copying: a copy would wait for the newest load.
    int count = 0;
    bool ok = true;
    auto fetch = [&](float (&v)[NV]) -> bool {
      int img, r;
      if (!next_item(img, r)) return false;
      load_row(img, r, v);
      return true;
    };
    auto put = [&](const float (&v)[NV]) -> bool {
      const int slot = count % nslots;
      bool good = ptx::mbar_wait_bounded(xempty_bar(slot), ((uint32_t)(count / nslots) & 1u) ^ 1u, abort_flag,
                                         WAIT_LIMIT_NS);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      store_row(base + (uint32_t)slot * SLOT, v);
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(xfull_bar(slot));
      ++count;
      return true;
    };
    float v0[NV], v1[NV], v2[NV];
    bool h0 = fetch(v0), h1 = h0 && fetch(v1), h2 = false;
    while (h0 && ok) {
      h2 = h1 && fetch(v2);
      ok = put(v0);
      if (!ok || !h1) break;
      h0 = h2 && fetch(v0);
      ok = put(v1);
      if (!ok || !h2) break;
      h1 = h0 && fetch(v1);
      ok = put(v2);
    }
  } else if (warp == 11 || warp == 12) {
    // ------------------------------------------------------------ gradient stages
    // 64 threads: thread = output channel; the whole row of up to 32 pixels, zeros past Wo.
    const int o = (warp - 11) * 32 + lane;
    const int og = ob * BO + o;
    const bool vec = (p.Wo & 3) == 0 && (((uintptr_t)p.g) & 15u) == 0;
    auto load_row = [&](int i, float (&v)[32]) {
      int img, y;
      row_of(i, img, y);
      const bool ok_o = og < p.O;
      const float* s = p.g + ((size_t)(img * p.O + (ok_o ? og : 0)) * p.Ho + y) * p.Wo;
      if (vec) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
          if (ok_o && 4 * q < p.Wo) t = __ldg(reinterpret_cast<const float4*>(s) + q);
          v[4 * q] = t.x;
          v[4 * q + 1] = t.y;
          v[4 * q + 2] = t.z;
          v[4 * q + 3] = t.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = (ok_o && e < p.Wo) ? __ldg(s + e) : 0.0f;
      }
    };
    auto store_row = [&](uint32_t stage_addr, const float (&v)[32]) {
      const uint32_t row_hi = stage_addr + (uint32_t)o * ROW_BYTES, row_lo = row_hi + G_PLANE;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) f32::split1(v[4 * q + e], hi[e], lo[e]);
        const uint32_t off = (((uint32_t)q) ^ ((uint32_t)o & 7u)) << 4;
        ptx::st_shared_v4(row_hi + off, __float_as_uint(hi[0]), __float_as_uint(hi[1]), __float_as_uint(hi[2]),
                          __float_as_uint(hi[3]));
        ptx::st_shared_v4(row_lo + off, __float_as_uint(lo[0]), __float_as_uint(lo[1]), __float_as_uint(lo[2]),
                          __float_as_uint(lo[3]));
      }
    };
    bool ok = true;
    int loaded = 0, stored = 0;
    auto fetch = [&](float (&v)[32]) -> bool {
      if (loaded >= R) return false;
      load_row(loaded++, v);
      return true;
    };
    auto put = [&](const float (&v)[32]) -> bool {
      const int i = stored;
      bool good = ptx::mbar_wait_bounded(gempty_bar(i % GS), ((uint32_t)(i / GS) & 1u) ^ 1u, abort_flag, WAIT_LIMIT_NS);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      store_row(base + G_OFF + (uint32_t)(i % GS) * G_STAGE, v);
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(gfull_bar(i % GS));
      ++stored;
      return true;
    };
    float v0[32], v1[32], v2[32];  // rotate by name, as in the window fill
    bool h0 = fetch(v0), h1 = h0 && fetch(v1), h2 = false;
    while (h0 && ok) {
      h2 = h1 && fetch(v2);
      ok = put(v0);
      if (!ok || !h1) break;
      h0 = h2 && fetch(v0);
      ok = put(v1);
      if (!ok || !h2) break;
      h1 = h0 && fetch(v1);
      ok = put(v2);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                 // lane quarter = horizontal tap b
    const int half = warp >= 8 ? 1 : 0;     // output channels 32 * half ..
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    float sum[MAX_KH * 32];
#pragma unroll
    for (int e = 0; e < MAX_KH * 32; ++e) sum[e] = 0.0f;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    const int chunks = (R + CHUNK_ROWS - 1) / CHUNK_ROWS;
    for (int ch = 0; ch < chunks; ++ch) {
      ok = ptx::mbar_wait_bounded(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
#pragma unroll
      for (int a = 0; a < MAX_KH; ++a) {
        if (a < kh) {
#pragma unroll
          for (int h16 = 0; h16 < 2; ++h16) {
            uint32_t v[16];
            ptx::tmem_ld_32x16(lane_base + acc * ACC_COLS + (uint32_t)a * BO + half * 32 + h16 * 16, v);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e)
              sum[a * 32 + h16 * 16 + e] = __fadd_rn(sum[a * 32 + h16 * 16 + e], __uint_as_float(v[e]));
          }
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(tempty_bar(acc));
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (ok) {
      const int cg = grp * 32 + lane;
      if (q < kw && cg < p.C) {
        const size_t per_part = (size_t)p.O * p.C * kh * kw;
        float* out = p.partial + (size_t)blockIdx.x * per_part;
#pragma unroll
        for (int a = 0; a < MAX_KH; ++a) {
          if (a < kh) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int og = ob * BO + half * 32 + e;
              if (og < p.O) out[(((size_t)og * p.C + cg) * kh + a) * kw + q] = sum[a * 32 + e];
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(p.status, VTLB_ST_GEMM_TIMEOUT);
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out[i] = sum over the parts of partial[part][i], in a fixed order.  A weight gradient has few
// elements and many parts (one per CTA of the kernel above), so eight threads share an element:
// thread (group, element) adds the parts = group (mod 8) in ascending order, the eight sums are then
// added in group order.  32 elements per CTA.
__global__ void __launch_bounds__(256) reduce_parts_kernel(const float* __restrict__ partial, int parts, size_t n,
                                                           float* __restrict__ out) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ float part_sum[8][33];
  const int e = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const size_t i = (size_t)blockIdx.x * 32 + e;
  float s = 0.0f;
  if (i < n)
    for (int k = grp; k < parts; k += 8) s = __fadd_rn(s, partial[(size_t)k * n + i]);
  part_sum[grp][e] = s;
  __syncthreads();
  if (grp == 0 && i < n) {
    float t = part_sum[0][e];
#pragma unroll
    for (int k = 1; k < 8; ++k) t = __fadd_rn(t, part_sum[k][e]);
    out[i] = t;
  }
}

// dW[O][C][kh][kw] of one convolution; `partial` must hold parts(...) * O*C*kh*kw floats.
inline int parts_for(vtlb_ctx* ctx, int B, int C, int O, int Ho) {
  const int G = (C + 31) / 32, OB = (O + BO - 1) / BO;
  int parts = ctx->sm_count / (G * OB);
  if (parts < 1) parts = 1;
  const int rows = B * Ho;
  if (parts > rows) parts = rows;
  const int rpp = (rows + parts - 1) / parts;
  return (rows + rpp - 1) / rpp;
}

inline int launch(vtlb_ctx* ctx, const float* x, const float* g, float* partial, float* dW, int B, int C, int H, int W,
                  int O, int Ho, int Wo, int kh, int kw, int ph, int pw) {
  const int G = (C + 31) / 32, OB = (O + BO - 1) / BO;
  const int rows = B * Ho;
  const int parts = parts_for(ctx, B, C, O, Ho);
  Params p{x, g, partial, B, C, H, W, O, Ho, Wo, kh, kw, ph, pw, rows, (rows + parts - 1) / parts, ctx->d_status};
  static std::atomic<uint64_t> configured{0};
  if (!(configured.load(std::memory_order_relaxed) >> (ctx->device & 63) & 1)) {
    VTLB_CUDA(ctx, cudaFuncSetAttribute(conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_TOTAL));
    configured.fetch_or(1ull << (ctx->device & 63), std::memory_order_relaxed);
  }
  const bool timed = ctx->prof_on && ctx->prof_ev && ctx->prof_n < vtlb_ctx::kProfSlots;
  if (timed) cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n], ctx->stream);
  VTLB_CUDA(ctx, vtlb_launch_early(conv_wgrad_kernel, dim3(parts, G, OB), dim3(NUM_THREADS), SMEM_TOTAL, ctx->stream, p));
  if (timed) {
    cudaEventRecord(ctx->prof_ev[2 * ctx->prof_n + 1], ctx->stream);
    ctx->prof_n++;
    ctx->prof_flops += 2.0 * B * Ho * Wo * (double)O * C * kh * kw;
  }
  VTLB_LAUNCHED(ctx);
  const size_t n = (size_t)O * C * kh * kw;
  VTLB_CUDA(ctx, vtlb_launch_early(reduce_parts_kernel, dim3((unsigned)((n + 31) / 32)), dim3(256), 0, ctx->stream,
                                   (const float*)partial, parts, n, dW));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

}  // namespace cwgrad
