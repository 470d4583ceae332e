// INT8 quantised linear path: per-row symmetric quantisation, int8 x int8 ->
// int32 GEMM on tcgen05 (kind::i8) and the fused dequant + bias + ReLU epilogue.
// The reference has no quantisation code; the arithmetic is the one stated in
// include/vtlb.h and every f32 operation below rounds on its own (__fmul_rn,
// __fadd_rn, __fdiv_rn) so that results are bit-identical to a plain C loop
// compiled without FMA contraction.
#include <stdlib.h>

#include "gemm_tc2.cuh"
#include "gemm_i8_skinny.cuh"

namespace {

// Row counts up to which the register-resident quantise kernel is launched early
// (programmatic stream serialisation, common.cuh).
constexpr int kEarlyQuantRows = 512;

// ---------------------------------------------------------------- quantise rows
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ int quant1(float a, float inv) {
  int q = __float2int_rn(__fmul_rn(a, inv));  // ties-to-even, like rintf
  return max(-127, min(127, q));
}

// One CTA per row.  Pass 1: row max-abs (float4 loads, warp shuffles).  Pass 2
// re-reads the row (it is still in L1/L2: a row is at most a few tens of KB)
// and writes 16 codes per thread as one 16-byte store.  Algorithmic HBM traffic:
// 4K bytes read + K bytes written + 4 bytes of scale per row.
template <bool HAVE_AMAX>
__global__ void __launch_bounds__(256) quant_rows_i8_kernel(const float* __restrict__ A, int M,
                                                            int K, int ldq,
                                                            int8_t* __restrict__ Q,
                                                            float* __restrict__ scale,
                                                            const float* __restrict__ amax_in) {
  __shared__ float s_part[8];
  __shared__ float s_amax;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early: the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int row = blockIdx.x;
  if (row >= M) return;
  const float* a = A + (size_t)row * K;
  const bool vec = ((K & 3) == 0) && ((((uintptr_t)A) & 15u) == 0);
  float amax;
  if (HAVE_AMAX) {
    amax = amax_in[row];
  } else {
    float m = 0.0f;
    if (vec) {
      const float4* a4 = reinterpret_cast<const float4*>(a);
      for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
        float4 v = a4[i];
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      }
    } else {
      for (int i = threadIdx.x; i < K; i += blockDim.x) m = fmaxf(m, fabsf(a[i]));
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.0f;
      t = warp_max(t);
      if (threadIdx.x == 0) s_amax = t;
    }
    __syncthreads();
    amax = s_amax;
  }
  const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
  if (threadIdx.x == 0) scale[row] = __fdiv_rn(amax, 127.0f);
  int8_t* q = Q + (size_t)row * ldq;
  if (vec && (K & 15) == 0) {
    const float4* a4 = reinterpret_cast<const float4*>(a);
    int4* q16 = reinterpret_cast<int4*>(q);
    for (int i = threadIdx.x; i < K / 16; i += blockDim.x) {
      int w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 v = a4[i * 4 + j];
        int b0 = quant1(v.x, inv), b1 = quant1(v.y, inv), b2 = quant1(v.z, inv),
            b3 = quant1(v.w, inv);
        w[j] = (b0 & 0xff) | ((b1 & 0xff) << 8) | ((b2 & 0xff) << 16) | ((b3 & 0xff) << 24);
      }
      q16[i] = make_int4(w[0], w[1], w[2], w[3]);
    }
  } else {
    for (int i = threadIdx.x; i < K; i += blockDim.x) q[i] = (int8_t)quant1(a[i], inv);
  }
}

// Rows of at most 1024 * VPT elements with K % 4 == 0: every thread keeps its part of the row
// in registers (VPT coalesced float4 loads issued back to back), so the row is read exactly
// once from memory and the quantising pass costs no memory reads at all.
template <int VPT, bool HAVE_AMAX>
__global__ void __launch_bounds__(256) quant_rows_i8_reg_kernel(const float* __restrict__ A, int M, int K,
                                                                int ldq, int8_t* __restrict__ Q,
                                                                float* __restrict__ scale,
                                                                const float* __restrict__ amax_in) {
  __shared__ float s_part[8];
  __shared__ float s_amax;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early: the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int row = blockIdx.x;
  const float4* a4 = reinterpret_cast<const float4*>(A + (size_t)row * K);
  const int n4 = K >> 2;
  float4 v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + 256 * i;
    v[i] = idx < n4 ? __ldcs(a4 + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float amax;
  if (HAVE_AMAX) {
    amax = amax_in[row];
  } else {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < 8 ? s_part[threadIdx.x] : 0.0f;
      t = warp_max(t);
      if (threadIdx.x == 0) s_amax = t;
    }
    __syncthreads();
    amax = s_amax;
  }
  const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
  if (threadIdx.x == 0) scale[row] = __fdiv_rn(amax, 127.0f);
  int* q4 = reinterpret_cast<int*>(Q + (size_t)row * ldq);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + 256 * i;
    if (idx < n4) {
      const int b0 = quant1(v[i].x, inv), b1 = quant1(v[i].y, inv), b2 = quant1(v[i].z, inv),
                b3 = quant1(v[i].w, inv);
      q4[idx] = (b0 & 0xff) | ((b1 & 0xff) << 8) | ((b2 & 0xff) << 16) | ((b3 & 0xff) << 24);
    }
  }
}

__global__ void __launch_bounds__(256) row_absmax_kernel(const float* __restrict__ A, int M, int K,
                                                         float* __restrict__ amax) {
  __shared__ float s_part[8];
  const int row = blockIdx.x;
  if (row >= M) return;
  const float* a = A + (size_t)row * K;
  float m = 0.0f;
  for (int i = threadIdx.x; i < K; i += blockDim.x) m = fmaxf(m, fabsf(a[i]));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.0f;
    t = warp_max(t);
    if (threadIdx.x == 0) amax[row] = t;
  }
}

// ---------------------------------------------------------------- epilogues
struct EpiStoreI32 {
  static constexpr bool kTmaCapable = true;
  int32_t* C;
  int ldc;
  int tma;  // store through the output tensor map (tm.out[0]) instead of per-thread stores
  __device__ __forceinline__ bool transform(int, int, uint32_t (&)[32], int, int) const { return false; }
  __device__ __forceinline__ void activate(uint32_t (&)[32]) const {}
  struct Pre {};  // nothing to fetch ahead of the accumulator
  __device__ __forceinline__ Pre prefetch(int, int, int, int) const { return Pre{}; }
  __device__ __forceinline__ void transform_pre(const Pre&, int, uint32_t (&)[32]) const {}
  __device__ __forceinline__ float chunk_amax(int, const uint32_t (&)[32], int) const { return 0.0f; }
  __device__ __forceinline__ void commit_amax(int, int, float) const {}
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&v)[32], int M,
                                             int N, int /*split*/) const {
    if (row >= M) return;
    int32_t* c = C + (size_t)row * ldc + col0;
    if (col0 + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<int4*>(c + j) = make_int4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) c[j] = (int32_t)v[j];
    }
  }
};

__device__ __forceinline__ float dequant1(uint32_t acc, float sa, float sw, float bias,
                                          bool has_bias, int relu) {
  float t = __fmul_rn(sa, sw);
  float u = __fmul_rn(__int2float_rn((int)acc), t);
  float y = has_bias ? __fadd_rn(u, bias) : u;
  if (relu && y < 0.0f) y = 0.0f;
  return y;
}

struct EpiDequant {
  static constexpr bool kTmaCapable = true;
  float* Y;
  const float* sa;
  const float* sw;
  const float* bias;  // may be null
  int ldy;
  int relu;
  int tma;  // store through the output tensor map (needs N % 4 == 0)
  // when set: amax[row] = max(amax[row], max_col |y[row, col]|), the row maxima the next layer's
  // dynamic quantisation needs, so that nobody has to read Y again for them.  Non-negative floats
  // order like their bit patterns, hence an integer atomicMax; the caller zeroes the array.
  float* amax = nullptr;
  // largest |v| of a chunk (columns at or past N do not count); commit_amax folds it into amax[row]
  __device__ __forceinline__ float chunk_amax(int col0, const uint32_t (&v)[32], int N) const {
    float m = 0.0f;
    if (amax == nullptr) return m;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < N) m = fmaxf(m, fabsf(__uint_as_float(v[j])));
    return m;
  }
  __device__ __forceinline__ void commit_amax(int row, int M, float m) const {
    if (amax != nullptr && row < M) atomicMax(reinterpret_cast<int*>(amax + row), __float_as_int(m));
  }
  __device__ __forceinline__ void note_amax(int row, int col0, const uint32_t (&v)[32], int M, int N) const {
    commit_amax(row, M, chunk_amax(col0, v, N));
  }
  // dequantises the chunk in registers; rows and columns past the edge yield values the
  // clipped TMA store never writes
  __device__ __forceinline__ bool transform(int row, int col0, uint32_t (&v)[32], int M, int N) const {
    const float s = row < M ? sa[row] : 0.0f;
    const bool hb = bias != nullptr;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float4 w4 = make_float4(0.f, 0.f, 0.f, 0.f), b4 = w4;
      if (col0 + j < N) {
        w4 = __ldg(reinterpret_cast<const float4*>(sw + col0 + j));
        if (hb) b4 = __ldg(reinterpret_cast<const float4*>(bias + col0 + j));
      }
      v[j] = __float_as_uint(dequant1(v[j], s, w4.x, b4.x, hb, relu));
      v[j + 1] = __float_as_uint(dequant1(v[j + 1], s, w4.y, b4.y, hb, relu));
      v[j + 2] = __float_as_uint(dequant1(v[j + 2], s, w4.z, b4.z, hb, relu));
      v[j + 3] = __float_as_uint(dequant1(v[j + 3], s, w4.w, b4.w, hb, relu));
    }
    note_amax(row, col0, v, M, N);
    return false;
  }
  __device__ __forceinline__ void activate(uint32_t (&)[32]) const {}
  // The same dequantisation with its operands fetched ahead (CTA-pair kernel): this lane's row
  // scale, and for each of the warp's four 32-column chunks (64 columns apart) the weight scale
  // and bias of ONE column, `col` being this lane's column in the first chunk.
  struct Pre {
    float s;
    float w[4], b[4];
  };
  __device__ __forceinline__ Pre prefetch(int row, int col, int M, int N) const {
    Pre p;
    p.s = row < M ? __ldg(sa + row) : 0.0f;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c = col + cc * 64;
      p.w[cc] = c < N ? __ldg(sw + c) : 0.0f;
      p.b[cc] = (bias != nullptr && c < N) ? __ldg(bias + c) : 0.0f;
    }
    return p;
  }
  __device__ __forceinline__ void transform_pre(const Pre& p, int cc, uint32_t (&v)[32]) const {
    const bool hb = bias != nullptr;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float w = __shfl_sync(0xffffffffu, p.w[cc], j);
      const float b = __shfl_sync(0xffffffffu, p.b[cc], j);
      v[j] = __float_as_uint(dequant1(v[j], p.s, w, b, hb, relu));
    }
  }
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&v)[32], int M,
                                             int N, int /*split*/) const {
    if (row >= M) return;
    const float s = sa[row];
    float* y = Y + (size_t)row * ldy + col0;
    const bool hb = bias != nullptr;
    uint32_t o[32];
#pragma unroll
    for (int j = 0; j < 32; ++j)
      o[j] = col0 + j < N ? __float_as_uint(dequant1(v[j], s, __ldg(sw + col0 + j), hb ? __ldg(bias + col0 + j) : 0.0f,
                                                      hb, relu))
                          : 0u;
    note_amax(row, col0, o, M, N);
    if (col0 + 32 <= N && (ldy & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(y + j) = make_float4(__uint_as_float(o[j]), __uint_as_float(o[j + 1]),
                                                        __uint_as_float(o[j + 2]), __uint_as_float(o[j + 3]));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) y[j] = __uint_as_float(o[j]);
    }
  }
};

// ---------------------------------------------------------------- very small M (GEMV-like)
// With a single row of activations (up to VTLB_I8_GEMV_MAX_M rows) the problem is streaming W
// once from HBM (N*K bytes).  Each warp owns one output channel at a time and walks its row of W in pieces of
// U * 512 bytes, all U 16-byte loads of a lane issued before the first is used (a whole
// 4096-byte row in flight per warp at U = 8), accumulating with dp4a against up to MT
// rows of A (exact int32).
template <int MT, int U, bool FUSED>
__global__ void __launch_bounds__(128) gemv_i8_kernel(const int8_t* __restrict__ Aq,
                                                      const int8_t* __restrict__ Wq, int M, int N,
                                                      int K, int ldk, int32_t* __restrict__ acc_out,
                                                      float* __restrict__ Y,
                                                      const float* __restrict__ sa,
                                                      const float* __restrict__ sw,
                                                      const float* __restrict__ bias, int relu) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early: the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int gwarp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int n = gwarp; n < N; n += nwarps) {
    int acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0;
    const int8_t* wrow = Wq + (size_t)n * ldk;
    for (int k0 = lane * 16; k0 < ldk; k0 += 512 * U) {
      int4 w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + 512 * u;
        w[u] = make_int4(0, 0, 0, 0);
        if (k < ldk) w[u] = __ldcs(reinterpret_cast<const int4*>(wrow + k));  // read once: streaming
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + 512 * u;
        if (k >= ldk) break;
        // bytes at k >= K inside the padded leading dimension are never used: mask them
        if (k + 16 > K) {
          const int valid = K - k;  // 1..15 valid bytes (ldk is K rounded up to 16)
          int* wp = reinterpret_cast<int*>(&w[u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int vb = valid - 4 * j;
            wp[j] &= vb >= 4 ? -1 : (vb <= 0 ? 0 : (int)((1u << (8 * vb)) - 1u));
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          if (m < M) {
            const int4 a = __ldg(reinterpret_cast<const int4*>(Aq + (size_t)m * ldk + k));
            int t = acc[m];
            t = __dp4a(a.x, w[u].x, t);
            t = __dp4a(a.y, w[u].y, t);
            t = __dp4a(a.z, w[u].z, t);
            t = __dp4a(a.w, w[u].w, t);
            acc[m] = t;
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      int t = acc[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      acc[m] = t;
    }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m >= M) continue;
        if (FUSED)
          Y[(size_t)m * N + n] = dequant1((uint32_t)acc[m], sa[m], sw[n], bias ? bias[n] : 0.0f,
                                          bias != nullptr, relu);
        else
          acc_out[(size_t)m * N + n] = acc[m];
      }
    }
  }
}

// Above this many rows the tensor-core kernels are faster than dp4a
// (VTLB_I8_GEMV_MAX_M overrides, 0..16, for measurements).
int gemv_max_m() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("VTLB_I8_GEMV_MAX_M");
    v = e ? atoi(e) : 1;
    if (v < 0) v = 0;
    if (v > 16) v = 16;
  }
  return v;
}

// Few rows (up to 128) on one wave of 128-channel tiles: the swapped-operand kernel with K
// cut across a cluster (gemm_i8_skinny.cuh).  VTLB_I8_SKINNY=0 switches it off.
bool use_skinny(vtlb_ctx* ctx, int M, int N) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("VTLB_I8_SKINNY");
    on = e ? atoi(e) != 0 : 1;
  }
  return on && skinny::usable(ctx, M, N);
}

template <bool FUSED>
int launch_gemv(vtlb_ctx* ctx, const int8_t* Aq, const int8_t* Wq, int M, int N, int K,
                int32_t* acc, float* Y, const float* sa, const float* sw, const float* bias,
                int relu) {
  const int ldk = vtlb_i8_ld(K);
  int blocks = (N + 3) / 4;  // four warps per block, one channel per warp at a time
  if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
  if (blocks < 1) blocks = 1;
#define VTLB_GEMV(MT)                                                                        \
  VTLB_CUDA(ctx, vtlb_launch_early(gemv_i8_kernel<MT, 8, FUSED>, dim3(blocks), dim3(128), 0, ctx->stream, \
                                   Aq, Wq, M, N, K, ldk, acc, Y, sa, sw, bias, relu))
  if (M <= 1) VTLB_GEMV(1);
  else if (M <= 2) VTLB_GEMV(2);
  else if (M <= 4) VTLB_GEMV(4);
  else if (M <= 8) VTLB_GEMV(8);
  else VTLB_GEMV(16);
#undef VTLB_GEMV
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

int make_i8_tmaps(vtlb_ctx* ctx, gemm::TmapSet* tm, const void* Aq, const void* Wq, int M, int N,
                  int K, int bn) {
  const int ldk = vtlb_i8_ld(K);
  int rc = gemm::encode_tmap_2d(ctx, &tm->a[0], false, Aq, (uint64_t)K, (uint64_t)M, (uint64_t)ldk,
                                128, gemm::BM);
  if (rc) return rc;
  rc = gemm::encode_tmap_2d(ctx, &tm->b[0], false, Wq, (uint64_t)K, (uint64_t)N, (uint64_t)ldk, 128,
                            bn);
  if (rc) return rc;
  tm->a[1] = tm->a[0];
  tm->b[1] = tm->b[0];
  return VTLB_OK;
}

// Tile width: 256 columns when that still gives every SM a tile, else narrower
// so that small problems spread over more CTAs.
int pick_bn(vtlb_ctx* ctx, int M, int N) {
  const int tm = (M + gemm::BM - 1) / gemm::BM;
  if (tm * ((N + 255) / 256) >= ctx->sm_count) return 256;
  if (tm * ((N + 127) / 128) >= ctx->sm_count / 2) return 128;
  return 64;
}

// CTA pairs (256 x 256 tiles) pay off once there are enough such tiles to occupy the pairs;
// VTLB_I8_PAIR=0/1 forces the choice (for measurements).
bool use_pair_kernel(vtlb_ctx* ctx, int M, int N) {
  static int forced = -2;
  if (forced == -2) {
    const char* e = getenv("VTLB_I8_PAIR");
    forced = e ? atoi(e) : -1;
  }
  if (forced == 0) return false;
  if (forced == 1) return true;
  return gemm2::pair_worthwhile(ctx, M, N);
}

// `chunks` > 1: Aq is stored as that many column shards one after another, each a dense
// [M, K/chunks] matrix (the layout an all-gather of per-rank column slabs leaves behind); the
// A operand is then read through a 3-D tensor map (k within shard, row, shard).
template <class Epi>
int run_i8(vtlb_ctx* ctx, const void* Aq, const void* Wq, int M, int N, int K, Epi epi, void* out,
           int chunks = 1) {
  gemm::TmapSet tm;
  // 4-byte outputs with a 16-byte-multiple row pitch go out through TMA stores
  epi.tma = (N % 4 == 0) && vtlb_aligned16(out);
  if (epi.tma) {
    int rc0 = gemm::encode_tmap_2d(ctx, &tm.out[0], true, out, (uint64_t)N, (uint64_t)M, (uint64_t)N * 4, 32, 32);
    if (rc0) return rc0;
    tm.out[1] = tm.out[0];
  }
  const int chunk_k = chunks > 1 ? K / chunks : 0;
  const bool pair = use_pair_kernel(ctx, M, N);
  const int bn = pair ? 128 : pick_bn(ctx, M, N);  // a CTA of a pair loads 128 rows of B
  int rc = make_i8_tmaps(ctx, &tm, Aq, Wq, M, N, K, bn);
  if (rc) return rc;
  if (chunk_k) {
    if ((rc = gemm::encode_tmap_3d_u8(ctx, &tm.a[0], Aq, (uint64_t)chunk_k, (uint64_t)M, (uint64_t)chunks,
                                      (uint64_t)chunk_k, (uint64_t)M * chunk_k, 128, gemm::BM)))
      return rc;
    tm.a[1] = tm.a[0];
  }
  if (pair) {
    static int k_split = -1;
    if (k_split < 0) {
      const char* e = getenv("VTLB_I8_K_SPLIT");
      k_split = e ? atoi(e) : 1;
    }
    return gemm2::launch_pair<gemm::KIND_I8, Epi>(ctx, tm, epi, M, N, K, chunk_k, k_split != 0);
  }
  if (bn == 256) return gemm::launch<gemm::KIND_I8, 256, 4, Epi>(ctx, tm, epi, M, N, K, 1, chunk_k);
  if (bn == 128) return gemm::launch<gemm::KIND_I8, 128, 6, Epi>(ctx, tm, epi, M, N, K, 1, chunk_k);
  return gemm::launch<gemm::KIND_I8, 64, 8, Epi>(ctx, tm, epi, M, N, K, 1, chunk_k);
}

int check_i8_args(vtlb_ctx* ctx, const char* fn, int M, int N, int K) {
  if (M < 0 || N < 0 || K <= 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: bad shape M=%d N=%d K=%d (K must be > 0)", fn, M, N, K);
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_i8_ld(int K) { return (K + 15) / 16 * 16; }

VTLB_API int vtlb_quant_rows_i8(vtlb_ctx* ctx, const void* d_A, int M, int K, void* d_Q,
                                void* d_scale, const void* d_amax_in_or_null) {
  VTLB_ENTER(ctx);
  if (M < 0 || K <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_quant_rows_i8: bad shape %dx%d", M, K);
  if (M == 0) return VTLB_OK;
  if (!d_A || !d_Q || !d_scale) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_quant_rows_i8: null pointer");
  if (!vtlb_aligned16(d_Q)) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_quant_rows_i8: Q not 16-byte aligned");
  vtlb_prof_scope prof(ctx, VTLB_PHASE_ELEMENTWISE);
  const int ldq = vtlb_i8_ld(K);
  if ((K & 3) == 0 && K <= 8192 && vtlb_aligned16(d_A)) {  // register-resident rows
    const float* A = (const float*)d_A;
    int8_t* Q = (int8_t*)d_Q;
    float* sc = (float*)d_scale;
    const float* am = (const float*)d_amax_in_or_null;
#define VTLB_QREG(VPT)                                                                            \
  do {                                                                                            \
    if (M > kEarlyQuantRows) { /* long launches gain nothing from an early start (measured) */   \
      if (am) quant_rows_i8_reg_kernel<VPT, true><<<M, 256, 0, ctx->stream>>>(A, M, K, ldq, Q, sc, am);  \
      else quant_rows_i8_reg_kernel<VPT, false><<<M, 256, 0, ctx->stream>>>(A, M, K, ldq, Q, sc, am);    \
    } else if (am)                                                                                \
      VTLB_CUDA(ctx, vtlb_launch_early(quant_rows_i8_reg_kernel<VPT, true>, dim3(M), dim3(256), 0,    \
                                       ctx->stream, A, M, K, ldq, Q, sc, am));                      \
    else                                                                                          \
      VTLB_CUDA(ctx, vtlb_launch_early(quant_rows_i8_reg_kernel<VPT, false>, dim3(M), dim3(256), 0,   \
                                       ctx->stream, A, M, K, ldq, Q, sc, am));                      \
  } while (0)
    if (K <= 1024) VTLB_QREG(1);
    else if (K <= 2048) VTLB_QREG(2);
    else if (K <= 4096) VTLB_QREG(4);
    else VTLB_QREG(8);
#undef VTLB_QREG
    VTLB_LAUNCHED(ctx);
    return VTLB_OK;
  }
  if (d_amax_in_or_null)
    quant_rows_i8_kernel<true><<<M, 256, 0, ctx->stream>>>((const float*)d_A, M, K, ldq,
                                                           (int8_t*)d_Q, (float*)d_scale,
                                                           (const float*)d_amax_in_or_null);
  else
    quant_rows_i8_kernel<false><<<M, 256, 0, ctx->stream>>>((const float*)d_A, M, K, ldq,
                                                            (int8_t*)d_Q, (float*)d_scale, nullptr);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_row_absmax_f32(vtlb_ctx* ctx, const void* d_A, int M, int K, void* d_amax) {
  VTLB_ENTER(ctx);
  if (M < 0 || K <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_row_absmax_f32: bad shape %dx%d", M, K);
  if (M == 0) return VTLB_OK;
  if (!d_A || !d_amax) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_row_absmax_f32: null pointer");
  row_absmax_kernel<<<M, 256, 0, ctx->stream>>>((const float*)d_A, M, K, (float*)d_amax);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_gemm_i8_i32(vtlb_ctx* ctx, const void* d_Aq, const void* d_Wq, int M, int N,
                              int K, void* d_acc) {
  VTLB_ENTER(ctx);
  int rc = check_i8_args(ctx, "vtlb_gemm_i8_i32", M, N, K);
  if (rc) return rc;
  if (M == 0 || N == 0) return VTLB_OK;
  if (!d_Aq || !d_Wq || !d_acc) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_gemm_i8_i32: null pointer");
  if (!vtlb_aligned16(d_Aq) || !vtlb_aligned16(d_Wq) || !vtlb_aligned16(d_acc))
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_gemm_i8_i32: pointers must be 16-byte aligned");
  if (M <= gemv_max_m())
    return launch_gemv<false>(ctx, (const int8_t*)d_Aq, (const int8_t*)d_Wq, M, N, K,
                              (int32_t*)d_acc, nullptr, nullptr, nullptr, nullptr, 0);
  if (use_skinny(ctx, M, N)) {
    skinny::Params p = {};
    p.acc = (int32_t*)d_acc;
    return skinny::launch<false>(ctx, d_Aq, d_Wq, M, N, K, p);
  }
  EpiStoreI32 epi{(int32_t*)d_acc, N};
  return run_i8(ctx, d_Aq, d_Wq, M, N, K, epi, d_acc);
}

// The general form behind the three entry points below.
static int linear_i8_fwd_impl(vtlb_ctx* ctx, const char* fn, const void* d_Aq, int shards, const void* d_sa,
                              const void* d_Wq, const void* d_sw, const void* d_bias_or_null, void* d_Y, int M, int N,
                              int K, int relu, void* d_row_amax_or_null) {
  int rc = check_i8_args(ctx, fn, M, N, K);
  if (rc) return rc;
  if (shards < 1 || K % shards || (shards > 1 && (K / shards) % 128))
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: K=%d must split into %d shards of a multiple of 128 columns", fn, K, shards);
  if (M == 0 || N == 0) return VTLB_OK;
  if (!d_Aq || !d_Wq || !d_sa || !d_sw || !d_Y) return vtlb_fail(ctx, VTLB_EINVAL, "%s: null pointer", fn);
  if (!vtlb_aligned16(d_Aq) || !vtlb_aligned16(d_Wq) || !vtlb_aligned16(d_Y) || !vtlb_aligned16(d_sw) ||
      (d_bias_or_null && !vtlb_aligned16(d_bias_or_null)))
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: pointers must be 16-byte aligned", fn);
  if (shards == 1 && (M <= gemv_max_m() || use_skinny(ctx, M, N))) {
    if (M <= gemv_max_m()) {
      rc = launch_gemv<true>(ctx, (const int8_t*)d_Aq, (const int8_t*)d_Wq, M, N, K, nullptr, (float*)d_Y,
                             (const float*)d_sa, (const float*)d_sw, (const float*)d_bias_or_null, relu);
    } else {
      skinny::Params p = {};
      p.Y = (float*)d_Y;
      p.sa = (const float*)d_sa;
      p.sw = (const float*)d_sw;
      p.bias = (const float*)d_bias_or_null;
      p.relu = relu;
      rc = skinny::launch<true>(ctx, d_Aq, d_Wq, M, N, K, p);
    }
    if (rc || !d_row_amax_or_null) return rc;
    row_absmax_kernel<<<M, 256, 0, ctx->stream>>>((const float*)d_Y, M, N, (float*)d_row_amax_or_null);
    VTLB_LAUNCHED(ctx);
    return VTLB_OK;
  }
  EpiDequant epi{(float*)d_Y, (const float*)d_sa, (const float*)d_sw, (const float*)d_bias_or_null, N, relu};
  if (d_row_amax_or_null) {
    VTLB_CUDA(ctx, cudaMemsetAsync(d_row_amax_or_null, 0, (size_t)M * sizeof(float), ctx->stream));
    epi.amax = (float*)d_row_amax_or_null;
  }
  return run_i8(ctx, d_Aq, d_Wq, M, N, K, epi, d_Y, shards);
}

VTLB_API int vtlb_linear_i8_fwd(vtlb_ctx* ctx, const void* d_Aq, const void* d_sa,
                                const void* d_Wq, const void* d_sw, const void* d_bias_or_null,
                                void* d_Y, int M, int N, int K, int relu) {
  VTLB_ENTER(ctx);
  return linear_i8_fwd_impl(ctx, "vtlb_linear_i8_fwd", d_Aq, 1, d_sa, d_Wq, d_sw, d_bias_or_null, d_Y, M, N, K, relu,
                            nullptr);
}

VTLB_API int vtlb_linear_i8_fwd_sharded_a(vtlb_ctx* ctx, const void* d_Aq_shards, int shards,
                                          const void* d_sa, const void* d_Wq, const void* d_sw,
                                          const void* d_bias_or_null, void* d_Y, int M, int N, int K,
                                          int relu) {
  VTLB_ENTER(ctx);
  return linear_i8_fwd_impl(ctx, "vtlb_linear_i8_fwd_sharded_a", d_Aq_shards, shards, d_sa, d_Wq, d_sw, d_bias_or_null,
                            d_Y, M, N, K, relu, nullptr);
}

VTLB_API int vtlb_linear_i8_fwd_amax(vtlb_ctx* ctx, const void* d_Aq_shards, int shards, const void* d_sa,
                                     const void* d_Wq, const void* d_sw, const void* d_bias_or_null, void* d_Y,
                                     int M, int N, int K, int relu, void* d_row_amax) {
  VTLB_ENTER(ctx);
  if (!d_row_amax) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_linear_i8_fwd_amax: null row-maximum output");
  return linear_i8_fwd_impl(ctx, "vtlb_linear_i8_fwd_amax", d_Aq_shards, shards, d_sa, d_Wq, d_sw, d_bias_or_null, d_Y,
                            M, N, K, relu, d_row_amax);
}


// ---------------------------------------------------------------- INT8 issue-rate yardstick
// What the tensor cores deliver when nothing has to be loaded: every CTA pair issues
// tcgen05.mma.cta_group::2.kind::i8 (M = 256, N = 256, K = 32) back to back on operands that sit in
// shared memory for the whole launch, into one accumulator.  The result is meaningless; the rate is the
// ceiling of any INT8 GEMM on this device at the clocks it runs at, measured instead of derived from a
// bf16 figure.  No global memory is read or written apart from the status word.
namespace {

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
i8_issue_yardstick_kernel(int mma_groups, uint32_t* status) {
  constexpr uint32_t TILE = 128 * 128;  // 128 rows of 128 bytes: this CTA's half of A, and of B
  constexpr uint32_t IDESC = ptx::umma_idesc(ptx::kCfmtS32, ptx::kFmtS8, 256, 256);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bar = base + 2 * TILE;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_raw + (bar - raw) + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = gemm2::cluster_ctarank();
  for (uint32_t i = threadIdx.x; i < 2 * TILE / 16; i += blockDim.x)  // defined operands (zeros)
    ptx::st_shared_v4(base + i * 16, 0u, 0u, 0u, 0u);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::fence_proxy_async();
  if (warp == 1) {
    gemm2::tmem_alloc2(ptx::smem_u32(tmem_slot), 256);
    gemm2::tmem_relinquish2();
  }
  ptx::tc_fence_before();
  __syncthreads();
  gemm2::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == 0 && lane == 0 && rank == 0) {
    const uint64_t da = ptx::umma_desc_k_sw128(base), db = ptx::umma_desc_k_sw128(base + TILE);
    for (int g = 0; g < mma_groups; ++g) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) gemm2::umma_i8_pair(tmem_base, da + 2u * kk, db + 2u * kk, IDESC, (g | kk) ? 1u : 0u);
    }
    gemm2::umma_commit_pair(bar);  // arrives in both CTAs once every MMA has completed
  }
  if (warp == 0) {
    // both CTAs stay until the MMAs have stopped reading their shared memory
    bool ok = ptx::mbar_wait_bounded(bar, 0, abort_flag, gemm::WAIT_LIMIT_NS, 200);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && lane == 0) atomicOr(status, VTLB_ST_GEMM_TIMEOUT);
  }
  ptx::tc_fence_before();
  __syncthreads();
  gemm2::cluster_sync_all();
  ptx::tc_fence_after();
  if (warp == 1) {
    __syncwarp();
    gemm2::tmem_dealloc2(tmem_base, 256);
  }
}

}  // namespace

VTLB_API int vtlb_int8_issue_yardstick(vtlb_ctx* ctx, int mma_groups, double* tops_out) {
  VTLB_ENTER(ctx);
  if (!tops_out || mma_groups < 1 || mma_groups > (1 << 20))
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_int8_issue_yardstick: bad arguments");
  constexpr int SMEM = 2 * 128 * 128 + 64 + 1024;
  const int pairs = ctx->sm_count / 2;
  cudaEvent_t e0, e1;
  VTLB_CUDA(ctx, cudaEventCreate(&e0));
  VTLB_CUDA(ctx, cudaEventCreate(&e1));
  i8_issue_yardstick_kernel<<<2 * pairs, 128, SMEM, ctx->stream>>>(mma_groups, ctx->d_status);  // warm-up
  VTLB_CUDA(ctx, cudaEventRecord(e0, ctx->stream));
  i8_issue_yardstick_kernel<<<2 * pairs, 128, SMEM, ctx->stream>>>(mma_groups, ctx->d_status);
  VTLB_CUDA(ctx, cudaEventRecord(e1, ctx->stream));
  ctx->launches += 2;
  cudaError_t e = cudaGetLastError();
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventSynchronize(e1);
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (e != cudaSuccess) return vtlb_fail(ctx, VTLB_ECUDA, "vtlb_int8_issue_yardstick: %s", cudaGetErrorString(e));
  *tops_out = 2.0 * 256 * 256 * 32 * 4.0 * mma_groups * pairs / (ms * 1e-3) / 1e12;
  return VTLB_OK;
}
