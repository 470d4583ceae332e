// Pieces shared by the f32 GEMM users (f32.cu, conv.cu): the TF32 hi/lo split, the
// operand planes in the context scratch, and the launcher of the 3xTF32 tcgen05 GEMM.
#pragma once
#include <stdlib.h>

#include "gemm_tc2.cuh"

namespace f32 {

__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
// x = hi + lo + O(2^-22 |x|), both representable in TF32 (10-bit mantissa)
__device__ __forceinline__ void split1(float x, float& hi, float& lo) {
  hi = tf32_rna(x);
  lo = tf32_rna(x - hi);
}

inline int grid_for(vtlb_ctx* ctx, size_t work_items, int per_block) {
  size_t b = (work_items + per_block - 1) / per_block;
  size_t cap = (size_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

// Two K-major operands, each as a pair of TF32 planes [rows, ld] in the context scratch.
struct Planes {
  float *a_hi, *a_lo, *b_hi, *b_lo;
  int ld;       // row stride in elements: K rounded up to 4 (TMA wants 16-byte strides)
  void* extra;  // `extra_bytes` of additional scratch behind the planes
};
inline int alloc_planes(vtlb_ctx* ctx, int rows_a, int rows_b, int K, size_t extra_bytes, Planes* p) {
  p->ld = (int)vtlb_round_up((size_t)K, 4);
  const size_t a = vtlb_round_up((size_t)rows_a * p->ld, 64), b = vtlb_round_up((size_t)rows_b * p->ld, 64);
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, (2 * a + 2 * b) * sizeof(float) + vtlb_round_up(extra_bytes, 256) + 256, &scr);
  if (rc) return rc;
  p->a_hi = (float*)scr;
  p->a_lo = p->a_hi + a;
  p->b_hi = p->a_lo + a;
  p->b_lo = p->b_hi + b;
  p->extra = p->b_lo + b;
  return VTLB_OK;
}

inline int bn_override() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("VTLB_F32_BN");
    v = e ? atoi(e) : 0;
  }
  return v;
}

// How many K ranges a launch with `want` splits really gets (empty ranges are dropped).
inline int effective_splits(int K, int want) {
  const int total_kb = (K + 31) / 32;
  if (want < 1) want = 1;
  if (want > total_kb) want = total_kb;
  const int per = (total_kb + want - 1) / want;
  return (total_kb + per - 1) / per;
}

// D[M,N] = A[M,K] . B[N,K]^T on the planes, epilogue functor `epi`.
// `fused` (optional) receives bit 0 = the epilogue writes the requested operand planes of the result,
// bit 1 = it applies the ReLU-backward mask; what it does not do, the caller does in separate passes.
template <class Epi>
int launch_tf32x3(vtlb_ctx* ctx, const Planes& p, int M, int N, int K, Epi epi, int splits = 1,
                  int* fused = nullptr) {
  if (fused) *fused = 0;
  gemm::TmapSet tm;
  if constexpr (Epi::kTmaCapable) {
    // outputs with a 16-byte-multiple row pitch go out through TMA stores
    epi.tma = (epi.ldy % 4 == 0) && vtlb_aligned16(epi.Y) && (!epi.pre || vtlb_aligned16(epi.pre)) &&
              (!epi.bias || N % 4 == 0);
    if (epi.tma) {
      int rc0 = gemm::encode_tmap_2d(ctx, &tm.out[0], true, epi.Y, N, M, (uint64_t)epi.ldy * 4, 32, 32);
      if (rc0) return rc0;
      tm.out[1] = tm.out[0];
      if (epi.pre &&
          (rc0 = gemm::encode_tmap_2d(ctx, &tm.out[1], true, epi.pre, N, M, (uint64_t)epi.ldy * 4, 32, 32)))
        return rc0;
    }
    if constexpr (gemm::EpiHasPlanes<Epi>::value) {
      // planes of the result leave through TMA stores too; without that path the caller splits
      // the stored result in a pass of its own
      if (!epi.tma || N % 4 != 0 || (epi.mask && !vtlb_aligned16(epi.mask))) {
        epi.planes = 0;
        epi.mask_fused = 0;
      } else {
        epi.mask_fused = epi.mask != nullptr;
      }
      if (epi.planes & 1) {
        int rc0 = gemm::encode_tmap_2d(ctx, &tm.out[2], true, epi.rows_hi, N, M, (uint64_t)epi.ld_rows * 4, 32, 32);
        if (!rc0) rc0 = gemm::encode_tmap_2d(ctx, &tm.out[3], true, epi.rows_lo, N, M, (uint64_t)epi.ld_rows * 4, 32, 32);
        if (rc0) return rc0;
      }
      if (fused) *fused = (epi.planes ? 1 : 0) | (epi.mask_fused ? 2 : 0);
    }
  }
  int bn = bn_override();
  if (bn != 64 && bn != 128) {
    const int tiles_m = (M + gemm::BM - 1) / gemm::BM;
    bn = (tiles_m * ((N + 127) / 128) * splits >= ctx->sm_count / 2) ? 128 : 64;
    if (N <= 64) bn = 64;
  }
  const uint64_t stride = (uint64_t)p.ld * 4;
  int rc;
  // large problems: CTA pairs, 256 x 256 tiles (VTLB_F32_PAIR=0 keeps them on single CTAs)
  static int pair_env = -2;
  if (pair_env == -2) {
    const char* e = getenv("VTLB_F32_PAIR");
    pair_env = e ? atoi(e) : -1;
  }
  if (splits == 1 && pair_env != 0 && gemm2::pair_worthwhile(ctx, M, N)) {
    if ((rc = gemm::encode_tmap_2d(ctx, &tm.a[0], true, p.a_hi, K, M, stride, 32, gemm::BM))) return rc;
    if ((rc = gemm::encode_tmap_2d(ctx, &tm.a[1], true, p.a_lo, K, M, stride, 32, gemm::BM))) return rc;
    if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[0], true, p.b_hi, K, N, stride, 32, 128))) return rc;
    if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[1], true, p.b_lo, K, N, stride, 32, 128))) return rc;
    return gemm2::launch_pair<gemm::KIND_TF32X3, Epi>(ctx, tm, epi, M, N, K);
  }
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.a[0], true, p.a_hi, K, M, stride, 32, gemm::BM))) return rc;
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.a[1], true, p.a_lo, K, M, stride, 32, gemm::BM))) return rc;
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[0], true, p.b_hi, K, N, stride, 32, bn))) return rc;
  if ((rc = gemm::encode_tmap_2d(ctx, &tm.b[1], true, p.b_lo, K, N, stride, 32, bn))) return rc;
  if (bn == 128) return gemm::launch<gemm::KIND_TF32X3, 128, 3, Epi>(ctx, tm, epi, M, N, K, splits);
  return gemm::launch<gemm::KIND_TF32X3, 64, 4, Epi>(ctx, tm, epi, M, N, K, splits);
}

// Epilogue: y = acc + bias[col] (one f32 add, as the reference's broadcast add on the
// rounded matmul result), optional store of the pre-activation, optional ReLU.
struct EpiBiasRelu {
  static constexpr bool kTmaCapable = true;
  static constexpr bool kPlanes = true;
  float* Y;
  const float* bias;  // may be null
  float* pre;         // may be null
  int ldy;
  int relu;
  int tma;  // store through tm.out[0] (and tm.out[1] for the pre-activation)
  // ReLU backward on the way out (TMA path only): y = mask[row][col] < 0 ? 0 : y, mask laid out like Y
  // (the pre-activation the layer below cached; nn/gates/activation/relu.v:21-25)
  const float* mask;
  int mask_fused;
  // TF32 operand planes of the stored result (TMA path only; see gemm::epilogue_chunk):
  // bit 0: [M, ld_rows] in Y's layout, bit 1: [N, ld_cols] of Y transposed
  int planes;
  float *rows_hi, *rows_lo, *cols_hi, *cols_lo;
  int ld_rows, ld_cols;
  // Bit j set = the mask zeroes column col0 + j of this row.  The GEMM kernels call this at the
  // start of a tile, long before the values exist, so that the loads' latency is off the path of
  // the stores at the tile's end; they then apply the bits and run the rest with mask_fused = 0.
  __device__ __forceinline__ uint32_t load_mask_bits(int row, int col0, int M, int N) const {
    uint32_t bits = 0;
    if (mask_fused && row < M) {
      const float* mrow = mask + (size_t)row * ldy + col0;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (col0 + j < N) {
          const float4 m4 = __ldg(reinterpret_cast<const float4*>(mrow + j));
          bits |= (m4.x < 0.f ? 1u : 0u) << j | (m4.y < 0.f ? 2u : 0u) << j | (m4.z < 0.f ? 4u : 0u) << j |
                  (m4.w < 0.f ? 8u : 0u) << j;
        }
      }
    }
    return bits;
  }
  // adds the bias in registers; returns true when the pre-activation has to be stored
  // separately before activate() applies the ReLU
  __device__ __forceinline__ bool transform(int row, int col0, uint32_t (&v)[32], int M, int N,
                                            bool mask_applied = false) const {
    if (mask_fused && !mask_applied && row < M) {
      const float* mrow = mask + (size_t)row * ldy + col0;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (col0 + j < N) {
          const float4 m4 = __ldg(reinterpret_cast<const float4*>(mrow + j));
          if (m4.x < 0.f) v[j] = 0u;
          if (m4.y < 0.f) v[j + 1] = 0u;
          if (m4.z < 0.f) v[j + 2] = 0u;
          if (m4.w < 0.f) v[j + 3] = 0u;
        }
      }
    }
    if (bias) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (col0 + j < N) {
          const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + col0 + j));
          v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), b4.x));
          v[j + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 1]), b4.y));
          v[j + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 2]), b4.z));
          v[j + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[j + 3]), b4.w));
        }
      }
    }
    if (pre) return true;
    activate(v);
    return false;
  }
  __device__ __forceinline__ void activate(uint32_t (&v)[32]) const {
    if (relu) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (__uint_as_float(v[j]) < 0.f) v[j] = 0u;
    }
  }
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&v)[32], int M, int N,
                                             int /*split*/) const {
    if (row >= M) return;
    float* y = Y + (size_t)row * ldy + col0;
    float* p = pre ? pre + (size_t)row * ldy + col0 : nullptr;
    if (col0 + 32 <= N && (ldy & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                               __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
        if (bias) {
          const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + col0 + j));
          o.x = __fadd_rn(o.x, b4.x);
          o.y = __fadd_rn(o.y, b4.y);
          o.z = __fadd_rn(o.z, b4.z);
          o.w = __fadd_rn(o.w, b4.w);
        }
        if (p) *reinterpret_cast<float4*>(p + j) = o;
        if (relu) {
          o.x = o.x < 0.f ? 0.f : o.x;
          o.y = o.y < 0.f ? 0.f : o.y;
          o.z = o.z < 0.f ? 0.f : o.z;
          o.w = o.w < 0.f ? 0.f : o.w;
        }
        *reinterpret_cast<float4*>(y + j) = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < N) {
          float o = __uint_as_float(v[j]);
          if (bias) o = __fadd_rn(o, bias[col0 + j]);
          if (p) p[j] = o;
          if (relu && o < 0.f) o = 0.f;
          y[j] = o;
        }
    }
  }
};

// Epilogue of a split-K launch: partial[split][row][col] = acc.
struct EpiPartial {
  static constexpr bool kTmaCapable = false;
  float* P;
  int ldp;
  size_t split_stride;
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&v)[32], int M, int N,
                                             int split) const {
    if (row >= M) return;
    float* y = P + split * split_stride + (size_t)row * ldp + col0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < N) y[j] = __uint_as_float(v[j]);
  }
};

// Writes op(src) as K-major TF32 planes hi/lo [rows, ld]; rows x kdim is the logical operand
// and `transposed` says src is stored [kdim, rows].
int split_operand(vtlb_ctx* ctx, const float* src, int rows, int kdim, bool transposed, int ld,
                  float* hi, float* lo);

// C[M,N] = op(A).op(B) (+bias, pre-activation copy, ReLU) on CUDA cores, for small products.
// With `a_rowsum` the launch also writes a_rowsum[m] = sum over k of op(A)(m, k) (f64 sums, rounded
// once) when it can (K not cut into ranges); *rowsum_done says whether it did.  With `mask` (shaped
// like C) the result is zeroed where mask < 0: a ReLU backward on the way out.
int sgemm_small(vtlb_ctx* ctx, int transA, int transB, int M, int N, int K, const float* A,
                const float* B, float* C, const float* bias, int relu, float* pre,
                float* a_rowsum = nullptr, bool* rowsum_done = nullptr, const float* mask = nullptr);

// Linear layers with at most 16 output features and at least 2048 inputs (linear_narrow.cu): Y = X.W^T + b,
// dX = G.W, dW = G^T.X with db = column sums of G (either of dW / db may be null), each streaming its
// long operand once.  narrow_linear_ok checks shape and the alignment of the three long operands.
bool narrow_linear_ok(int M, int N, int K, const void* a, const void* b, const void* c);
int narrow_linear_fwd(vtlb_ctx* ctx, const float* X, const float* W, const float* bias, float* Y, int M, int N, int K,
                      int relu, float* pre);
int narrow_linear_dx(vtlb_ctx* ctx, const float* G, const float* W, float* dX, int M, int N, int K);
int narrow_linear_dw(vtlb_ctx* ctx, const float* G, const float* X, float* dW, float* db, int M, int N, int K);

// out[i] = sum_s partial[s][i] (fixed order, f32 round-to-nearest), n elements.
int reduce_splits(vtlb_ctx* ctx, const float* partial, int splits, size_t n, float* out);

}  // namespace f32
