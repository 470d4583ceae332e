// Conv2D forward/backward (NCHW, groups = 1, dilation = 1) and 2-D max pooling.
// Reference: nn/internal/conv2d_forward_cpu_f32.v:26-62, conv2d_backward_cpu_f32.v:26-97,
// nn/internal/layers.v:21-84; replaces compute.conv2d_cuda / conv2d_backward_cuda
// (nn/internal/conv2d_cuda_d_cuda.v:51, conv2d_backward_cuda_d_cuda.v:25).
//
// The convolution runs as GEMMs on the same 3xTF32 tcgen05 kernel as Linear.  A
// memory-bound pass lowers the operands into K-major TF32 planes in the context
// scratch (im2col for the input, permutes for the gradient), with K = C*kh*kw in the
// weight tensor's own (ic, kh, kw) order so the weights need no re-layout:
//   forward : y[(b,oh,ow), oc] = col[(b,oh,ow), k] . W[oc, k]^T + bias[oc]
//   d_weight: dW[oc, k]        = gT[oc, m] . colT[k, m]^T      (split-K over m = (b,oh,ow))
//   d_input : dcolT[k, m]      = Wt[k, oc] . gM[m, oc]^T, then a col2im gather
//   d_bias  : per-channel sums of g (f64 partials)
#include "conv_igemm.cuh"
#include "conv_slab.cuh"
#include "conv_wgrad.cuh"
#include "f32_common.cuh"

namespace {

using f32::split1;

struct ConvDims {
  int B, C, H, W, O, kh, kw, ph, pw, sh, sw, OH, OW;
  int dh = 1, dw = 1;  // dilation (conv2d_forward_cpu_f32.v:26-62: ih = oh*s - p + kh*d)
  __host__ __device__ int P() const { return OH * OW; }
  __host__ __device__ int K() const { return C * kh * kw; }
  __host__ __device__ long long M() const { return (long long)B * OH * OW; }
};

// colT planes [K, ld >= M]: one row k = (ic, kh, kw) per blockIdx.y, so the decomposition of k
// costs nothing per element; a thread produces four consecutive m (one 16-byte store per plane)
// and walks (b, oh, ow) incrementally.  All index arithmetic is 32-bit (M < 2^31 is checked).
__global__ void __launch_bounds__(256) im2colT_split_kernel(const float* __restrict__ x, ConvDims d, int ld,
                                                            float* __restrict__ hi, float* __restrict__ lo) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int M = (int)d.M(), K = d.K(), P = d.OH * d.OW, khw = d.kh * d.kw;
  const bool vec = (ld & 3) == 0;
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    const int ic = k / khw, r = k - ic * khw;
    const int kh = r / d.kw, kw = r - kh * d.kw;
    float* hrow = hi + (size_t)k * ld;
    float* lrow = lo + (size_t)k * ld;
    for (int m4 = (blockIdx.x * blockDim.x + threadIdx.x) * 4; m4 < M; m4 += gridDim.x * blockDim.x * 4) {
      int b = m4 / P;
      const int p = m4 - b * P;
      int oh = p / d.OW, ow = p - oh * d.OW;
      float h[4], l[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = 0.0f;
        const int ih = oh * d.sh - d.ph + kh * d.dh, iw = ow * d.sw - d.pw + kw * d.dw;
        if (m4 + j < M && ih >= 0 && ih < d.H && iw >= 0 && iw < d.W)
          v = __ldg(x + (((size_t)b * d.C + ic) * d.H + ih) * d.W + iw);
        split1(v, h[j], l[j]);
        if (++ow == d.OW) {
          ow = 0;
          if (++oh == d.OH) {
            oh = 0;
            ++b;
          }
        }
      }
      if (vec && m4 + 3 < M) {
        *reinterpret_cast<float4*>(hrow + m4) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(lrow + m4) = make_float4(l[0], l[1], l[2], l[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (m4 + j < M) {
            hrow[m4 + j] = h[j];
            lrow[m4 + j] = l[j];
          }
      }
    }
  }
}

// col planes [M, ld >= K]: 32 x 32 tiles through shared memory (read along m, write along k).
// blockIdx.y picks the 32 columns k, whose (ic, kh, kw) are worked out once per block.
__global__ void __launch_bounds__(256) im2col_split_kernel(const float* __restrict__ x, ConvDims d, int ld,
                                                           float* __restrict__ hi, float* __restrict__ lo) {
  __shared__ float tile[32][33];
  __shared__ int k_off[32], k_h[32], k_w[32];  // offset of (ic, kh, kw) inside an image; -1: k >= K
  const int M = (int)d.M(), K = d.K(), P = d.OH * d.OW, khw = d.kh * d.kw;
  const int tiles_m = (M + 31) / 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int k0 = blockIdx.y * 32; k0 < K; k0 += gridDim.y * 32) {
    __syncthreads();
    if (threadIdx.x < 32) {
      const int k = k0 + threadIdx.x;
      if (k < K) {
        const int ic = k / khw, r = k - ic * khw;
        const int kh = r / d.kw, kw = r - kh * d.kw;
        k_off[threadIdx.x] = (ic * d.H + kh * d.dh) * d.W + kw * d.dw;
        k_h[threadIdx.x] = kh * d.dh;
        k_w[threadIdx.x] = kw * d.dw;
      } else {
        k_off[threadIdx.x] = -1;
        k_h[threadIdx.x] = 0;
        k_w[threadIdx.x] = 0;
      }
    }
    __syncthreads();
    for (int t = blockIdx.x; t < tiles_m; t += gridDim.x) {
      const int m0 = t * 32;
      const int m = m0 + tx;
      const int b = m / P, p = m - b * P;
      const int oh = p / d.OW, ow = p - oh * d.OW;
      const int ih0 = oh * d.sh - d.ph, iw0 = ow * d.sw - d.pw;
      const long long xb = ((long long)b * d.C * d.H + ih0) * d.W + iw0;  // + k_off: inside x whenever in bounds
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const int kk = ty + j;
        const int ih = ih0 + k_h[kk], iw = iw0 + k_w[kk];
        float v = 0.0f;
        if (m < M && k_off[kk] >= 0 && ih >= 0 && ih < d.H && iw >= 0 && iw < d.W) v = __ldg(x + (xb + k_off[kk]));
        tile[kk][tx] = v;
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const int mo = m0 + ty + j;
        const int k = k0 + tx;
        if (mo < M && k < K) {
          float h, l;
          split1(tile[tx][ty + j], h, l);
          hi[(size_t)mo * ld + k] = h;
          lo[(size_t)mo * ld + k] = l;
        }
      }
      __syncthreads();
    }
  }
}

// g is NCHW [B, O, P].  gT planes [O, ld >= M]: gT[oc][b*P + p] = g[b][oc][p] (rows of P copied).
// blockIdx.y walks the (b, oc) rows; four values per thread where the rows allow 16-byte accesses.
__global__ void __launch_bounds__(256) grad_to_OM_split_kernel(const float* __restrict__ g, int B, int O, int P,
                                                               int ld, float* __restrict__ hi,
                                                               float* __restrict__ lo) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const bool vec = (P & 3) == 0 && (ld & 3) == 0;
  for (int row = blockIdx.y; row < B * O; row += gridDim.y) {
    const int b = row / O, oc = row - b * O;
    const float* src = g + (size_t)row * P;
    const size_t o = (size_t)oc * ld + (size_t)b * P;
    for (int p4 = (blockIdx.x * blockDim.x + threadIdx.x) * 4; p4 < P; p4 += gridDim.x * blockDim.x * 4) {
      if (vec) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src + p4));
        float4 h, l;
        split1(v.x, h.x, l.x);
        split1(v.y, h.y, l.y);
        split1(v.z, h.z, l.z);
        split1(v.w, h.w, l.w);
        *reinterpret_cast<float4*>(hi + o + p4) = h;
        *reinterpret_cast<float4*>(lo + o + p4) = l;
      } else {
        for (int j = 0; j < 4 && p4 + j < P; ++j) {
          float h, l;
          split1(src[p4 + j], h, l);
          hi[o + p4 + j] = h;
          lo[o + p4 + j] = l;
        }
      }
    }
  }
}

// gM planes [M, ld >= O]: gM[b*P + p][oc] = g[b][oc][p]: a [O, P] -> [P, O] transpose per image.
__global__ void __launch_bounds__(256) grad_to_MO_split_kernel(const float* __restrict__ g, int B, int O, int P,
                                                               int ld, float* __restrict__ hi,
                                                               float* __restrict__ lo) {
  __shared__ float tile[32][33];
  const int tiles_o = (O + 31) / 32, tiles_p = (P + 31) / 32;
  const long long ntiles = (long long)B * tiles_o * tiles_p;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int b = (int)(t / (tiles_o * tiles_p));
    const int r = (int)(t % (tiles_o * tiles_p));
    const int o0 = (r / tiles_p) * 32, p0 = (r % tiles_p) * 32;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int oc = o0 + ty + j, p = p0 + tx;
      tile[ty + j][tx] = (oc < O && p < P) ? g[((size_t)b * O + oc) * P + p] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      const int p = p0 + ty + j, oc = o0 + tx;
      if (p < P && oc < O) {
        float h, l;
        split1(tile[tx][ty + j], h, l);
        const size_t o = ((size_t)b * P + p) * ld + oc;
        hi[o] = h;
        lo[o] = l;
      }
    }
    __syncthreads();
  }
}

// dx[b, ic, ih, iw] = sum over (kh, kw) of dcolT[(ic, kh, kw), (b, oh, ow)] where the window
// position maps back onto (ih, iw); a gather, so no atomics and a fixed summation order.  dcolT is
// stored [K, ldm >= M]: consecutive threads (iw) read consecutive m.
__global__ void __launch_bounds__(256) col2im_gather_kernel(const float* __restrict__ dcolT, ConvDims d, int ldm,
                                                            float* __restrict__ dx) {
  // blockIdx.y walks the (b, ic) planes, threads the H*W positions of a plane; 32-bit arithmetic
  const int HW = d.H * d.W, khw = d.kh * d.kw;
  const bool unit_stride = d.sh == 1 && d.sw == 1;
  for (int plane = blockIdx.y; plane < d.B * d.C; plane += gridDim.y) {
    const int b = plane / d.C, ic = plane - b * d.C;
    const float* src = dcolT + (size_t)ic * khw * ldm + (size_t)b * d.OH * d.OW;
    float* dst = dx + (size_t)plane * HW;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < HW; i += gridDim.x * blockDim.x) {
      const int ih = i / d.W, iw = i - ih * d.W;
      float s = 0.0f;
      for (int kh = 0; kh < d.kh; ++kh) {
        const int th = ih + d.ph - kh * d.dh;
        if (th < 0) continue;
        int oh = th;
        if (!unit_stride) {
          if (th % d.sh) continue;
          oh = th / d.sh;
        }
        if (oh >= d.OH) continue;
        for (int kw = 0; kw < d.kw; ++kw) {
          const int tw = iw + d.pw - kw * d.dw;
          if (tw < 0) continue;
          int ow = tw;
          if (!unit_stride) {
            if (tw % d.sw) continue;
            ow = tw / d.sw;
          }
          if (ow >= d.OW) continue;
          s = __fadd_rn(s, __ldg(src + (size_t)(kh * d.kw + kw) * ldm + oh * d.OW + ow));
        }
      }
      dst[i] = s;
    }
  }
}

// per-channel sums of g [B, O, P] in f64: partial[s][oc] over images b == s (mod S)
__global__ void __launch_bounds__(256) chan_sum_partial_kernel(const float* __restrict__ g, int B, int O, int P,
                                                               double* __restrict__ partial) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ double sm[8];
  const int oc = blockIdx.x, s = blockIdx.y, S = gridDim.y;
  double acc = 0.0;
  for (int b = s; b < B; b += S) {
    const float* row = g + ((size_t)b * O + oc) * P;
    if ((P & 3) == 0) {  // rows start 16-byte aligned
      double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
      for (int p = threadIdx.x * 4; p < P; p += blockDim.x * 4) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(row + p));
        a0 += (double)v.x;
        a1 += (double)v.y;
        a2 += (double)v.z;
        a3 += (double)v.w;
      }
      acc += (a0 + a1) + (a2 + a3);
    } else {
      for (int p = threadIdx.x; p < P; p += blockDim.x) acc += (double)row[p];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sm[w];
    partial[(size_t)s * O + oc] = t;
  }
}
__global__ void chan_sum_final_kernel(const double* __restrict__ partial, int S, int O, float* __restrict__ out) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int oc = blockIdx.x * blockDim.x + threadIdx.x;
  if (oc >= O) return;
  double t = 0.0;
  for (int s = 0; s < S; ++s) t += partial[(size_t)s * O + oc];
  out[oc] = (float)t;
}

// Forward epilogue: D[m, oc] -> y[b, oc, oh, ow] (+ bias[oc], optional pre-activation copy and
// ReLU).  For each output channel the 32 lanes of a warp hold 32 consecutive pixels, so every
// store instruction writes one contiguous 128-byte run.
struct EpiConvOut {
  static constexpr bool kTmaCapable = false;  // NCHW scatter: its own per-channel coalesced stores
  float* Y;
  const float* bias;
  float* pre;
  int O, P, relu;
  // the staged epilogues of the implicit-GEMM kernels: the bias of channel oc (0 without a bias)
  __device__ __forceinline__ float bias_at(int oc, int N) const {
    return (bias && oc < N) ? __ldg(bias + oc) : 0.0f;
  }
  __device__ __forceinline__ void operator()(int row, int col0, const uint32_t (&v)[32], int M, int N,
                                             int /*split*/) const {
    if (row >= M) return;
    const int b = row / P, p = row - b * P;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int oc = col0 + j;
      if (oc < N) {
        float o = __uint_as_float(v[j]);
        if (bias) o = __fadd_rn(o, __ldg(bias + oc));
        const size_t idx = ((size_t)b * O + oc) * P + p;
        if (pre) pre[idx] = o;
        if (relu && o < 0.f) o = 0.f;
        Y[idx] = o;
      }
    }
  }
};

// ---------------------------------------------------------------- max pooling
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          int32_t* __restrict__ idx, int B, int C, int H, int W,
                                                          int kh, int kw, int ph, int pw, int sh, int sw,
                                                          int OH, int OW) {
  // 32-bit arithmetic: the host checks B*C*H*W < 2^31
  const int n = B * C * OH * OW;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int w = i % OW;
    const int r = i / OW;
    const int h = r % OH;
    const int nc = r / OH;
    int hs = h * sh - ph, ws = w * sw - pw;
    int he = hs + kh, we = ws + kw;
    hs = max(hs, 0);
    ws = max(ws, 0);
    he = min(he, H);
    we = min(we, W);
    float best = -INFINITY;
    int bi = -1;
    for (int a = hs; a < he; ++a)
      for (int c = ws; c < we; ++c) {
        const int fi = (nc * H + a) * W + c;
        const float val = x[fi];
        if (bi < 0 || val > best) {
          best = val;
          bi = fi;
        }
      }
    y[i] = best;
    idx[i] = bi;
  }
}
// The common case, 2 x 2 windows at stride 2 without padding on rows of a multiple of 4 values:
// a thread reads 16 bytes of two adjacent rows and writes two outputs.  Candidates are visited
// in the same order, with the same comparison, as in the general kernel.
__global__ void __launch_bounds__(256) maxpool2x2_fwd_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                             int32_t* __restrict__ idx, int planes, int H, int W) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int OH = H >> 1, OW = W >> 1, W4 = W >> 2;
  const int n = planes * OH * W4;  // items: (plane, output row, group of 4 input columns)
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int j = i % W4;
    const int r = i / W4;
    const int h = r % OH;
    const int nc = r / OH;
    const int f0 = (nc * H + 2 * h) * W + 4 * j;  // flat index of the first value of the upper row
    const float4 a = __ldg(reinterpret_cast<const float4*>(x + f0));
    const float4 b = __ldg(reinterpret_cast<const float4*>(x + f0 + W));
    float best0 = a.x;
    int bi0 = f0;
    if (a.y > best0) { best0 = a.y; bi0 = f0 + 1; }
    if (b.x > best0) { best0 = b.x; bi0 = f0 + W; }
    if (b.y > best0) { best0 = b.y; bi0 = f0 + W + 1; }
    float best1 = a.z;
    int bi1 = f0 + 2;
    if (a.w > best1) { best1 = a.w; bi1 = f0 + 3; }
    if (b.z > best1) { best1 = b.z; bi1 = f0 + W + 2; }
    if (b.w > best1) { best1 = b.w; bi1 = f0 + W + 3; }
    const int o = (nc * OH + h) * OW + 2 * j;
    *reinterpret_cast<float2*>(y + o) = make_float2(best0, best1);
    *reinterpret_cast<int2*>(idx + o) = make_int2(bi0, bi1);
  }
}
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ idx,
                                                          float* __restrict__ dx, size_t n_out) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n_out; i += (size_t)gridDim.x * blockDim.x) {
    const int32_t t = idx[i];
    if (t >= 0) atomicAdd(dx + t, g[i]);  // windows overlap only when stride < kernel
  }
}

// Backward of the 2x2 / stride 2 / no padding window.  The windows tile the input, so every input
// element has exactly one window: dX is written directly (no zero fill, no scatter), items as in
// the forward kernel.  With `c` (the pre-activation cached by a ReLU whose output the pool read)
// that ReLU's backward is applied as well: only the winning position of a window carries a
// gradient, and it is dropped where c there is negative (the reference's comparison: zero and NaN
// pass) -- one gathered read instead of another pass over the full-size tensor.
__global__ void __launch_bounds__(256) maxpool2x2_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ idx,
                                                             const float* __restrict__ c, float* __restrict__ dx,
                                                             int planes, int H, int W) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int OH = H >> 1, OW = W >> 1, W4 = W >> 2;
  const int n = planes * OH * W4;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int j = i % W4;
    const int r = i / W4;
    const int h = r % OH;
    const int nc = r / OH;
    const int f0 = (nc * H + 2 * h) * W + 4 * j;
    const int o = (nc * OH + h) * OW + 2 * j;
    float2 gv = __ldg(reinterpret_cast<const float2*>(g + o));
    const int2 t = __ldg(reinterpret_cast<const int2*>(idx + o));
    if (c) {
      if (__ldg(c + t.x) < 0.0f) gv.x = 0.0f;
      if (__ldg(c + t.y) < 0.0f) gv.y = 0.0f;
    }
    const int p0 = t.x - f0, p1 = t.y - f0;
    float4 a, b;
    a.x = p0 == 0 ? gv.x : 0.0f;
    a.y = p0 == 1 ? gv.x : 0.0f;
    b.x = p0 == W ? gv.x : 0.0f;
    b.y = p0 == W + 1 ? gv.x : 0.0f;
    a.z = p1 == 2 ? gv.y : 0.0f;
    a.w = p1 == 3 ? gv.y : 0.0f;
    b.z = p1 == W + 2 ? gv.y : 0.0f;
    b.w = p1 == W + 3 ? gv.y : 0.0f;
    *reinterpret_cast<float4*>(dx + f0) = a;
    *reinterpret_cast<float4*>(dx + f0 + W) = b;
  }
}

// B operand of the implicit GEMM with the channel running fastest in k (t = tap index):
//   forward        planes [O, ld >= taps*C]: out[oc][t*C + ic] = W[oc][ic][t]
//   input gradient planes [C, ld >= taps*O]: out[ic][t*O + oc] = W[oc][ic][t]
__global__ void __launch_bounds__(256) regroup_weights_split_kernel(const float* __restrict__ w, int O, int C, int taps,
                                                                    int for_input_grad, int ld, float* __restrict__ hi,
                                                                    float* __restrict__ lo) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done from here on
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int n = O * C * taps;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int t = i % taps, r = i / taps, ic = r % C, oc = r / C;
    float h, l;
    split1(w[i], h, l);
    const size_t o = for_input_grad ? (size_t)ic * ld + (size_t)t * O + oc : (size_t)oc * ld + (size_t)t * C + ic;
    hi[o] = h;
    lo[o] = l;
  }
}

// The implicit GEMM serves the forward product and (for unit stride) the input gradient as long
// as the (channel, tap) table fits in shared memory; VTLB_CONV_IGEMM=0 keeps the lowered path.
bool use_igemm(int K) {
  static int env = -1;
  if (env < 0) {
    const char* e = getenv("VTLB_CONV_IGEMM");
    env = e ? atoi(e) : 1;
  }
  return env != 0 && K <= igemm::MAX_K;
}
bool igemm_taps_ok(int kh, int kw) { return kh * kw <= 32; }  // one validity bit per tap in a 32-bit word

int check_conv(vtlb_ctx* ctx, const char* fn, ConvDims& d) {
  if (d.B <= 0 || d.C <= 0 || d.H <= 0 || d.W <= 0 || d.O <= 0 || d.kh <= 0 || d.kw <= 0 || d.ph < 0 ||
      d.pw < 0 || d.sh <= 0 || d.sw <= 0 || d.dh <= 0 || d.dw <= 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: bad convolution geometry", fn);
  d.OH = (d.H + 2 * d.ph - d.dh * (d.kh - 1) - 1) / d.sh + 1;
  d.OW = (d.W + 2 * d.pw - d.dw * (d.kw - 1) - 1) / d.sw + 1;
  if (d.OH <= 0 || d.OW <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "%s: empty output", fn);
  if (d.M() > 0x7fffffffLL || d.M() * d.K() > (1LL << 40) || (long long)d.B * d.O > 0x7fffffffLL ||
      (long long)d.B * d.C * d.H * d.W > 0x7fffffffLL)
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: problem too large for the lowered GEMM", fn);
  return VTLB_OK;
}

}  // namespace

namespace {

int conv2d_fwd_impl(vtlb_ctx* ctx, const char* fn, const void* d_x, const void* d_w, const void* d_bias_or_null,
                    void* d_y, int B, int C, int H, int W, int O, int kh, int kw, int ph, int pw, int sh, int sw,
                    int dh, int dw, int relu, void* d_pre_or_null) {
  ConvDims d{B, C, H, W, O, kh, kw, ph, pw, sh, sw, 0, 0};
  d.dh = dh;
  d.dw = dw;
  int rc = check_conv(ctx, fn, d);
  if (rc) return rc;
  if (!d_x || !d_w || !d_y) return vtlb_fail(ctx, VTLB_EINVAL, "%s: null pointer", fn);
  const int M = (int)d.M(), K = d.K();
  f32::Planes p;
  if (dh == 1 && dw == 1 && use_igemm(K) && igemm_taps_ok(kh, kw)) {  // dilated windows take the lowered route
    if ((rc = f32::alloc_planes(ctx, 0, O, K, 0, &p))) return rc;
    VTLB_CUDA(ctx, vtlb_launch_early(regroup_weights_split_kernel, dim3(f32::grid_for(ctx, (size_t)O * K, 256)), dim3(256),
                                     0, ctx->stream, (const float*)d_w, O, C, kh * kw, 0, p.ld, p.b_hi, p.b_lo));
    VTLB_LAUNCHED(ctx);
    const igemm::Geometry g{B, C, H, W, d.OH, d.OW, sh, sw, kh, kw, -ph, -pw, 1, K};
    EpiConvOut epi{(float*)d_y, (const float*)d_bias_or_null, (float*)d_pre_or_null, O, d.P(), relu};
    cslab::Tiling tl;
    if (cslab::usable(g, &tl) && vtlb_aligned16(d_y) && (!d_pre_or_null || vtlb_aligned16(d_pre_or_null)))
      return cslab::launch(ctx, (const float*)d_x, g, tl, p.b_hi, p.b_lo, p.ld, epi, O);
    return igemm::launch(ctx, (const float*)d_x, g, p.b_hi, p.b_lo, p.ld, epi, M, O);
  }
  if ((rc = f32::alloc_planes(ctx, M, O, K, 0, &p))) return rc;
  {
    const int ky = (K + 31) / 32 < 64 ? (K + 31) / 32 : 64;
    int gx = (ctx->sm_count * 16 + ky - 1) / ky;
    if (gx > (M + 31) / 32) gx = (M + 31) / 32;
    im2col_split_kernel<<<dim3(gx, ky), 256, 0, ctx->stream>>>((const float*)d_x, d, p.ld, p.a_hi, p.a_lo);
  }
  VTLB_LAUNCHED(ctx);
  if ((rc = f32::split_operand(ctx, (const float*)d_w, O, K, false, p.ld, p.b_hi, p.b_lo))) return rc;
  EpiConvOut epi{(float*)d_y, (const float*)d_bias_or_null, (float*)d_pre_or_null, O, d.P(), relu};
  return f32::launch_tf32x3(ctx, p, M, O, K, epi);
}

int conv2d_bwd_impl(vtlb_ctx* ctx, const void* d_g, const void* d_x, const void* d_w, void* d_dx_or_null,
                    void* d_dw_or_null, void* d_db_or_null, int B, int C, int H, int W, int O, int kh, int kw, int ph,
                    int pw, int sh, int sw, int dh, int dw) {
  ConvDims d{B, C, H, W, O, kh, kw, ph, pw, sh, sw, 0, 0};
  d.dh = dh;
  d.dw = dw;
  const bool dilated = dh != 1 || dw != 1;
  int rc = check_conv(ctx, "vtlb_conv2d_bwd_f32", d);
  if (rc) return rc;
  if (!d_g) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_conv2d_bwd_f32: null gradient");
  const int M = (int)d.M(), K = d.K(), P = d.P();
  const float* g = (const float*)d_g;
  if (d_dw_or_null && cwgrad::usable(sh, sw, kh, kw, d.OW, dilated ? 2 : 1)) {
    // unit stride, window at most 3 x 3, output rows of at most 32 pixels: the implicit GEMM over pixels
    if (!d_x) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_conv2d_bwd_f32: d_weight needs x");
    const int parts = cwgrad::parts_for(ctx, B, C, O, d.OH);
    void* scr = nullptr;
    if ((rc = vtlb_scratch(ctx, (size_t)parts * O * K * sizeof(float), &scr))) return rc;
    if ((rc = cwgrad::launch(ctx, (const float*)d_x, g, (float*)scr, (float*)d_dw_or_null, B, C, H, W, O, d.OH, d.OW,
                             kh, kw, ph, pw)))
      return rc;
  } else if (d_dw_or_null) {  // dW[oc, k] = sum_m g[m, oc] * col[m, k]
    if (!d_x) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_conv2d_bwd_f32: d_weight needs x");
    const int mn_tiles = ((O + 127) / 128) * ((K + 63) / 64);
    int want = (2 * ctx->sm_count + mn_tiles - 1) / mn_tiles;
    const int max_by_len = (M + 1023) / 1024;  // at least 1024 rows of the contraction per range
    if (want > max_by_len) want = max_by_len;
    const int S = f32::effective_splits(M, want);
    f32::Planes p;
    if ((rc = f32::alloc_planes(ctx, O, K, M, (size_t)S * O * K * sizeof(float), &p))) return rc;
    {
      const long long rows = (long long)B * O;
      VTLB_CUDA(ctx, vtlb_launch_early(grad_to_OM_split_kernel,
                                       dim3((P + 1023) / 1024, (unsigned)(rows < 32768 ? rows : 32768)), dim3(256), 0,
                                       ctx->stream, g, B, O, P, p.ld, p.a_hi, p.a_lo));
    }
    VTLB_LAUNCHED(ctx);
    {
      const int ky = K < 4096 ? K : 4096;
      int gx = (ctx->sm_count * 16 + ky - 1) / ky;
      if (gx > (M + 1023) / 1024) gx = (M + 1023) / 1024;
      if (gx < 1) gx = 1;
      VTLB_CUDA(ctx, vtlb_launch_early(im2colT_split_kernel, dim3(gx, ky), dim3(256), 0, ctx->stream, (const float*)d_x,
                                       d, p.ld, p.b_hi, p.b_lo));
    }
    VTLB_LAUNCHED(ctx);
    if (S == 1) {
      f32::EpiBiasRelu epi{(float*)d_dw_or_null, nullptr, nullptr, K, 0};
      if (!vtlb_aligned16(d_dw_or_null)) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_conv2d_bwd_f32: dW not 16-byte aligned");
      if ((rc = f32::launch_tf32x3(ctx, p, O, K, M, epi, 1))) return rc;
    } else {
      f32::EpiPartial epi{(float*)p.extra, K, (size_t)O * K};
      if ((rc = f32::launch_tf32x3(ctx, p, O, K, M, epi, S))) return rc;
      if ((rc = f32::reduce_splits(ctx, (const float*)p.extra, S, (size_t)O * K, (float*)d_dw_or_null))) return rc;
    }
  }
  if (d_dx_or_null && !dilated && sh == 1 && sw == 1 && use_igemm(O * kh * kw) && igemm_taps_ok(kh, kw) &&
      (long long)B * O * d.OH * d.OW <= 0x7fffffffLL) {
    // dx[(b, ih, iw), ic] = sum over (oc, a, b) of g[b][oc][ih + ph - a][iw + pw - b] * W[oc][ic][a][b]
    if (!d_w) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_conv2d_bwd_f32: d_input needs the weights");
    const int Kd = O * kh * kw;
    f32::Planes p;
    if ((rc = f32::alloc_planes(ctx, 0, C, Kd, 0, &p))) return rc;
    VTLB_CUDA(ctx, vtlb_launch_early(regroup_weights_split_kernel, dim3(f32::grid_for(ctx, (size_t)O * C * kh * kw, 256)),
                                     dim3(256), 0, ctx->stream, (const float*)d_w, O, C, kh * kw, 1, p.ld, p.b_hi, p.b_lo));
    VTLB_LAUNCHED(ctx);
    const igemm::Geometry gg{B, O, d.OH, d.OW, H, W, 1, 1, kh, kw, ph, pw, -1, Kd};
    EpiConvOut epi{(float*)d_dx_or_null, nullptr, nullptr, C, H * W, 0};
    cslab::Tiling tl;
    if (cslab::usable(gg, &tl) && vtlb_aligned16(d_dx_or_null))
      rc = cslab::launch(ctx, g, gg, tl, p.b_hi, p.b_lo, p.ld, epi, C);
    else
      rc = igemm::launch(ctx, g, gg, p.b_hi, p.b_lo, p.ld, epi, B * H * W, C);
    if (rc) return rc;
  } else if (d_dx_or_null) {  // dcolT[k, m] = sum_oc W[oc, k] * g[m, oc]; dx = col2im(dcolT)
    if (!d_w) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_conv2d_bwd_f32: d_input needs the weights");
    const int ldm = (int)vtlb_round_up((size_t)M, 4);
    f32::Planes p;
    if ((rc = f32::alloc_planes(ctx, K, M, O, (size_t)K * ldm * sizeof(float), &p))) return rc;
    if ((rc = f32::split_operand(ctx, (const float*)d_w, K, O, true, p.ld, p.a_hi, p.a_lo))) return rc;
    const long long tiles = (long long)B * ((O + 31) / 32) * ((P + 31) / 32);
    grad_to_MO_split_kernel<<<f32::grid_for(ctx, (size_t)tiles, 1), 256, 0, ctx->stream>>>(g, B, O, P, p.ld, p.b_hi,
                                                                                          p.b_lo);
    VTLB_LAUNCHED(ctx);
    f32::EpiBiasRelu epi{(float*)p.extra, nullptr, nullptr, ldm, 0};
    if ((rc = f32::launch_tf32x3(ctx, p, K, M, O, epi))) return rc;
    {
      const long long planes = (long long)B * C;
      col2im_gather_kernel<<<dim3((H * W + 255) / 256 < 64 ? (H * W + 255) / 256 : 64,
                                  (unsigned)(planes < 32768 ? planes : 32768)),
                             256, 0, ctx->stream>>>((const float*)p.extra, d, ldm, (float*)d_dx_or_null);
    }
    VTLB_LAUNCHED(ctx);
  }
  if (d_db_or_null) {
    int S = B < 32 ? B : 32;
    void* scr = nullptr;
    if ((rc = vtlb_scratch(ctx, (size_t)S * O * sizeof(double), &scr))) return rc;
    VTLB_CUDA(ctx, vtlb_launch_early(chan_sum_partial_kernel, dim3(O, S), dim3(256), 0, ctx->stream, g, B, O, P,
                                     (double*)scr));
    VTLB_LAUNCHED(ctx);
    VTLB_CUDA(ctx, vtlb_launch_early(chan_sum_final_kernel, dim3((O + 127) / 128), dim3(128), 0, ctx->stream,
                                     (const double*)scr, S, O, (float*)d_db_or_null));
    VTLB_LAUNCHED(ctx);
  }
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_conv2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, const void* d_w, const void* d_bias_or_null,
                                 void* d_y, int B, int C, int H, int W, int O, int kh, int kw, int ph, int pw,
                                 int sh, int sw, int relu, void* d_pre_or_null) {
  VTLB_ENTER(ctx);
  return conv2d_fwd_impl(ctx, "vtlb_conv2d_fwd_f32", d_x, d_w, d_bias_or_null, d_y, B, C, H, W, O, kh, kw, ph, pw, sh,
                         sw, 1, 1, relu, d_pre_or_null);
}

VTLB_API int vtlb_conv2d_fwd_f32_dilated(vtlb_ctx* ctx, const void* d_x, const void* d_w, const void* d_bias_or_null,
                                         void* d_y, int B, int C, int H, int W, int O, int kh, int kw, int ph,
                                         int pw, int sh, int sw, int dh, int dw, int relu, void* d_pre_or_null) {
  VTLB_ENTER(ctx);
  return conv2d_fwd_impl(ctx, "vtlb_conv2d_fwd_f32_dilated", d_x, d_w, d_bias_or_null, d_y, B, C, H, W, O, kh, kw, ph,
                         pw, sh, sw, dh, dw, relu, d_pre_or_null);
}

VTLB_API int vtlb_conv2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_x, const void* d_w,
                                 void* d_dx_or_null, void* d_dw_or_null, void* d_db_or_null, int B, int C, int H,
                                 int W, int O, int kh, int kw, int ph, int pw, int sh, int sw) {
  VTLB_ENTER(ctx);
  return conv2d_bwd_impl(ctx, d_g, d_x, d_w, d_dx_or_null, d_dw_or_null, d_db_or_null, B, C, H, W, O, kh, kw, ph, pw,
                         sh, sw, 1, 1);
}

VTLB_API int vtlb_conv2d_bwd_f32_dilated(vtlb_ctx* ctx, const void* d_g, const void* d_x, const void* d_w,
                                         void* d_dx_or_null, void* d_dw_or_null, void* d_db_or_null, int B, int C,
                                         int H, int W, int O, int kh, int kw, int ph, int pw, int sh, int sw, int dh,
                                         int dw) {
  VTLB_ENTER(ctx);
  return conv2d_bwd_impl(ctx, d_g, d_x, d_w, d_dx_or_null, d_dw_or_null, d_db_or_null, B, C, H, W, O, kh, kw, ph, pw,
                         sh, sw, dh, dw);
}

VTLB_API int vtlb_maxpool2d_fwd_f32(vtlb_ctx* ctx, const void* d_x, void* d_y, void* d_idx, int B, int C, int H,
                                    int W, int kh, int kw, int ph, int pw, int sh, int sw) {
  VTLB_ENTER(ctx);
  if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2d_fwd_f32: bad geometry");
  const int OH = (H + 2 * ph - kh) / sh + 1, OW = (W + 2 * pw - kw) / sw + 1;
  if (OH <= 0 || OW <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2d_fwd_f32: empty output");
  if ((long long)B * C * H * W > 0x7fffffffLL)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2d_fwd_f32: input too large for 32-bit indices");
  if (!d_x || !d_y || !d_idx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2d_fwd_f32: null pointer");
  const size_t n = (size_t)B * C * OH * OW;
  if (kh == 2 && kw == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && (W & 3) == 0 && (H & 1) == 0 &&
      vtlb_aligned16(d_x) && vtlb_aligned16(d_y) && vtlb_aligned16(d_idx)) {
    VTLB_CUDA(ctx, vtlb_launch_early(maxpool2x2_fwd_kernel, dim3(f32::grid_for(ctx, n / 2, 1024)), dim3(256), 0,
                                     ctx->stream, (const float*)d_x, (float*)d_y, (int32_t*)d_idx, B * C, H, W));
    VTLB_LAUNCHED(ctx);
    return VTLB_OK;
  }
  maxpool_fwd_kernel<<<f32::grid_for(ctx, n, 1024), 256, 0, ctx->stream>>>(
      (const float*)d_x, (float*)d_y, (int32_t*)d_idx, B, C, H, W, kh, kw, ph, pw, sh, sw, OH, OW);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_maxpool2x2_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_idx, const void* d_relu_cache_or_null,
                                     void* d_dx, int B, int C, int H, int W) {
  VTLB_ENTER(ctx);
  if (!d_g || !d_idx || !d_dx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2x2_bwd_f32: null pointer");
  if (B < 0 || C <= 0 || H <= 0 || W <= 0 || (W & 3) || (H & 1) || (size_t)B * C * H * W > 0x7fffffffu)
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2x2_bwd_f32: needs H %% 2 = 0, W %% 4 = 0, < 2^31 elements (got %dx%dx%dx%d)",
                     B, C, H, W);
  if (!vtlb_aligned16(d_g) || !vtlb_aligned16(d_idx) || !vtlb_aligned16(d_dx))
    return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2x2_bwd_f32: pointers must be 16-byte aligned");
  const size_t n = (size_t)B * C * (H / 2) * (W / 4);
  if (n == 0) return VTLB_OK;
  VTLB_CUDA(ctx, vtlb_launch_early(maxpool2x2_bwd_kernel, dim3(f32::grid_for(ctx, n, 1024)), dim3(256), 0, ctx->stream,
                                   (const float*)d_g, (const int32_t*)d_idx, (const float*)d_relu_cache_or_null, (float*)d_dx,
                                   B * C, H, W));
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_maxpool2d_bwd_f32(vtlb_ctx* ctx, const void* d_g, const void* d_idx, void* d_dx, size_t n_out,
                                    size_t n_in) {
  VTLB_ENTER(ctx);
  if (!d_g || !d_idx || !d_dx) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_maxpool2d_bwd_f32: null pointer");
  VTLB_CUDA(ctx, cudaMemsetAsync(d_dx, 0, n_in * sizeof(float), ctx->stream));
  if (n_out == 0) return VTLB_OK;
  maxpool_bwd_kernel<<<f32::grid_for(ctx, n_out, 1024), 256, 0, ctx->stream>>>((const float*)d_g, (const int32_t*)d_idx,
                                                                              (float*)d_dx, n_out);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

