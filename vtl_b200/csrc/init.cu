// Parameter initialisers: the random fills behind vtl's kaiming_uniform / kaiming_normal
// (nn/internal/init.v:35-70 -> vtl.random / vtl.normal, rand.v:57-79).
//
// The reference draws from V's global generator, seeded from the wall clock, so its streams
// cannot be reproduced; what is reproduced is the distribution (range or mean / sigma).  Here
// every element is a pure function of (seed, index) -- a counter-based generator -- so a fill is
// reproducible, independent of the launch geometry, and a CPU restatement can be compared
// element by element:
//   z   = splitmix64(seed + (i + 1) * 0x9E3779B97F4A7C15)
//   uniform: u = (z >> 40) * 2^-24  in [0, 1);   x = lo + u * (hi - lo)   (two f32 roundings)
//   normal : u1 = ((z >> 32) + 1) * 2^-32 in (0, 1], u2 = (z & 0xffffffff) * 2^-32,
//            x = (f32)(mu + sigma * sqrt(-2 ln u1) * cos(2 pi u2))        (Box-Muller in f64)
// Memory-bound: 4 bytes written per element.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

__global__ void __launch_bounds__(256) init_uniform_kernel(float* __restrict__ out, size_t n, float lo,
                                                           float span, uint64_t seed) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t z = splitmix64(seed + (i + 1) * 0x9E3779B97F4A7C15ull);
    const float u = (float)(uint32_t)(z >> 40) * 5.9604644775390625e-8f;  // exact: 24 bits * 2^-24
    out[i] = __fadd_rn(lo, __fmul_rn(u, span));
  }
}

__global__ void __launch_bounds__(256) init_normal_kernel(float* __restrict__ out, size_t n, double mu,
                                                          double sigma, uint64_t seed) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t z = splitmix64(seed + (i + 1) * 0x9E3779B97F4A7C15ull);
    const double u1 = ((double)(uint32_t)(z >> 32) + 1.0) * 2.3283064365386963e-10;  // 2^-32
    const double u2 = (double)(uint32_t)z * 2.3283064365386963e-10;
    const double r = sqrt(-2.0 * log(u1));
    out[i] = (float)(mu + sigma * (r * cos(6.283185307179586476925286766559 * u2)));
  }
}

int init_grid(vtlb_ctx* ctx, size_t n) {
  size_t b = (n + 255) / 256, cap = (size_t)ctx->sm_count * 8;
  return (int)(b > cap ? cap : (b < 1 ? 1 : b));
}

}  // namespace

VTLB_API int vtlb_init_uniform_f32(vtlb_ctx* ctx, void* d_out, size_t n, float lo, float hi, uint64_t seed) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_out) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_init_uniform_f32: null pointer");
  if (!(lo <= hi)) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_init_uniform_f32: need lo <= hi");
  init_uniform_kernel<<<init_grid(ctx, n), 256, 0, ctx->stream>>>((float*)d_out, n, lo, hi - lo, seed);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}

VTLB_API int vtlb_init_normal_f32(vtlb_ctx* ctx, void* d_out, size_t n, double mu, double sigma, uint64_t seed) {
  VTLB_ENTER(ctx);
  if (n == 0) return VTLB_OK;
  if (!d_out) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_init_normal_f32: null pointer");
  if (!(sigma >= 0.0)) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_init_normal_f32: sigma must be >= 0");
  init_normal_kernel<<<init_grid(ctx, n), 256, 0, ctx->stream>>>((float*)d_out, n, mu, sigma, seed);
  VTLB_LAUNCHED(ctx);
  return VTLB_OK;
}
