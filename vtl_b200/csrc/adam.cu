// Fused multi-tensor optimizer steps: Adam, AdamW, SGD, RMSProp.  One launch updates every parameter tensor
// of the model: 28 bytes of HBM traffic per parameter (read g, theta, m, v;
// write theta, m, v), 32 with the fused gradient clear.
//
// Adam follows adam_step_f32_cpu (nn/optimizers/adam_step_f32.v:6-21) in f32
// with each operation rounded on its own; AdamW follows AdamWOptimizer.update
// (nn/optimizers/adamw.v:78-106): f64 arithmetic on f32 state, m and v rounded
// to f32 before the parameter update reads them.  One deliberate deviation: the
// moments are the textbook m = b1*m + (1-b1)*g, v = b2*v + (1-b2)*g*g, as the
// reference's Adam computes them; adamw.v:86-93 as written hands its closures
// the operands in the other order (napply passes the receiver first, fun.v:37-44)
// and would evaluate m = b1*g + (1-b1)*m, v = b2*g + (1-b2)*v*v.  SGD follows internal.sgd_optimize
// (nn/internal/optimizers.v:6-13: theta - (f32)lr * g in f32, 12 bytes per parameter) and RMSProp
// RMSPropOptimizer.update (nn/optimizers/rmsprop.v:70-91: f64 arithmetic on f32 state, 20 bytes).
#include "common.cuh"

namespace {

constexpr int MAXT = 56;          // tensors per launch (kernel-parameter budget)
constexpr int CHUNK = 4096;       // elements per CTA
struct Table {
  float* g[MAXT];
  float* th[MAXT];
  float* m[MAXT];
  float* v[MAXT];
  unsigned long long n[MAXT];
  int first_block[MAXT + 1];
  int nt;
};

struct AdamF32 {
  static constexpr bool kUseM = true, kUseV = true;
  float b1, b2, omb1, omb2, lr, eps;
  __device__ __forceinline__ void operator()(float g, float& th, float& m, float& v) const {
    m = __fadd_rn(__fmul_rn(b1, m), __fmul_rn(omb1, g));
    v = __fadd_rn(__fmul_rn(b2, v), __fmul_rn(__fmul_rn(omb2, g), g));
    const float denom = __fadd_rn(__fsqrt_rn(v), eps);  // == (f32)sqrt((f64)v) + eps
    th = __fsub_rn(th, __fdiv_rn(__fmul_rn(lr, m), denom));
  }
};

struct AdamWF64 {
  static constexpr bool kUseM = true, kUseV = true;
  double b1, b2, omb1, omb2, lr_t, eps, wd;
  __device__ __forceinline__ void operator()(float g, float& th, float& m, float& v) const {
    const double gd = (double)g;
    m = (float)__dadd_rn(__dmul_rn(b1, (double)m), __dmul_rn(omb1, gd));
    v = (float)__dadd_rn(__dmul_rn(b2, (double)v), __dmul_rn(__dmul_rn(omb2, gd), gd));
    const double t = (double)th, mm = (double)m, vv = (double)v;
    const double upd = __dadd_rn(__ddiv_rn(mm, __dadd_rn(__dsqrt_rn(vv), eps)), __dmul_rn(wd, t));
    th = (float)__dsub_rn(t, __dmul_rn(lr_t, upd));
  }
};

struct SgdF32 {  // no state
  static constexpr bool kUseM = false, kUseV = false;
  float lr;
  __device__ __forceinline__ void operator()(float g, float& th, float&, float&) const {
    th = __fsub_rn(th, __fmul_rn(lr, g));
  }
};

struct RmsPropF64 {  // v = running average of the squared gradient
  static constexpr bool kUseM = false, kUseV = true;
  double lr, alpha, oma, eps, wd;
  __device__ __forceinline__ void operator()(float g, float& th, float&, float& v) const {
    const double gd = (double)g;
    v = (float)__dadd_rn(__dmul_rn(alpha, (double)v), __dmul_rn(__dmul_rn(oma, gd), gd));
    const double t = (double)th, vv = (double)v;
    const double upd = __dadd_rn(__ddiv_rn(gd, __dadd_rn(__dsqrt_rn(vv), eps)), __dmul_rn(wd, t));
    th = (float)__dsub_rn(t, __dmul_rn(lr, upd));
  }
};

template <class Op>
__global__ void __launch_bounds__(256) adam_kernel(const __grid_constant__ Table tb, const Op op,
                                                   int zero_grad) {
  asm volatile("griddepcontrol.wait;" ::: "memory");  // launched early (vtlb_launch_early): the kernel in front is done
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // a small GEMM behind this kernel may start early
  int ti = 0;
  while (ti + 1 < tb.nt && (int)blockIdx.x >= tb.first_block[ti + 1]) ++ti;
  const size_t n = tb.n[ti];
  const size_t start = (size_t)(blockIdx.x - tb.first_block[ti]) * CHUNK;
  const size_t end = start + CHUNK < n ? start + CHUNK : n;
  float* __restrict__ g = tb.g[ti];
  float* __restrict__ th = tb.th[ti];
  float* __restrict__ m = tb.m[ti];
  float* __restrict__ v = tb.v[ti];
  const bool vec = ((((uintptr_t)g) | ((uintptr_t)th) | (Op::kUseM ? (uintptr_t)m : 0) |
                     (Op::kUseV ? (uintptr_t)v : 0)) & 15u) == 0;
  size_t i = start;
  if (vec) {
    const size_t vend = start + ((end - start) & ~(size_t)3);
    for (size_t j = start + threadIdx.x * 4; j < vend; j += 256 * 4) {
      float4 g4 = *reinterpret_cast<const float4*>(g + j);
      float4 t4 = *reinterpret_cast<float4*>(th + j);
      float4 m4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = m4;
      if constexpr (Op::kUseM) m4 = *reinterpret_cast<float4*>(m + j);
      if constexpr (Op::kUseV) v4 = *reinterpret_cast<float4*>(v + j);
      op(g4.x, t4.x, m4.x, v4.x);
      op(g4.y, t4.y, m4.y, v4.y);
      op(g4.z, t4.z, m4.z, v4.z);
      op(g4.w, t4.w, m4.w, v4.w);
      *reinterpret_cast<float4*>(th + j) = t4;
      if constexpr (Op::kUseM) *reinterpret_cast<float4*>(m + j) = m4;
      if constexpr (Op::kUseV) *reinterpret_cast<float4*>(v + j) = v4;
      if (zero_grad) *reinterpret_cast<float4*>(g + j) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    i = vend;
  }
  for (size_t j = i + threadIdx.x; j < end; j += 256) {
    float tt = th[j], mm = 0.0f, vv = 0.0f;
    if constexpr (Op::kUseM) mm = m[j];
    if constexpr (Op::kUseV) vv = v[j];
    op(g[j], tt, mm, vv);
    th[j] = tt;
    if constexpr (Op::kUseM) m[j] = mm;
    if constexpr (Op::kUseV) v[j] = vv;
    if (zero_grad) g[j] = 0.0f;
  }
}

template <class Op>
int run(vtlb_ctx* ctx, const char* fn, int n_tensors, const vtlb_adam_tensor* tensors, const Op& op,
        int zero_grad) {
  if (n_tensors < 0 || (n_tensors > 0 && !tensors))
    return vtlb_fail(ctx, VTLB_EINVAL, "%s: bad tensor list", fn);
  vtlb_prof_scope prof(ctx, VTLB_PHASE_OPTIMIZER);
  int i = 0;
  while (i < n_tensors) {
    Table tb;
    tb.nt = 0;
    int blocks = 0;
    while (i < n_tensors && tb.nt < MAXT) {
      const vtlb_adam_tensor& t = tensors[i++];
      if (t.n == 0) continue;
      if (!t.d_grad || !t.d_theta || (Op::kUseM && !t.d_m) || (Op::kUseV && !t.d_v))
        return vtlb_fail(ctx, VTLB_EINVAL, "%s: tensor %d has a null pointer", fn, i - 1);
      const int k = tb.nt++;
      tb.g[k] = (float*)t.d_grad;
      tb.th[k] = (float*)t.d_theta;
      tb.m[k] = (float*)t.d_m;
      tb.v[k] = (float*)t.d_v;
      tb.n[k] = t.n;
      tb.first_block[k] = blocks;
      blocks += (int)((t.n + CHUNK - 1) / CHUNK);
    }
    if (tb.nt == 0) break;
    tb.first_block[tb.nt] = blocks;
    VTLB_CUDA(ctx, vtlb_launch_early(adam_kernel<Op>, dim3(blocks), dim3(256), 0, ctx->stream, tb, op, zero_grad));
    VTLB_LAUNCHED(ctx);
  }
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_adam_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors,
                                double beta1, double beta2, double lr_t, double epsilon,
                                int zero_grad) {
  VTLB_ENTER(ctx);
  AdamF32 op{(float)beta1, (float)beta2, (float)(1.0 - beta1), (float)(1.0 - beta2), (float)lr_t,
             (float)epsilon};
  return run(ctx, "vtlb_adam_step_f32", n_tensors, tensors, op, zero_grad);
}

VTLB_API int vtlb_adamw_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors,
                                 double beta1, double beta2, double lr_t, double epsilon,
                                 double weight_decay, int zero_grad) {
  VTLB_ENTER(ctx);
  AdamWF64 op{beta1, beta2, 1.0 - beta1, 1.0 - beta2, lr_t, epsilon, weight_decay};
  return run(ctx, "vtlb_adamw_step_f32", n_tensors, tensors, op, zero_grad);
}

VTLB_API int vtlb_sgd_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors, double learning_rate,
                               int zero_grad) {
  VTLB_ENTER(ctx);
  SgdF32 op{(float)learning_rate};
  return run(ctx, "vtlb_sgd_step_f32", n_tensors, tensors, op, zero_grad);
}

VTLB_API int vtlb_rmsprop_step_f32(vtlb_ctx* ctx, int n_tensors, const vtlb_adam_tensor* tensors,
                                   double learning_rate, double alpha, double epsilon, double weight_decay,
                                   int zero_grad) {
  VTLB_ENTER(ctx);
  RmsPropF64 op{learning_rate, alpha, 1.0 - alpha, epsilon, weight_decay};
  return run(ctx, "vtlb_rmsprop_step_f32", n_tensors, tensors, op, zero_grad);
}
