// Implementation of the C++ host mirror (see vtl_host.hpp).  Every device operation is a
// call into the C ABI of include/vtlb.h; nothing here touches CUDA directly.
#include "vtl_host.hpp"

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace vtl {

// ---------------------------------------------------------------- session / storage
Session::Session(int device) {
  if (const char* e = std::getenv("VTL_PLANE_KINDS")) plane_kinds = std::atoi(e) & 3;
  int rc = vtlb_ctx_create(device, &ctx);
  if (rc != VTLB_OK) throw Error(rc, vtlb_last_error(nullptr));
}
Session::~Session() {
  seed_one.reset();  // freed through the context: before the context goes
  if (ctx && owns_ctx) vtlb_ctx_destroy(ctx);
}
void Session::check(int rc) const {
  if (rc != VTLB_OK) throw Error(rc, vtlb_last_error(ctx));
}
void Session::comm_init(int nranks_, int rank_, const void* id128) {
  check(vtlb_comm_init_rank(ctx, nranks_, rank_, id128));
  nranks = nranks_;
  rank = rank_;
  comm_on = true;
}

DeviceBuf::DeviceBuf(Session* s_, size_t bytes_) : s(s_), ptr(nullptr), bytes(bytes_), owned(true) {
  s->check(vtlb_alloc(s->ctx, bytes < 16 ? 16 : bytes, &ptr));
}
DeviceBuf::~DeviceBuf() {
  if (ptr && owned) vtlb_free(s->ctx, ptr);
}

std::shared_ptr<PlanePair> PlanePair::make(Session* s, int rows, int kdim) {
  auto pp = std::make_shared<PlanePair>();
  const size_t plane = ((size_t)rows * vtlb_plane_ld(kdim) + 63) / 64 * 64;  // keeps lo 256-byte aligned
  pp->buf = std::make_shared<DeviceBuf>(s, 2 * plane * sizeof(float));
  pp->p.hi = pp->buf->ptr;
  pp->p.lo = static_cast<float*>(pp->buf->ptr) + plane;
  return pp;
}

static size_t numel(const std::vector<int>& shape) {
  size_t n = 1;
  for (int d : shape) n *= (size_t)d;
  return n;
}

Tensor Tensor::empty(Session* s, std::vector<int> shape) {
  Tensor t;
  t.buf_ = std::make_shared<DeviceBuf>(s, numel(shape) * sizeof(float));
  t.shape_ = std::move(shape);
  return t;
}
Tensor Tensor::zeros(Session* s, std::vector<int> shape) {
  Tensor t = empty(s, std::move(shape));
  s->check(vtlb_memset0(s->ctx, t.data(), t.size() * sizeof(float)));
  return t;
}
Tensor Tensor::ones(Session* s, std::vector<int> shape) {
  Tensor t = empty(s, std::move(shape));
  s->check(vtlb_fill_f32(s->ctx, t.data(), 1.0f, t.size()));
  return t;
}
Tensor Tensor::from_array(Session* s, const float* host, std::vector<int> shape) {
  Tensor t = empty(s, std::move(shape));
  s->check(vtlb_h2d(s->ctx, t.data(), host, t.size() * sizeof(float)));
  s->check(vtlb_sync(s->ctx));  // the host array is only borrowed for the call
  return t;
}
Tensor Tensor::view(const std::shared_ptr<DeviceBuf>& buf, size_t offset_elems, std::vector<int> shape) {
  Tensor t;
  t.buf_ = buf;
  t.off_ = offset_elems;
  t.shape_ = std::move(shape);
  return t;
}
void Tensor::to_array(float* host) const {
  Session* s = session();
  s->check(vtlb_d2h(s->ctx, host, data(), size() * sizeof(float)));
}
Tensor Tensor::reshape(std::vector<int> new_shape) const {
  if (numel(new_shape) != size()) throw Error(VTLB_EINVAL, "reshape: element count differs");
  Tensor t = *this;
  if (new_shape != shape_) {  // the planes describe the 2-D layout they were written for
    t.rows_planes.reset();
    t.cols_planes.reset();
  }
  t.shape_ = std::move(new_shape);
  return t;
}
size_t Tensor::size() const { return numel(shape_); }

// ---------------------------------------------------------------- initialisers (nn/internal/init.v)
std::pair<long long, long long> compute_fans(const std::vector<int>& shape) {
  if (shape.size() < 2) throw Error(VTLB_EINVAL, "compute_fans: the shape needs at least two dimensions");
  long long product = 1;
  for (size_t i = 1; i < shape.size(); ++i) product *= shape[i];  // shape[1..], shape[1] included
  return {(long long)shape[0] * product, (long long)shape[1] * product};
}

Tensor variance_scaled(Session* s, const std::vector<int>& shape, double scale, FanMode mode, Distribution dist,
                       uint64_t seed) {
  const auto fans = compute_fans(shape);
  double sd;
  switch (mode) {
    case FanMode::fan_in: sd = std::sqrt(scale / (double)fans.first); break;
    case FanMode::fan_out: sd = std::sqrt(scale / (double)fans.second); break;
    default: sd = std::sqrt(scale * 2.0 / (double)(fans.first + fans.second)); break;
  }
  Tensor t = Tensor::empty(s, shape);
  if (dist == Distribution::uniform) {
    const float limit = (float)(std::sqrt(3.0) * sd);  // vtl.cast[T](math.sqrt(3.0) * std)
    s->check(vtlb_init_uniform_f32(s->ctx, t.data(), t.size(), -limit, limit, seed));
  } else {
    s->check(vtlb_init_normal_f32(s->ctx, t.data(), t.size(), 0.0, sd, seed));
  }
  return t;
}
Tensor kaiming_uniform(Session* s, const std::vector<int>& shape, uint64_t seed) {
  return variance_scaled(s, shape, 2.0, FanMode::fan_in, Distribution::uniform, seed);
}
Tensor kaiming_normal(Session* s, const std::vector<int>& shape, uint64_t seed) {
  return variance_scaled(s, shape, 2.0, FanMode::fan_in, Distribution::normal, seed);
}

// ---------------------------------------------------------------- autograd
VarPtr Context::variable(const Tensor& value, bool requires_grad) {
  auto v = std::make_shared<Variable>();
  v->value = value;
  v->context = this;
  v->requires_grad = requires_grad;
  // The reference allocates zeros_like(value) here (autograd/variable.v:48-57).  The zero
  // gradient is kept implicit (grad_is_zero) until something is accumulated into it.
  v->grad_is_zero = true;
  return v;
}

void Context::register_node(std::string name, std::unique_ptr<Gate> gate, VarPtr result,
                            std::vector<VarPtr> parents) {
  if (parents.empty()) throw Error(VTLB_EINVAL, "register: it is needed to specify at least one parent");
  if (no_grad) return;
  Node n;
  n.gate = std::move(gate);
  n.parents = std::move(parents);
  n.result = std::move(result);
  n.name = std::move(name);
  nodes.push_back(std::move(n));
}

// autograd/variable.v:87-109: seed with ones, drop nodes recorded after this variable, then
// walk the tape backwards; parent.grad = parent.grad.add(diff).
void Variable::backprop() {
  Session* s = context->device_session;
  auto& nodes = context->nodes;
  while (!nodes.empty() && nodes.back().result.get() != this) nodes.pop_back();
  if (value.size() == 1 && !nodes.empty() && nodes.back().gate->ignores_upstream()) {
    // a scalar loss: its gate never looks at the seed, so every step can share one tensor of ones
    // (one launch less per training step; the loss variable's grad still reads 1.0 afterwards)
    if (!s->seed_one) {
      Tensor one = Tensor::ones(s, {1});
      s->seed_one = one.buffer();
    }
    grad = Tensor::view(s->seed_one, 0, value.shape());
  } else {
    grad = Tensor::ones(s, value.shape());
  }
  grad_is_zero = false;
  while (!nodes.empty()) {
    Node node = std::move(nodes.back());
    nodes.pop_back();
    if (node.result->grad_is_zero) continue;  // nothing flowed into this result
    std::vector<Tensor> diffs = node.gate->backward(node.result->grad);
    for (size_t i = 0; i < diffs.size() && i < node.parents.size(); ++i) {
      Variable& p = *node.parents[i];
      if (!p.requires_grad || !diffs[i].defined()) continue;
      if (p.grad_is_zero) {  // zeros + diff == diff: alias instead of adding
        p.grad = diffs[i];
        p.grad_is_zero = false;
      } else {
        // Either operand may be a parameter gradient whose all-reduce is still running on the
        // communication stream (a weight used twice, or two backprops before an update): the
        // add on the compute stream has to come after it.
        if (s->comm_on) s->check(vtlb_comm_wait(s->ctx));
        s->check(vtlb_add_inplace_f32(s->ctx, p.grad.data(), diffs[i].data(), p.grad.size()));
        p.grad.rows_planes.reset();  // they described the first contribution alone
        p.grad.cols_planes.reset();
        // masked + masked stays masked; otherwise the ReLU gate masks the sum (masking twice is harmless)
        p.grad.relu_masked = p.grad.relu_masked && diffs[i].relu_masked;
      }
    }
    node.result->grad = Tensor();  // intermediate gradients are dead once consumed
    node.result->grad_is_zero = true;
  }
}

// ---------------------------------------------------------------- gates
namespace {

// Gradients of one layer's parameters live in one allocation ("bucket": dW followed by db)
// so that a data-parallel session reduces them with a single collective, started as soon
// as they are written and overlapped with the rest of backprop.
struct GradBucket {
  Tensor dW, db;
  static GradBucket make(Session* s, const std::vector<int>& wshape, const std::vector<int>& bshape) {
    const size_t nw = numel(wshape), nb = numel(bshape);
    const size_t off_b = (nw + 63) / 64 * 64;
    auto buf = std::make_shared<DeviceBuf>(s, (off_b + nb) * sizeof(float));
    if (off_b != nw)  // padding travels through the all-reduce: keep it defined
      s->check(vtlb_memset0(s->ctx, static_cast<float*>(buf->ptr) + nw, (off_b - nw) * sizeof(float)));
    GradBucket g;
    g.dW = Tensor::view(buf, 0, wshape);
    g.db = Tensor::view(buf, off_b, bshape);
    return g;
  }
  void allreduce(Session* s) const {
    if (!s->comm_on) return;
    const size_t n = db.offset() + db.size();
    s->check(vtlb_allreduce_sum_f32_async(s->ctx, dW.buffer()->ptr, n));
  }
};

// nn/gates/layers/linear.v:25-95
struct LinearGate : Gate {
  VarPtr input, weight, bias;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    const int M = g.shape()[0], N = weight->value.shape()[0], K = weight->value.shape()[1];
    Tensor dX;
    if (input->requires_grad) dX = Tensor::empty(s, {M, K});
    GradBucket b;
    const bool need_w = weight->requires_grad, need_b = bias->requires_grad;
    if (need_w || need_b) b = GradBucket::make(s, {N, K}, {1, N});
    // Large products hand their operand planes from producer to consumer (include/vtlb.h): the
    // gradient's planes come with g when the layer above produced it, the input's transposed planes
    // with the activation; dX is masked by the ReLU below this layer in the same launch and leaves
    // its own planes for the layer below.
    const bool tc = s->pass_planes && vtlb_f32_planes_worthwhile(s->ctx, M, N, K) != 0;  // tensor-core route
    const bool planes = tc && 2.0 * M * N * K >= s->plane_min_flops;
    const Tensor& xin = input->value;
    const vtlb_planes* g_rows = tc && g.rows_planes ? &g.rows_planes->p : nullptr;
    const vtlb_planes* g_cols = tc && g.cols_planes ? &g.cols_planes->p : nullptr;
    const vtlb_planes* x_cols = tc && xin.cols_planes ? &xin.cols_planes->p : nullptr;
    const float* mask = nullptr;
    // (every route of the library applies the mask: in the epilogue of the tensor-core and the small
    // CUDA-core product, as a pass of its own behind the streaming kernel for narrow layers)
    if (dX.defined() && s->pass_planes && input->relu_cache.defined() && input->relu_cache.size() == dX.size()) {
      mask = input->relu_cache.data();
      dX.relu_masked = true;
    }
    if (dX.defined() && planes && mask) {  // somebody below will multiply with this gradient
      if (s->plane_kinds & 1) dX.rows_planes = PlanePair::make(s, M, K);
      if (s->plane_kinds & 2) dX.cols_planes = PlanePair::make(s, K, M);
    }
    s->check(vtlb_linear_bwd_f32_planes(s->ctx, g.data(), xin.data(), weight->value.data(),
                                        dX.defined() ? dX.data() : nullptr, need_w ? b.dW.data() : nullptr,
                                        need_b ? b.db.data() : nullptr, M, N, K, g_rows, g_cols, x_cols, mask,
                                        dX.rows_planes ? &dX.rows_planes->p : nullptr,
                                        dX.cols_planes ? &dX.cols_planes->p : nullptr));
    if (need_w || need_b) b.allreduce(s);
    return {dX, need_w ? b.dW : Tensor(), need_b ? b.db : Tensor()};
  }
};

// nn/gates/activation/relu.v:21-25 (cache = the layer's input, i.e. the pre-activation)
struct ReLUGate : Gate {
  Tensor cache;
  std::vector<Tensor> backward(const Tensor& g) override {
    if (g.relu_masked) {  // the GEMM that produced g applied this mask already
      Tensor dx = g;
      dx.relu_masked = false;  // it is now the gradient of the pre-activation
      return {dx};
    }
    Session* s = g.session();
    Tensor dx = Tensor::empty(s, g.shape());
    s->check(vtlb_relu_bwd_f32(s->ctx, g.data(), cache.data(), dx.data(), g.size()));
    return {dx};
  }
};

struct FlattenGate : Gate {
  std::vector<int> in_shape;
  std::vector<Tensor> backward(const Tensor& g) override { return {g.reshape(in_shape)}; }
};

// nn/layers/conv2d.v:143-152
struct Conv2DGate : Gate {
  VarPtr input, weight, bias;
  int kh, kw;
  Conv2DConfig cfg;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    const auto& xs = input->value.shape();
    const int B = xs[0], C = xs[1], H = xs[2], W = xs[3], O = weight->value.shape()[0];
    Tensor dX;
    if (input->requires_grad) dX = Tensor::empty(s, xs);
    GradBucket b = GradBucket::make(s, weight->value.shape(), {1, O});
    s->check(vtlb_conv2d_bwd_f32_dilated(s->ctx, g.data(), input->value.data(), weight->value.data(),
                                         dX.defined() ? dX.data() : nullptr, b.dW.data(), b.db.data(), B, C, H, W, O,
                                         kh, kw, cfg.pad_h, cfg.pad_w, cfg.stride_h, cfg.stride_w, cfg.dilation_h,
                                         cfg.dilation_w));
    b.allreduce(s);
    return {dX, b.dW, b.db};
  }
};

struct MaxPool2DGate : Gate {
  std::shared_ptr<DeviceBuf> indices;
  std::vector<int> in_shape;
  bool tiles_2x2 = false;  // 2x2 window, stride 2, no padding, H % 2 = 0, W % 4 = 0: the direct kernel applies
  Tensor relu_cache;       // the input is a ReLU's output: its backward is fused (its cached pre-activation)
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    Tensor dx = Tensor::empty(s, in_shape);
    if (tiles_2x2) {
      s->check(vtlb_maxpool2x2_bwd_f32(s->ctx, g.data(), indices->ptr,
                                       relu_cache.defined() ? relu_cache.data() : nullptr, dx.data(), in_shape[0],
                                       in_shape[1], in_shape[2], in_shape[3]));
      dx.relu_masked = relu_cache.defined();  // the ReLU gate in front hands it through
    } else {
      s->check(vtlb_maxpool2d_bwd_f32(s->ctx, g.data(), indices->ptr, dx.data(), g.size(), dx.size()));
    }
    return {dx};
  }
};

// The loss kernels produce the gradient together with the loss value; the gate hands it
// out.  Upstream is the [1] tensor of ones that backprop() seeds (g.size == 1, g == 1).
struct LossGate : Gate {
  Tensor d_output;
  std::vector<Tensor> backward(const Tensor&) override { return {d_output}; }
  bool ignores_upstream() const override { return true; }
};

}  // namespace

// ---------------------------------------------------------------- Variable.matmul
namespace {
// autograd/gates_blas.v:25-46
struct MatMulGate : Gate {
  VarPtr a, b;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    const int M = a->value.shape()[0], K = a->value.shape()[1], N = b->value.shape()[1];
    Tensor dA, dB;
    if (a->requires_grad) {  // dA[M,K] = G[M,N] . B^T  (B is [K,N]: the B operand is "transposed")
      dA = Tensor::empty(s, {M, K});
      s->check(vtlb_gemm_f32(s->ctx, 0, 1, M, K, N, g.data(), b->value.data(), dA.data(), nullptr, 0));
    }
    if (b->requires_grad) {  // dB[K,N] = A^T . G
      dB = Tensor::empty(s, {K, N});
      s->check(vtlb_gemm_f32(s->ctx, 1, 0, K, N, M, a->value.data(), g.data(), dB.data(), nullptr, 0));
    }
    return {dA, dB};
  }
};
}  // namespace

VarPtr matmul(const VarPtr& a, const VarPtr& b) {
  Context* ctx = a->context;
  Session* s = ctx->device_session;
  const auto& as = a->value.shape();
  const auto& bs = b->value.shape();
  if (as.size() != 2 || bs.size() != 2) throw Error(VTLB_EINVAL, "matmul: both operands must be 2-D");
  if (as[1] != bs[0]) throw Error(VTLB_EINVAL, "matmul: inner dimensions differ");
  Tensor c = Tensor::empty(s, {as[0], bs[1]});
  s->check(vtlb_gemm_f32(s->ctx, 0, 0, as[0], bs[1], as[1], a->value.data(), b->value.data(), c.data(), nullptr, 0));
  VarPtr out = ctx->variable(c);
  auto g = std::make_unique<MatMulGate>();
  g->a = a;
  g->b = b;
  ctx->register_node("MatMul", std::move(g), out, {a, b});
  return out;
}

// ---------------------------------------------------------------- layers
LinearLayer::LinearLayer(Context* ctx, int in, int out) : in_features(in), out_features(out) {
  Session* s = ctx->device_session;
  // nn/layers/linear.v:25-26: Kaiming-normal weights, zero bias.  The reference's draw comes from a
  // wall-clock-seeded generator; here from the session's seed, so it can be repeated.
  weights = ctx->variable(kaiming_normal(s, {out, in}, s->next_init_seed()));
  bias = ctx->variable(Tensor::zeros(s, {1, out}));
}

static VarPtr linear_run(LinearLayer& L, const VarPtr& input, bool relu) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& xs = input->value.shape();
  if (xs.size() != 2 || xs[1] != L.in_features)
    throw Error(VTLB_EINVAL, "LinearLayer.forward: input must be [batch, in_features]");
  const int M = xs[0];
  Tensor y = Tensor::empty(s, {M, L.out_features});
  Tensor pre;
  if (relu) pre = Tensor::empty(s, {M, L.out_features});
  // While a tape is recorded, a large layer followed by its ReLU leaves the operand planes of its
  // output for the products that read it next: the next layer's forward (rows) and that layer's
  // weight gradient (transposed).
  const bool planes = s->pass_planes && relu && !ctx->no_grad &&
                      vtlb_f32_planes_worthwhile(s->ctx, M, L.out_features, L.in_features) &&
                      2.0 * M * L.out_features * L.in_features >= s->plane_min_flops;
  if (planes) {
    if (s->plane_kinds & 1) y.rows_planes = PlanePair::make(s, M, L.out_features);
    if (s->plane_kinds & 2) y.cols_planes = PlanePair::make(s, L.out_features, M);
  }
  const Tensor& xin = input->value;
  s->check(vtlb_linear_fwd_f32_planes(s->ctx, xin.data(), L.weights->value.data(), L.bias->value.data(), y.data(), M,
                                      L.out_features, L.in_features, relu ? 1 : 0, relu ? pre.data() : nullptr,
                                      s->pass_planes && xin.rows_planes ? &xin.rows_planes->p : nullptr,
                                      y.rows_planes ? &y.rows_planes->p : nullptr,
                                      y.cols_planes ? &y.cols_planes->p : nullptr));
  auto gate = std::make_unique<LinearGate>();
  gate->input = input;
  gate->weight = L.weights;
  gate->bias = L.bias;
  if (!relu) {
    VarPtr out = ctx->variable(y);
    ctx->register_node("Linear", std::move(gate), out, {input, L.weights, L.bias});
    return out;
  }
  VarPtr mid = ctx->variable(pre);
  ctx->register_node("Linear", std::move(gate), mid, {input, L.weights, L.bias});
  VarPtr out = ctx->variable(y);
  out->relu_cache = pre;
  auto rg = std::make_unique<ReLUGate>();
  rg->cache = pre;
  ctx->register_node("ReLU", std::move(rg), out, {mid});
  return out;
}
VarPtr LinearLayer::forward(const VarPtr& input) { return linear_run(*this, input, false); }
VarPtr LinearLayer::forward_with_relu(const VarPtr& input) { return linear_run(*this, input, true); }

VarPtr ReLULayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  Tensor y = Tensor::empty(s, input->value.shape());
  s->check(vtlb_relu_fwd_f32(s->ctx, input->value.data(), y.data(), y.size()));
  VarPtr out = ctx->variable(y);
  out->relu_cache = input->value;
  auto g = std::make_unique<ReLUGate>();
  g->cache = input->value;
  ctx->register_node("ReLU", std::move(g), out, {input});
  return out;
}

std::vector<int> FlattenLayer::output_shape() const { return {(int)numel(in_shape)}; }
VarPtr FlattenLayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  const int B = input->value.shape()[0];
  VarPtr out = ctx->variable(input->value.reshape({B, (int)(input->value.size() / B)}));
  auto g = std::make_unique<FlattenGate>();
  g->in_shape = input->value.shape();
  ctx->register_node("Flatten", std::move(g), out, {input});
  return out;
}

Conv2DLayer::Conv2DLayer(Context* ctx, std::vector<int> in_shape_, int out_ch_, int kh_, int kw_,
                         Conv2DConfig cfg_)
    : in_ch(in_shape_[0]), out_ch(out_ch_), kh(kh_), kw(kw_), cfg(cfg_), in_shape(std::move(in_shape_)) {
  Session* s = ctx->device_session;
  weight = ctx->variable(kaiming_normal(s, {out_ch, in_ch, kh, kw}, s->next_init_seed()));  // conv2d.v:49
  bias = ctx->variable(Tensor::zeros(s, {1, out_ch}));
}
std::vector<int> Conv2DLayer::output_shape() const {
  const int oh = (in_shape[1] + 2 * cfg.pad_h - cfg.dilation_h * (kh - 1) - 1) / cfg.stride_h + 1;
  const int ow = (in_shape[2] + 2 * cfg.pad_w - cfg.dilation_w * (kw - 1) - 1) / cfg.stride_w + 1;
  return {out_ch, oh, ow};
}
VarPtr Conv2DLayer::run(const VarPtr& input, bool relu) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& xs = input->value.shape();
  if (xs.size() != 4 || xs[1] != in_ch) throw Error(VTLB_EINVAL, "Conv2DLayer.forward: input must be [B, C, H, W]");
  const auto os = output_shape();
  const int B = xs[0];
  Tensor y = Tensor::empty(s, {B, os[0], os[1], os[2]});
  Tensor pre;
  if (relu) pre = Tensor::empty(s, y.shape());
  s->check(vtlb_conv2d_fwd_f32_dilated(s->ctx, input->value.data(), weight->value.data(), bias->value.data(),
                                       y.data(), B, in_ch, xs[2], xs[3], out_ch, kh, kw, cfg.pad_h, cfg.pad_w,
                                       cfg.stride_h, cfg.stride_w, cfg.dilation_h, cfg.dilation_w, relu ? 1 : 0,
                                       relu ? pre.data() : nullptr));
  auto gate = std::make_unique<Conv2DGate>();
  gate->input = input;
  gate->weight = weight;
  gate->bias = bias;
  gate->kh = kh;
  gate->kw = kw;
  gate->cfg = cfg;
  if (!relu) {
    VarPtr out = ctx->variable(y);
    ctx->register_node("Conv2D", std::move(gate), out, {input, weight, bias});
    return out;
  }
  VarPtr mid = ctx->variable(pre);
  ctx->register_node("Conv2D", std::move(gate), mid, {input, weight, bias});
  VarPtr out = ctx->variable(y);
  out->relu_cache = pre;
  auto rg = std::make_unique<ReLUGate>();
  rg->cache = pre;
  ctx->register_node("ReLU", std::move(rg), out, {mid});
  return out;
}
VarPtr Conv2DLayer::forward(const VarPtr& input) { return run(input, false); }
VarPtr Conv2DLayer::forward_with_relu(const VarPtr& input) { return run(input, true); }

MaxPool2DLayer::MaxPool2DLayer(std::vector<int> in_shape_, int kh_, int kw_, int ph_, int pw_, int sh_, int sw_)
    : in_shape(std::move(in_shape_)), kh(kh_), kw(kw_), ph(ph_), pw(pw_), sh(sh_), sw(sw_) {}
std::vector<int> MaxPool2DLayer::output_shape() const {
  return {in_shape[0], (in_shape[1] + 2 * ph - kh) / sh + 1, (in_shape[2] + 2 * pw - kw) / sw + 1};
}
VarPtr MaxPool2DLayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& xs = input->value.shape();
  const auto os = output_shape();
  Tensor y = Tensor::empty(s, {xs[0], os[0], os[1], os[2]});
  auto idx = std::make_shared<DeviceBuf>(s, y.size() * sizeof(int32_t));
  s->check(vtlb_maxpool2d_fwd_f32(s->ctx, input->value.data(), y.data(), idx->ptr, xs[0], xs[1], xs[2],
                                  xs[3], kh, kw, ph, pw, sh, sw));
  VarPtr out = ctx->variable(y);
  auto g = std::make_unique<MaxPool2DGate>();
  g->indices = idx;
  g->in_shape = xs;
  g->tiles_2x2 = kh == 2 && kw == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && xs[2] % 2 == 0 && xs[3] % 4 == 0 &&
                 input->value.size() < 0x7fffffffu;
  if (g->tiles_2x2 && input->relu_cache.defined() && input->relu_cache.size() == input->value.size())
    g->relu_cache = input->relu_cache;
  ctx->register_node("MaxPool2D", std::move(g), out, {input});
  return out;
}

// ---------------------------------------------------------------- losses
VarPtr MSELoss::loss(const VarPtr& output, const Tensor& target, int global_rows) {
  Context* ctx = output->context;
  Session* s = ctx->device_session;
  if (target.size() != output->value.size()) throw Error(VTLB_EINVAL, "MSELoss: target shape differs from output");
  const size_t n = output->value.size();
  const size_t rows = output->value.shape()[0];
  const size_t n_div = global_rows > 0 ? n / rows * (size_t)global_rows : n;
  Tensor l = Tensor::empty(s, {1});
  Tensor d = Tensor::empty(s, output->value.shape());
  s->check(vtlb_mse_fwd_bwd_f32(s->ctx, output->value.data(), target.data(), n, n_div, l.data(), d.data()));
  // every rank holds its rows' share of the sum over the global divisor: the loss of the whole
  // batch is their sum (awaited with the gradient all-reduces, before the value is read)
  if (s->comm_on) s->check(vtlb_allreduce_sum_f32_async(s->ctx, l.data(), 1));
  VarPtr out = ctx->variable(l);
  auto g = std::make_unique<LossGate>();
  g->d_output = d;
  ctx->register_node("MSELoss", std::move(g), out, {output});
  return out;
}

VarPtr SoftmaxCrossEntropyLoss::loss(const VarPtr& output, const Tensor& target, int global_rows) {
  Context* ctx = output->context;
  Session* s = ctx->device_session;
  const auto& xs = output->value.shape();
  if (xs.size() != 2 || target.size() != output->value.size())
    throw Error(VTLB_EINVAL, "SoftmaxCrossEntropyLoss: expects [batch, classes] logits and targets");
  Tensor l = Tensor::empty(s, {1});
  Tensor d = Tensor::empty(s, xs);
  s->check(vtlb_softmax_ce_fwd_bwd_f32(s->ctx, output->value.data(), target.data(), xs[0], xs[1],
                                       global_rows > 0 ? global_rows : xs[0], l.data(), d.data()));
  if (s->comm_on) s->check(vtlb_allreduce_sum_f32_async(s->ctx, l.data(), 1));  // as in MSELoss
  VarPtr out = ctx->variable(l);
  auto g = std::make_unique<LossGate>();
  g->d_output = d;
  ctx->register_node("SoftmaxCrossEntropyLoss", std::move(g), out, {output});
  return out;
}

// ---------------------------------------------------------------- Sequential
Sequential::Sequential(Session* s) : ctx_(s) {}

std::vector<int> Sequential::cur_shape() const {
  if (layers.empty()) throw Error(VTLB_ESTATE, "Sequential: call input(shape) first");
  return layers.back()->output_shape();
}
void Sequential::input(std::vector<int> shape) { layers.push_back(std::make_unique<InputLayer>(std::move(shape))); }
void Sequential::linear(int output_size) {
  const auto sh = cur_shape();
  if (sh.size() != 1) throw Error(VTLB_EINVAL, "Sequential.linear: previous layer must be 1-D (flatten first)");
  layers.push_back(std::make_unique<LinearLayer>(&ctx_, sh[0], output_size));
}
void Sequential::relu() { layers.push_back(std::make_unique<ReLULayer>(cur_shape())); }
void Sequential::flatten() { layers.push_back(std::make_unique<FlattenLayer>(cur_shape())); }
void Sequential::conv2d(int in_channels, int out_channels, int kh, int kw, Conv2DConfig cfg) {
  const auto sh = cur_shape();
  if (sh.size() != 3 || sh[0] != in_channels) throw Error(VTLB_EINVAL, "Sequential.conv2d: previous layer must be [C, H, W]");
  layers.push_back(std::make_unique<Conv2DLayer>(&ctx_, sh, out_channels, kh, kw, cfg));
}
void Sequential::maxpool2d(int kh, int kw, int ph, int pw, int sh_, int sw_) {
  const auto sh = cur_shape();
  if (sh.size() != 3) throw Error(VTLB_EINVAL, "Sequential.maxpool2d: previous layer must be [C, H, W]");
  layers.push_back(std::make_unique<MaxPool2DLayer>(sh, kh, kw, ph, pw, sh_, sw_));
}
void Sequential::mse_loss() { loss_fn = std::make_unique<MSELoss>(); }
void Sequential::softmax_cross_entropy_loss() { loss_fn = std::make_unique<SoftmaxCrossEntropyLoss>(); }

VarPtr Sequential::forward(const VarPtr& train) {
  VarPtr cur = train;
  for (size_t i = 0; i < layers.size(); ++i) {
    Layer* l = layers[i].get();
    const bool relu_next = fuse_relu && i + 1 < layers.size() && !std::strcmp(layers[i + 1]->kind(), "relu");
    if (relu_next && !std::strcmp(l->kind(), "linear")) {
      cur = static_cast<LinearLayer*>(l)->forward_with_relu(cur);
      ++i;
    } else if (relu_next && !std::strcmp(l->kind(), "conv2d")) {
      cur = static_cast<Conv2DLayer*>(l)->forward_with_relu(cur);
      ++i;
    } else {
      cur = l->forward(cur);
    }
  }
  return cur;
}

VarPtr Sequential::loss(const VarPtr& output, const Tensor& target, int global_rows) {
  if (!loss_fn) throw Error(VTLB_ESTATE, "Sequential.loss: no loss configured");
  return loss_fn->loss(output, target, global_rows);
}

// ---------------------------------------------------------------- optimizers
AdamOptimizer::AdamOptimizer(AdamConfig c, bool decoupled_weight_decay)
    : learning_rate(c.learning_rate), beta1(c.beta1), beta2(c.beta2), epsilon(c.epsilon),
      weight_decay(c.weight_decay), beta1_t(c.beta1), beta2_t(c.beta2), adamw(decoupled_weight_decay) {}

void AdamOptimizer::build_params(const std::vector<std::unique_ptr<Layer>>& layers) {
  for (const auto& l : layers)
    for (const VarPtr& v : l->variables()) {
      Session* s = v->context->device_session;
      params.push_back(v);
      first_moments.push_back(Tensor::zeros(s, v->value.shape()));
      second_moments.push_back(Tensor::zeros(s, v->value.shape()));
    }
}

// adam.v:87-145 / adamw.v:78-106: lr_t from the running beta powers (advanced after use),
// one fused launch for every parameter, gradients reset to zero.
void AdamOptimizer::update() {
  if (params.empty()) return;
  Session* s = params[0]->context->device_session;
  const double lr_t = learning_rate * std::sqrt(1.0 - beta2_t) / (1.0 - beta1_t);
  beta1_t *= beta1;
  beta2_t *= beta2;
  std::vector<vtlb_adam_tensor> tb;
  for (size_t i = 0; i < params.size(); ++i) {
    Variable& v = *params[i];
    if (!v.requires_grad) continue;
    if (v.grad_is_zero) {  // no gradient reached it: the reference still steps it with g = 0
      v.grad = Tensor::zeros(s, v.value.shape());
      v.grad_is_zero = false;
    }
    tb.push_back({v.grad.data(), v.value.data(), first_moments[i].data(), second_moments[i].data(),
                  v.value.size()});
  }
  if (s->comm_on) s->check(vtlb_comm_wait(s->ctx));  // gradient all-reduces started in backprop
  if (adamw)
    s->check(vtlb_adamw_step_f32(s->ctx, (int)tb.size(), tb.data(), beta1, beta2, lr_t, epsilon, weight_decay, 0));
  else
    s->check(vtlb_adam_step_f32(s->ctx, (int)tb.size(), tb.data(), beta1, beta2, lr_t, epsilon, 0));
  for (auto& p : params) {  // v.grad = zeros_like(v.value)
    p->grad = Tensor();
    p->grad_is_zero = true;
  }
}

}  // namespace vtl
