// Host mirror of the layers and optimizers that sit next to the GEMM layers in the reference's
// examples: SoftmaxLayer (nn/layers/softmax.v), AvgPool2DLayer / GlobalAvgPool2DLayer
// (nn/layers/pool.v), BatchNorm1DLayer (nn/layers/batchnorm.v), SgdOptimizer
// (nn/optimizers/sgd.v) and RMSPropOptimizer (nn/optimizers/rmsprop.v).
#include "vtl_host.hpp"

namespace vtl {
namespace {

size_t count(const std::vector<int>& shape) {
  size_t n = 1;
  for (int d : shape) n *= (size_t)d;
  return n;
}

// nn/gates/activation/softmax: deriv_softmax on the cached INPUT
struct SoftmaxGate : Gate {
  Tensor input;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    const size_t n = (size_t)input.shape().back();
    Tensor dx = Tensor::empty(s, input.shape());
    s->check(vtlb_softmax_bwd_f32(s->ctx, g.data(), input.data(), input.size() / n, n, dx.data()));
    return {dx};
  }
};

struct AvgPool2DGate : Gate {
  std::vector<int> in_shape;  // [B, C, H, W]
  int kh, kw, ph, pw, sh, sw;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    Tensor dx = Tensor::empty(s, in_shape);
    s->check(vtlb_avgpool2d_bwd_f32(s->ctx, g.data(), dx.data(), in_shape[0], in_shape[1], in_shape[2], in_shape[3],
                                    kh, kw, ph, pw, sh, sw));
    return {dx};
  }
};

struct GlobalAvgPool2DGate : Gate {
  std::vector<int> in_shape;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    Tensor dx = Tensor::empty(s, in_shape);
    s->check(vtlb_global_avgpool2d_bwd_f32(s->ctx, g.data(), dx.data(), in_shape[0], in_shape[1], in_shape[2],
                                           in_shape[3]));
    return {dx};
  }
};

// nn/layers/batchnorm.v:123-137: the gate is registered with the input as its ONLY parent, so of
// the three gradients batchnorm1d_backward computes only dx reaches the tape (gamma and beta are
// stepped with zero gradients by the optimizers, as in the reference).
struct BatchNorm1DGate : Gate {
  Tensor input, gamma, mean, var;
  double eps;
  std::vector<Tensor> backward(const Tensor& g) override {
    Session* s = g.session();
    const int B = input.shape()[0], F = input.shape()[1];
    Tensor dx = Tensor::empty(s, input.shape());
    s->check(vtlb_batchnorm1d_bwd_f32(s->ctx, g.data(), input.data(), B, F, gamma.data(), mean.data(), var.data(), eps,
                                      dx.data(), nullptr, nullptr));
    return {dx};
  }
};

}  // namespace

VarPtr SoftmaxLayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& shape = input->value.shape();
  if (shape.empty()) throw Error(VTLB_EINVAL, "SoftmaxLayer.forward: input has no dimensions");
  const size_t n = (size_t)shape.back();
  Tensor y = Tensor::empty(s, shape);
  s->check(vtlb_softmax_fwd_f32(s->ctx, input->value.data(), input->value.size() / n, n, y.data()));
  VarPtr out = ctx->variable(y);
  if (input->requires_grad) {
    auto g = std::make_unique<SoftmaxGate>();
    g->input = input->value;
    ctx->register_node("Softmax", std::move(g), out, {input});
  }
  return out;
}

AvgPool2DLayer::AvgPool2DLayer(std::vector<int> in, int kh_, int kw_, int ph_, int pw_, int sh_, int sw_)
    : in_shape(std::move(in)), kh(kh_), kw(kw_), ph(ph_), pw(pw_), sh(sh_), sw(sw_) {
  if (in_shape.size() != 3) throw Error(VTLB_EINVAL, "AvgPool2DLayer: input shape must be [C, H, W]");
}
std::vector<int> AvgPool2DLayer::output_shape() const {
  return {in_shape[0], (in_shape[1] + 2 * ph - kh) / sh + 1, (in_shape[2] + 2 * pw - kw) / sw + 1};
}
VarPtr AvgPool2DLayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& xs = input->value.shape();
  if (xs.size() != 4) throw Error(VTLB_EINVAL, "AvgPool2DLayer.forward: input must be [B, C, H, W]");
  const auto os = output_shape();
  Tensor y = Tensor::empty(s, {xs[0], os[0], os[1], os[2]});
  s->check(vtlb_avgpool2d_fwd_f32(s->ctx, input->value.data(), y.data(), xs[0], xs[1], xs[2], xs[3], kh, kw, ph, pw, sh,
                                  sw));
  VarPtr out = ctx->variable(y);
  auto g = std::make_unique<AvgPool2DGate>();
  g->in_shape = xs;
  g->kh = kh, g->kw = kw, g->ph = ph, g->pw = pw, g->sh = sh, g->sw = sw;
  ctx->register_node("AvgPool2D", std::move(g), out, {input});
  return out;
}

VarPtr GlobalAvgPool2DLayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& xs = input->value.shape();
  if (xs.size() != 4) throw Error(VTLB_EINVAL, "GlobalAvgPool2DLayer.forward: input must be [B, C, H, W]");
  Tensor y = Tensor::empty(s, {xs[0], xs[1], 1, 1});
  s->check(vtlb_global_avgpool2d_fwd_f32(s->ctx, input->value.data(), y.data(), xs[0], xs[1], xs[2], xs[3]));
  VarPtr out = ctx->variable(y);
  auto g = std::make_unique<GlobalAvgPool2DGate>();
  g->in_shape = xs;
  ctx->register_node("GlobalAvgPool2D", std::move(g), out, {input});
  return out;
}

BatchNorm1DLayer::BatchNorm1DLayer(Context* ctx, int num_features_, BatchNorm1DConfig c)
    : num_features(num_features_), eps(c.eps), momentum(c.momentum) {
  Session* s = ctx->device_session;
  gamma = ctx->variable(Tensor::ones(s, {1, num_features}));
  beta = ctx->variable(Tensor::zeros(s, {1, num_features}));
  running_mean = Tensor::zeros(s, {1, num_features});
  running_var = Tensor::ones(s, {1, num_features});
}

// nn/layers/batchnorm.v:69-108: running statistics when the input does not require a gradient,
// batch statistics (and the running update) otherwise
VarPtr BatchNorm1DLayer::forward(const VarPtr& input) {
  Context* ctx = input->context;
  Session* s = ctx->device_session;
  const auto& xs = input->value.shape();
  if (xs.size() != 2 || xs[1] != num_features)
    throw Error(VTLB_EINVAL, "BatchNorm1DLayer.forward: input must be [batch, num_features]");
  Tensor y = Tensor::empty(s, xs);
  if (!input->requires_grad) {
    s->check(vtlb_batchnorm1d_infer_f32(s->ctx, input->value.data(), xs[0], xs[1], gamma->value.data(),
                                        beta->value.data(), running_mean.data(), running_var.data(), eps, y.data()));
    return ctx->variable(y);
  }
  Tensor mean = Tensor::empty(s, {1, num_features}), var = Tensor::empty(s, {1, num_features});
  s->check(vtlb_batchnorm1d_train_f32(s->ctx, input->value.data(), xs[0], xs[1], gamma->value.data(), beta->value.data(),
                                      eps, y.data(), mean.data(), var.data(), running_mean.data(), running_var.data(),
                                      momentum));
  ++num_batches_tracked;
  VarPtr out = ctx->variable(y);
  auto g = std::make_unique<BatchNorm1DGate>();
  g->input = input->value;
  g->gamma = gamma->value;
  g->mean = mean;
  g->var = var;
  g->eps = eps;
  ctx->register_node("BatchNorm1D", std::move(g), out, {input});
  return out;
}

// ---------------------------------------------------------------- Sequential builders
void Sequential::softmax() { layers.push_back(std::make_unique<SoftmaxLayer>()); }
void Sequential::avgpool2d(int kh, int kw, int ph, int pw, int sh_, int sw_) {
  const auto sh = cur_shape();
  if (sh.size() != 3) throw Error(VTLB_EINVAL, "Sequential.avgpool2d: previous layer must be [C, H, W]");
  layers.push_back(std::make_unique<AvgPool2DLayer>(sh, kh, kw, ph, pw, sh_, sw_));
}
void Sequential::global_avgpool2d() {
  const auto sh = cur_shape();
  if (sh.size() != 3) throw Error(VTLB_EINVAL, "Sequential.global_avgpool2d: previous layer must be [C, H, W]");
  layers.push_back(std::make_unique<GlobalAvgPool2DLayer>(sh));
}
void Sequential::batchnorm1d(int num_features, BatchNorm1DConfig c) {
  layers.push_back(std::make_unique<BatchNorm1DLayer>(&ctx_, num_features, c));
}

// ---------------------------------------------------------------- optimizers
namespace {
// collects {grad, theta, state} of every parameter that takes part in the step; a parameter no
// gradient reached is stepped with zeros, as the reference's update loops do
std::vector<vtlb_adam_tensor> step_table(Session* s, std::vector<VarPtr>& params, std::vector<Tensor>* state) {
  std::vector<vtlb_adam_tensor> tb;
  for (size_t i = 0; i < params.size(); ++i) {
    Variable& v = *params[i];
    if (!v.requires_grad) continue;
    if (v.grad_is_zero) {
      v.grad = Tensor::zeros(s, v.value.shape());
      v.grad_is_zero = false;
    }
    tb.push_back({v.grad.data(), v.value.data(), nullptr, state ? (*state)[i].data() : nullptr, v.value.size()});
  }
  return tb;
}
void clear_grads(std::vector<VarPtr>& params) {
  for (auto& p : params) {
    p->grad = Tensor();
    p->grad_is_zero = true;
  }
}
}  // namespace

void SgdOptimizer::build_params(const std::vector<std::unique_ptr<Layer>>& layers) {
  for (const auto& l : layers)
    for (const VarPtr& v : l->variables()) params.push_back(v);
}
void SgdOptimizer::update() {  // nn/optimizers/sgd.v:45-52
  if (params.empty()) return;
  Session* s = params[0]->context->device_session;
  auto tb = step_table(s, params, nullptr);
  if (s->comm_on) s->check(vtlb_comm_wait(s->ctx));
  s->check(vtlb_sgd_step_f32(s->ctx, (int)tb.size(), tb.data(), learning_rate, 0));
  clear_grads(params);
}

void RMSPropOptimizer::build_params(const std::vector<std::unique_ptr<Layer>>& layers) {
  for (const auto& l : layers)
    for (const VarPtr& v : l->variables()) {
      params.push_back(v);
      sq_avg.push_back(Tensor::zeros(v->context->device_session, v->value.shape()));
    }
}
void RMSPropOptimizer::update() {  // nn/optimizers/rmsprop.v:70-91
  if (params.empty()) return;
  Session* s = params[0]->context->device_session;
  auto tb = step_table(s, params, &sq_avg);
  if (s->comm_on) s->check(vtlb_comm_wait(s->ctx));
  s->check(vtlb_rmsprop_step_f32(s->ctx, (int)tb.size(), tb.data(), learning_rate, alpha, epsilon, weight_decay, 0));
  clear_grads(params);
}

}  // namespace vtl
