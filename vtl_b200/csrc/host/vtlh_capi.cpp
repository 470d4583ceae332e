// C driver around the host mirror (see vtlh.h).
#include "vtlh.h"

#include <cstring>
#include <memory>
#include <string>

#include "vtl_host.hpp"

using namespace vtl;

struct vtlh_session {
  std::unique_ptr<Session> s;
};
struct vtlh_model {
  Session* s;
  std::unique_ptr<Sequential> seq;
  std::unique_ptr<AdamOptimizer> opt;
  std::unique_ptr<SgdOptimizer> sgd;
  std::unique_ptr<RMSPropOptimizer> rms;
  std::vector<VarPtr> params;
  VarPtr last_input;
};

static thread_local std::string g_err;
const char* vtlh_last_error(void) { return g_err.c_str(); }

template <class F>
static int guard(F&& f) {
  try {
    f();
    return VTLB_OK;
  } catch (const Error& e) {
    g_err = e.what();
    return e.code;
  } catch (const std::exception& e) {
    g_err = e.what();
    return VTLB_EINVAL;
  }
}

// a Tensor over memory the caller owns
static Tensor borrow(Session* s, const void* d_ptr, int ndim, const int* shape) {
  struct NoFree : DeviceBuf {
    NoFree(Session* s_, void* p) : DeviceBuf(s_, p) {}
  };
  std::vector<int> sh(shape, shape + ndim);
  return Tensor::view(std::make_shared<NoFree>(s, const_cast<void*>(d_ptr)), 0, sh);
}

int vtlh_session_create(int device, vtlh_session** out) {
  return guard([&] {
    auto p = new vtlh_session;
    p->s = std::make_unique<Session>(device);
    *out = p;
  });
}
int vtlh_session_destroy(vtlh_session* s) {
  delete s;
  return VTLB_OK;
}
void* vtlh_session_ctx(vtlh_session* s) { return s->s->ctx; }
int vtlh_session_comm_init(vtlh_session* s, int nranks, int rank, const void* id128) {
  return guard([&] { s->s->comm_init(nranks, rank, id128); });
}

int vtlh_session_set_seed(vtlh_session* s, unsigned long long seed) {
  s->s->init_seed = seed;
  s->s->init_counter = 0;
  return VTLB_OK;
}
int vtlh_session_set_pass_planes(vtlh_session* s, int on) {
  s->s->pass_planes = on != 0;
  return VTLB_OK;
}
int vtlh_session_set_plane_min_flops(vtlh_session* s, double flops) {
  s->s->plane_min_flops = flops;
  return VTLB_OK;
}
int vtlh_compute_fans(int ndim, const int* shape, long long* f0, long long* f1) {
  return guard([&] {
    const auto f = compute_fans(std::vector<int>(shape, shape + ndim));
    *f0 = f.first;
    *f1 = f.second;
  });
}
int vtlh_variance_scaled(vtlh_session* s, int ndim, const int* shape, double scale, int fan_mode, int distribution,
                         unsigned long long seed, float* host_out) {
  return guard([&] {
    if (fan_mode < 0 || fan_mode > 2 || distribution < 0 || distribution > 1)
      throw Error(VTLB_EINVAL, "variance_scaled: unknown fan mode or distribution");
    Tensor t = variance_scaled(s->s.get(), std::vector<int>(shape, shape + ndim), scale, (FanMode)fan_mode,
                               (Distribution)distribution, seed);
    t.to_array(host_out);
  });
}

int vtlh_model_create(vtlh_session* s, vtlh_model** out) {
  return guard([&] {
    auto m = new vtlh_model;
    m->s = s->s.get();
    m->seq = std::make_unique<Sequential>(m->s);
    *out = m;
  });
}
int vtlh_model_destroy(vtlh_model* m) {
  delete m;
  return VTLB_OK;
}
int vtlh_model_input(vtlh_model* m, int ndim, const int* shape) {
  return guard([&] { m->seq->input(std::vector<int>(shape, shape + ndim)); });
}
int vtlh_model_linear(vtlh_model* m, int n) { return guard([&] { m->seq->linear(n); }); }
int vtlh_model_relu(vtlh_model* m) { return guard([&] { m->seq->relu(); }); }
int vtlh_model_flatten(vtlh_model* m) { return guard([&] { m->seq->flatten(); }); }
int vtlh_model_conv2d(vtlh_model* m, int ic, int oc, int kh, int kw, int ph, int pw, int sh, int sw) {
  return guard([&] { m->seq->conv2d(ic, oc, kh, kw, Conv2DConfig{ph, pw, sh, sw}); });
}
int vtlh_model_conv2d_dilated(vtlh_model* m, int ic, int oc, int kh, int kw, int ph, int pw, int sh, int sw, int dh,
                              int dw) {
  return guard([&] { m->seq->conv2d(ic, oc, kh, kw, Conv2DConfig{ph, pw, sh, sw, dh, dw}); });
}
int vtlh_model_maxpool2d(vtlh_model* m, int kh, int kw, int ph, int pw, int sh, int sw) {
  return guard([&] { m->seq->maxpool2d(kh, kw, ph, pw, sh, sw); });
}
int vtlh_model_mse_loss(vtlh_model* m) { return guard([&] { m->seq->mse_loss(); }); }
int vtlh_model_softmax_cross_entropy_loss(vtlh_model* m) {
  return guard([&] { m->seq->softmax_cross_entropy_loss(); });
}
int vtlh_model_set_fuse_relu(vtlh_model* m, int on) {
  m->seq->fuse_relu = on != 0;
  return VTLB_OK;
}

static void collect_params(vtlh_model* m) {
  m->params.clear();
  for (auto& l : m->seq->layers)
    for (auto& v : l->variables()) m->params.push_back(v);
}
int vtlh_model_adam(vtlh_model* m, double lr, double b1, double b2, double eps) {
  return guard([&] {
    m->sgd.reset();
    m->rms.reset();
    m->opt = std::make_unique<AdamOptimizer>(AdamConfig{lr, b1, b2, eps, 0.0}, false);
    m->opt->build_params(m->seq->layers);
    collect_params(m);
  });
}
int vtlh_model_adamw(vtlh_model* m, double lr, double b1, double b2, double eps, double wd) {
  return guard([&] {
    m->sgd.reset();
    m->rms.reset();
    m->opt = std::make_unique<AdamOptimizer>(AdamConfig{lr, b1, b2, eps, wd}, true);
    m->opt->build_params(m->seq->layers);
    collect_params(m);
  });
}

int vtlh_model_sgd(vtlh_model* m, double lr) {
  return guard([&] {
    m->opt.reset();
    m->rms.reset();
    m->sgd = std::make_unique<SgdOptimizer>(lr);
    m->sgd->build_params(m->seq->layers);
    collect_params(m);
  });
}
int vtlh_model_rmsprop(vtlh_model* m, double lr, double alpha, double eps, double wd) {
  return guard([&] {
    m->opt.reset();
    m->sgd.reset();
    m->rms = std::make_unique<RMSPropOptimizer>(RMSPropConfig{lr, alpha, eps, wd});
    m->rms->build_params(m->seq->layers);
    collect_params(m);
  });
}
int vtlh_model_softmax(vtlh_model* m) {
  return guard([&] { m->seq->softmax(); });
}
int vtlh_model_avgpool2d(vtlh_model* m, int kh, int kw, int ph, int pw, int sh, int sw) {
  return guard([&] { m->seq->avgpool2d(kh, kw, ph, pw, sh, sw); });
}
int vtlh_model_global_avgpool2d(vtlh_model* m) {
  return guard([&] { m->seq->global_avgpool2d(); });
}
int vtlh_model_batchnorm1d(vtlh_model* m, int num_features, double eps, double momentum) {
  return guard([&] { m->seq->batchnorm1d(num_features, BatchNorm1DConfig{eps, momentum}); });
}
// running statistics of the i-th BatchNorm1D layer of the model (which = 0: mean, 1: variance)
int vtlh_model_get_running_stat(vtlh_model* m, int bn_index, int which, float* host) {
  return guard([&] {
    int k = 0;
    for (auto& l : m->seq->layers)
      if (!std::strcmp(l->kind(), "batchnorm1d") && k++ == bn_index) {
        auto* bn = static_cast<BatchNorm1DLayer*>(l.get());
        (which ? bn->running_var : bn->running_mean).to_array(host);
        return;
      }
    throw Error(VTLB_EINVAL, "no such BatchNorm1D layer");
  });
}
int vtlh_model_get_sq_avg(vtlh_model* m, int i, float* host) {
  return guard([&] {
    if (!m->rms || i < 0 || i >= (int)m->rms->sq_avg.size()) throw Error(VTLB_EINVAL, "no RMSProp optimizer or bad index");
    m->rms->sq_avg[i].to_array(host);
  });
}

int vtlh_model_num_params(vtlh_model* m) {
  if (m->params.empty()) collect_params(m);
  return (int)m->params.size();
}
static Variable& param(vtlh_model* m, int i) {
  if (m->params.empty()) collect_params(m);
  if (i < 0 || i >= (int)m->params.size()) throw Error(VTLB_EINVAL, "parameter index out of range");
  return *m->params[i];
}
int vtlh_model_param_size(vtlh_model* m, int i, size_t* n) {
  return guard([&] { *n = param(m, i).value.size(); });
}
int vtlh_model_set_param(vtlh_model* m, int i, const float* host) {
  return guard([&] {
    Variable& v = param(m, i);
    m->s->check(vtlb_h2d(m->s->ctx, v.value.data(), host, v.value.size() * sizeof(float)));
    m->s->sync();
  });
}
int vtlh_model_get_param(vtlh_model* m, int i, float* host) {
  return guard([&] { param(m, i).value.to_array(host); });
}
int vtlh_model_get_grad(vtlh_model* m, int i, float* host) {
  return guard([&] {
    Variable& v = param(m, i);
    if (v.grad_is_zero || !v.grad.defined())
      std::memset(host, 0, v.value.size() * sizeof(float));
    else
      v.grad.to_array(host);
  });
}
int vtlh_model_get_moment(vtlh_model* m, int i, int second, float* host) {
  return guard([&] {
    if (!m->opt || i < 0 || i >= (int)m->opt->params.size()) throw Error(VTLB_EINVAL, "no optimizer or bad index");
    (second ? m->opt->second_moments[i] : m->opt->first_moments[i]).to_array(host);
  });
}

int vtlh_model_forward(vtlh_model* m, const void* d_x, int ndim, const int* xshape, void* d_y) {
  return guard([&] {
    Context* ctx = m->seq->ctx();
    ctx->nodes.clear();
    const bool ng = ctx->no_grad;
    ctx->no_grad = true;
    VarPtr x = ctx->variable(borrow(m->s, d_x, ndim, xshape), false);
    VarPtr y;
    try {
      y = m->seq->forward(x);
    } catch (...) {
      ctx->no_grad = ng;
      throw;
    }
    ctx->no_grad = ng;
    if (d_y) m->s->check(vtlb_d2d(m->s->ctx, d_y, y->value.data(), y->value.size() * sizeof(float)));
  });
}

int vtlh_model_train_step(vtlh_model* m, const void* d_x, int ndim, const int* xshape, const void* d_t, int tdim,
                          const int* tshape, int global_rows, int do_update, float* h_loss) {
  return guard([&] {
    Context* ctx = m->seq->ctx();
    ctx->nodes.clear();
    // the reference's ctx.variable(x) defaults to requires_grad = true (autograd/context.v:61-65),
    // so the gradient w.r.t. the network input is computed as well
    VarPtr x = ctx->variable(borrow(m->s, d_x, ndim, xshape), true);
    m->last_input = x;
    VarPtr y = m->seq->forward(x);
    Tensor t = borrow(m->s, d_t, tdim, tshape);
    VarPtr l = m->seq->loss(y, t, global_rows > 0 ? global_rows : -1);
    l->backprop();
    if (do_update) {
      if (m->opt)
        m->opt->update();
      else if (m->sgd)
        m->sgd->update();
      else if (m->rms)
        m->rms->update();
      else
        throw Error(VTLB_ESTATE, "train_step: no optimizer configured");
    } else if (m->s->comm_on) {
      m->s->check(vtlb_comm_wait(m->s->ctx));
    }
    if (h_loss) l->value.to_array(h_loss);
  });
}

int vtlh_model_zero_grad(vtlh_model* m) {
  return guard([&] {
    if (m->params.empty()) collect_params(m);
    for (auto& p : m->params) {
      p->grad = Tensor();
      p->grad_is_zero = true;
    }
  });
}

int vtlh_matmul_mse_backprop(vtlh_session* hs, const void* d_A, int M, int K, const void* d_B, int N,
                             const void* d_T, float* h_loss, float* h_C, float* h_dA, float* h_dB) {
  return guard([&] {
    Session* s = hs->s.get();
    Context ctx(s);
    const int as[2] = {M, K}, bs[2] = {K, N}, ts[2] = {M, N};
    VarPtr a = ctx.variable(borrow(s, d_A, 2, as)), b = ctx.variable(borrow(s, d_B, 2, bs));
    VarPtr c = matmul(a, b);
    MSELoss mse;
    VarPtr l = mse.loss(c, borrow(s, d_T, 2, ts), -1);
    l->backprop();
    if (h_loss) l->value.to_array(h_loss);
    if (h_C) c->value.to_array(h_C);
    if (h_dA) a->grad.to_array(h_dA);
    if (h_dB) b->grad.to_array(h_dB);
  });
}

int vtlh_model_get_input_grad(vtlh_model* m, float* host) {
  return guard([&] {
    if (!m->last_input || m->last_input->grad_is_zero) throw Error(VTLB_ESTATE, "no input gradient available");
    m->last_input->grad.to_array(host);
  });
}

int vtlh_model_save_checkpoint(vtlh_model* m, const char* path, int epoch, double loss, int with_optimizer) {
  return guard([&] {
    if (with_optimizer && !m->opt) throw Error(VTLB_ESTATE, "save_checkpoint: the model has no optimizer");
    m->seq->save_checkpoint(path, epoch, loss, with_optimizer ? m->opt.get() : nullptr);
  });
}
int vtlh_model_load_weights(vtlh_model* m, const char* path, int with_optimizer) {
  return guard([&] {
    if (with_optimizer && !m->opt) throw Error(VTLB_ESTATE, "load_weights: the model has no optimizer");
    m->seq->load_weights(path, with_optimizer ? m->opt.get() : nullptr);
  });
}
int vtlh_load_checkpoint(const char* path, int* epoch, double* loss) {
  return guard([&] {
    const auto meta = Sequential::load_checkpoint(path);
    if (epoch) *epoch = meta.first;
    if (loss) *loss = meta.second;
  });
}

struct vtlh_loader {
  Session* s;
  std::unique_ptr<DataLoader> dl;
};

int vtlh_loader_create(vtlh_session* s, const void* d_dataset, int ndim, const int* shape, const void* d_labels,
                       int lndim, const int* lshape, int batch_size, int shuffle, int drop_last,
                       unsigned long long seed, vtlh_loader** out) {
  return guard([&] {
    Session* ss = s->s.get();
    Tensor data = borrow(ss, d_dataset, ndim, shape);
    Tensor lab = d_labels ? borrow(ss, d_labels, lndim, lshape) : Tensor();
    DataLoaderConfig c;
    c.batch_size = batch_size;
    c.shuffle = shuffle != 0;
    c.drop_last = drop_last != 0;
    c.seed = seed;
    auto p = new vtlh_loader{ss, nullptr};
    try {
      p->dl = std::make_unique<DataLoader>(data, lab, c);
    } catch (...) {
      delete p;
      throw;
    }
    *out = p;
  });
}
int vtlh_loader_destroy(vtlh_loader* l) {
  delete l;
  return VTLB_OK;
}
int vtlh_loader_len(vtlh_loader* l) { return l->dl->len(); }
int vtlh_loader_total_samples(vtlh_loader* l) { return l->dl->total_samples(); }
int vtlh_loader_reset(vtlh_loader* l) {
  return guard([&] { l->dl->reset(); });
}
int vtlh_loader_indices(vtlh_loader* l, int* out) {
  std::memcpy(out, l->dl->indices.data(), l->dl->indices.size() * sizeof(int));
  return VTLB_OK;
}
int vtlh_loader_batch(vtlh_loader* l, int i, void* d_features, void* d_labels_out, int* rows) {
  return guard([&] {
    Tensor f, lab;
    *rows = 0;
    const bool with_labels = l->dl->labels.defined() && d_labels_out;
    const bool ok = with_labels ? l->dl->batch_with_labels(i, &f, &lab) : l->dl->batch(i, &f);
    if (!ok) return;
    l->s->check(vtlb_d2d(l->s->ctx, d_features, f.data(), f.size() * sizeof(float)));
    if (with_labels) l->s->check(vtlb_d2d(l->s->ctx, d_labels_out, lab.data(), lab.size() * sizeof(float)));
    *rows = f.shape()[0];
  });
}
int vtlh_loader_split(vtlh_loader* l, double val_fraction, vtlh_loader** train, vtlh_loader** val) {
  return guard([&] {
    auto parts = l->dl->split(val_fraction);
    *train = new vtlh_loader{l->s, std::move(parts.first)};
    *val = new vtlh_loader{l->s, std::move(parts.second)};
  });
}
