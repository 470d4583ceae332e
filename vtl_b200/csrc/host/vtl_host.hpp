// C++ mirror of the part of vtl's V API that sits above the device boundary:
// Tensor / Variable / Context (tape) / Layer / Sequential / Loss / Optimizer.
// It is the host side a V build of vtl would keep; here it is written in C++
// because no V compiler is available.  Names, argument meaning and error
// behaviour follow the reference (paths inside vlang/vtl are cited per class).
// It talks to the GPU only through the C ABI of include/vtlb.h.
//
// Difference from the reference, on purpose: tensors are device-resident
// (`value` and `grad` are device buffers, as Variable.gpu_activation hints at in
// autograd/variable.v:36), so a training step never round-trips through host
// arrays.  There is no CPU path: every operation needs a session.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../../include/vtlb.h"

namespace vtl {

struct Error : std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

// autograd_cuda.DeviceSession (autograd_cuda/device_session.v:13-36): owns the device
// context; attached to a Context through Context.device_session.
struct Session {
  vtlb_ctx* ctx = nullptr;
  int nranks = 1, rank = 0;
  // true once comm_init has run: gradients and loss values are then summed over the ranks.  A
  // communicator of a single rank takes the same code path (its collectives are copies in place).
  bool comm_on = false;
  bool owns_ctx = true;
  explicit Session(int device);
  ~Session();
  void check(int rc) const;  // throws Error with vtlb_last_error on rc != 0
  void comm_init(int nranks_, int rank_, const void* id128);
  void sync() const { check(vtlb_sync(ctx)); }
  std::shared_ptr<struct DeviceBuf> seed_one;  // a [1] tensor holding 1.0, filled once (Variable::backprop)
  // Seed of the parameter initialisers.  The reference seeds V's generator from the wall clock;
  // here layers draw their weights from (init_seed, running counter), so a model built twice
  // with the same seed starts from the same weights, on every rank of a data-parallel job.
  // Large Linear layers pass the TF32 operand planes of activations and gradients from the product
  // that writes them to the products that read them, and fold the ReLU backward into the gradient
  // product (off: every product splits its own operands, as a lone vtlb_linear_*_f32 call does).
  bool pass_planes = true;
  // Planes are handed on only by products of at least this many flops (2*M*N*K).  Measured on config 4:
  // at 65536 rows per GPU (2.2 TFLOP per product, the GPU under its power cap for seconds) the step is
  // 2 % shorter with the hand-over; at 8192 rows (0.27 TFLOP, the shard of an 8-GPU job) the epilogue's
  // extra stores cost the GEMMs more than the split passes they replace and the step is 3.6 % longer.
  // The ReLU backward is folded into the gradient product at every size (neutral to slightly faster).
  double plane_min_flops = 1.0e12;
  int plane_kinds = 3;  // which planes a large layer's product leaves: bit 0 rows, bit 1 transposed (VTL_PLANE_KINDS)
  uint64_t init_seed = 0, init_counter = 0;
  uint64_t next_init_seed() { return init_seed * 0x100000001B3ull + 0x9E3779B97F4A7C15ull * ++init_counter; }
};

struct DeviceBuf {  // one vtlb_alloc; freed (stream-ordered) when the last Tensor view dies
  Session* s;
  void* ptr;
  size_t bytes;
  bool owned;
  DeviceBuf(Session* s_, size_t bytes_);
  DeviceBuf(Session* s_, void* borrowed) : s(s_), ptr(borrowed), bytes(0), owned(false) {}  // caller's memory
  virtual ~DeviceBuf();
};

// TF32 hi/lo operand planes of a 2-D tensor T[R,C] (include/vtlb.h, vtlb_planes): "rows" planes are
// [R, ld(C)], "cols" planes [C, ld(R)] (T transposed).  Written by the GEMM that produces T and read
// by the GEMMs that consume it, so that no separate split pass runs in between.
struct PlanePair {
  std::shared_ptr<DeviceBuf> buf;  // hi followed by lo
  vtlb_planes p{nullptr, nullptr};
  static std::shared_ptr<PlanePair> make(Session* s, int rows, int kdim);
};

// vtl.Tensor[f32] (a_tensor.v): shape + storage; row-major, contiguous.  Several tensors
// may view one allocation (a layer's dW and db share a buffer so that data-parallel
// training reduces them with one collective).
class Tensor {
 public:
  Tensor() = default;
  static Tensor empty(Session* s, std::vector<int> shape);
  static Tensor zeros(Session* s, std::vector<int> shape);
  static Tensor ones(Session* s, std::vector<int> shape);
  static Tensor from_array(Session* s, const float* host, std::vector<int> shape);  // vtl.from_array
  static Tensor view(const std::shared_ptr<DeviceBuf>& buf, size_t offset_elems, std::vector<int> shape);
  void to_array(float* host) const;  // Tensor.to_array()
  Tensor reshape(std::vector<int> new_shape) const;
  size_t size() const;
  float* data() const { return buf_ ? reinterpret_cast<float*>(static_cast<char*>(buf_->ptr)) + off_ : nullptr; }
  Session* session() const { return buf_ ? buf_->s : nullptr; }
  const std::vector<int>& shape() const { return shape_; }
  const std::shared_ptr<DeviceBuf>& buffer() const { return buf_; }
  size_t offset() const { return off_; }
  bool defined() const { return (bool)buf_; }
  // Optional companions of a 2-D tensor that a tensor-core product left behind (they describe the
  // same values; copies of the Tensor share them, reshape drops them).
  std::shared_ptr<PlanePair> rows_planes, cols_planes;
  // Set on a gradient that already went through the backward of the ReLU whose output it belongs
  // to (the producing GEMM applied the mask): the ReLU gate then hands it on unchanged.
  bool relu_masked = false;

 private:
  std::shared_ptr<DeviceBuf> buf_;
  size_t off_ = 0;
  std::vector<int> shape_;
};

// nn/internal/init.v:7-70.  compute_fans keeps the reference's arithmetic as written:
// f0 = shape[0] * prod(shape[1..]), f1 = shape[1] * prod(shape[1..]) (the product runs over
// shape[1..], so shape[1] enters both), and for a 1-D shape it returns (shape[0], shape[1]) --
// reading past the end there, which this mirror reports as an error instead.
enum class FanMode { fan_avg, fan_in, fan_out };
enum class Distribution { uniform, normal };
std::pair<long long, long long> compute_fans(const std::vector<int>& shape);
// std = sqrt(scale / fan) (fan_avg: sqrt(2*scale / (f0 + f1))); uniform draws from
// [-sqrt(3)*std, +sqrt(3)*std), normal from N(0, std).  `seed` picks the stream.
Tensor variance_scaled(Session* s, const std::vector<int>& shape, double scale, FanMode mode, Distribution dist,
                       uint64_t seed);
Tensor kaiming_uniform(Session* s, const std::vector<int>& shape, uint64_t seed);
Tensor kaiming_normal(Session* s, const std::vector<int>& shape, uint64_t seed);

struct Context;
struct Gate;

// autograd.Variable (autograd/variable.v:17-57)
struct Variable {
  Tensor value, grad;
  // for the output of a ReLU: the pre-activation that ReLU cached.  A Linear gate that computes the
  // gradient w.r.t. this variable can apply the ReLU's backward in the same launch.
  Tensor relu_cache;
  Context* context = nullptr;
  bool requires_grad = true;
  bool grad_is_zero = true;  // grad holds zeros_like(value): the first accumulation may alias
  void backprop();           // autograd/variable.v:87-109
};
using VarPtr = std::shared_ptr<Variable>;

// autograd.Gate + Node + Payload (autograd/gate.v, node.v, payload.v): backward returns one
// gradient per parent, in parent order; an undefined Tensor means "no gradient".
struct Gate {
  virtual ~Gate() = default;
  virtual std::vector<Tensor> backward(const Tensor& upstream) = 0;
  // true for gates that never read their upstream gradient nor hand it on (the loss gates):
  // backprop() may then seed them with a shared tensor of ones instead of filling a fresh one
  virtual bool ignores_upstream() const { return false; }
};
struct Node {
  std::unique_ptr<Gate> gate;
  std::vector<VarPtr> parents;
  VarPtr result;  // payload.variable
  std::string name;
};

// autograd.Context (autograd/context.v:14-107): the tape.
struct Context {
  std::vector<Node> nodes;
  bool no_grad = false;
  Session* device_session = nullptr;
  explicit Context(Session* s) : device_session(s) {}
  VarPtr variable(const Tensor& value, bool requires_grad = true);  // ctx.variable(...)
  void register_node(std::string name, std::unique_ptr<Gate> gate, VarPtr result, std::vector<VarPtr> parents);
};

// Variable.matmul (autograd/variable_ops.v:82-94): C = A.B for 2-D variables, registered with
// a MatMulGate whose backward is dA = G.B^T, dB = A^T.G (autograd/gates_blas.v:41-46).
VarPtr matmul(const VarPtr& a, const VarPtr& b);

// nn/types/layer.v:6-60
struct Layer {
  virtual ~Layer() = default;
  virtual VarPtr forward(const VarPtr& input) = 0;
  virtual std::vector<VarPtr> variables() { return {}; }
  virtual std::vector<int> output_shape() const = 0;  // without the batch dimension
  virtual const char* kind() const = 0;
  // what a checkpoint records about the layer: the reference's type name and the configuration
  // map its builder registers (nn/models/sequential_info.v:40-215), in insertion order
  virtual const char* type_name() const = 0;
  virtual std::vector<std::pair<std::string, int>> config() const { return {}; }
};

// nn/layers/input.v
struct InputLayer : Layer {
  std::vector<int> shape;
  explicit InputLayer(std::vector<int> s) : shape(std::move(s)) {}
  VarPtr forward(const VarPtr& input) override { return input; }
  std::vector<int> output_shape() const override { return shape; }
  const char* kind() const override { return "input"; }
  const char* type_name() const override { return "InputLayer"; }
  std::vector<std::pair<std::string, int>> config() const override {
    std::vector<std::pair<std::string, int>> c;
    for (size_t i = 0; i < shape.size(); ++i) c.emplace_back("shape_" + std::to_string(i), shape[i]);
    return c;
  }
};

// nn/layers/linear.v:17-74 -- weights [out,in], bias [1,out]
struct LinearLayer : Layer {
  VarPtr weights, bias;
  int in_features, out_features;
  LinearLayer(Context* ctx, int in, int out);
  VarPtr forward(const VarPtr& input) override;
  // Linear followed by ReLU in one launch: returns the activated output and registers both
  // gates (the ReLU gate caches the pre-activation, as nn/layers/relu.v:34-49 does).
  VarPtr forward_with_relu(const VarPtr& input);
  std::vector<VarPtr> variables() override { return {weights, bias}; }
  std::vector<int> output_shape() const override { return {out_features}; }
  const char* kind() const override { return "linear"; }
  const char* type_name() const override { return "LinearLayer"; }
  std::vector<std::pair<std::string, int>> config() const override {
    return {{"in_features", in_features}, {"out_features", out_features}};
  }
};

// nn/layers/relu.v
struct ReLULayer : Layer {
  std::vector<int> shape;
  explicit ReLULayer(std::vector<int> s) : shape(std::move(s)) {}
  VarPtr forward(const VarPtr& input) override;
  std::vector<int> output_shape() const override { return shape; }
  const char* kind() const override { return "relu"; }
  const char* type_name() const override { return "ReLULayer"; }
};

// nn/layers/flatten.v:38-48
struct FlattenLayer : Layer {
  std::vector<int> in_shape;
  explicit FlattenLayer(std::vector<int> s) : in_shape(std::move(s)) {}
  VarPtr forward(const VarPtr& input) override;
  std::vector<int> output_shape() const override;
  const char* kind() const override { return "flatten"; }
  const char* type_name() const override { return "FlattenLayer"; }
};

// nn/layers/conv2d.v:15-105 -- weight [oc, ic, kh, kw], bias [1, oc]; groups = 1
struct Conv2DConfig {
  int pad_h = 0, pad_w = 0, stride_h = 1, stride_w = 1, dilation_h = 1, dilation_w = 1;
};
struct Conv2DLayer : Layer {
  VarPtr weight, bias;
  int in_ch, out_ch, kh, kw;
  Conv2DConfig cfg;
  std::vector<int> in_shape;  // [C, H, W]
  Conv2DLayer(Context* ctx, std::vector<int> in_shape, int out_ch, int kh, int kw, Conv2DConfig cfg);
  VarPtr forward(const VarPtr& input) override;
  VarPtr forward_with_relu(const VarPtr& input);
  std::vector<VarPtr> variables() override { return {weight, bias}; }
  std::vector<int> output_shape() const override;
  const char* kind() const override { return "conv2d"; }
  const char* type_name() const override { return "Conv2DLayer"; }
  std::vector<std::pair<std::string, int>> config() const override {
    return {{"in_channels", in_ch},        {"out_channels", out_ch},      {"kernel_h", kh},
            {"kernel_w", kw},              {"padding_h", cfg.pad_h},      {"padding_w", cfg.pad_w},
            {"stride_h", cfg.stride_h},    {"stride_w", cfg.stride_w},    {"dilation_h", cfg.dilation_h},
            {"dilation_w", cfg.dilation_w}, {"groups", 1}};
  }

 private:
  VarPtr run(const VarPtr& input, bool relu);
};

// nn/layers/maxpool.v
struct MaxPool2DLayer : Layer {
  std::vector<int> in_shape;  // [C, H, W]
  int kh, kw, ph, pw, sh, sw;
  MaxPool2DLayer(std::vector<int> in_shape, int kh, int kw, int ph, int pw, int sh, int sw);
  VarPtr forward(const VarPtr& input) override;
  std::vector<int> output_shape() const override;
  const char* kind() const override { return "maxpool2d"; }
  const char* type_name() const override { return "MaxPool2DLayer"; }
  std::vector<std::pair<std::string, int>> config() const override {
    return {{"kernel_h", kh}, {"kernel_w", kw}, {"padding_h", ph}, {"padding_w", pw}, {"stride_h", sh}, {"stride_w", sw}};
  }
};

// nn/layers/softmax.v: softmax over the last dimension; output_shape() is empty as in the reference
struct SoftmaxLayer : Layer {
  VarPtr forward(const VarPtr& input) override;
  std::vector<int> output_shape() const override { return {}; }
  const char* kind() const override { return "softmax"; }
  const char* type_name() const override { return "SoftmaxLayer"; }
};

// nn/layers/pool.v: average pooling (backward: the standard rule, see include/vtlb.h)
struct AvgPool2DLayer : Layer {
  std::vector<int> in_shape;  // [C, H, W]
  int kh, kw, ph, pw, sh, sw;
  AvgPool2DLayer(std::vector<int> in_shape, int kh, int kw, int ph, int pw, int sh, int sw);
  VarPtr forward(const VarPtr& input) override;
  std::vector<int> output_shape() const override;
  const char* kind() const override { return "avgpool2d"; }
  const char* type_name() const override { return "AvgPool2DLayer"; }
  std::vector<std::pair<std::string, int>> config() const override {
    return {{"kernel_h", kh}, {"kernel_w", kw}, {"padding_h", ph}, {"padding_w", pw}, {"stride_h", sh}, {"stride_w", sw}};
  }
};
struct GlobalAvgPool2DLayer : Layer {
  std::vector<int> in_shape;  // [C, H, W]
  explicit GlobalAvgPool2DLayer(std::vector<int> s) : in_shape(std::move(s)) {}
  VarPtr forward(const VarPtr& input) override;
  std::vector<int> output_shape() const override { return {in_shape[0], 1, 1}; }
  const char* kind() const override { return "global_avgpool2d"; }
  const char* type_name() const override { return "GlobalAvgPool2DLayer"; }
};

// nn/layers/batchnorm.v:16-108 -- gamma, beta [1, F]; running statistics are plain tensors
struct BatchNorm1DConfig {
  double eps = 1e-5, momentum = 0.1;
};
struct BatchNorm1DLayer : Layer {
  VarPtr gamma, beta;
  Tensor running_mean, running_var;
  int num_features, num_batches_tracked = 0;
  double eps, momentum;
  BatchNorm1DLayer(Context* ctx, int num_features, BatchNorm1DConfig c);
  VarPtr forward(const VarPtr& input) override;
  std::vector<VarPtr> variables() override { return {gamma, beta}; }
  std::vector<int> output_shape() const override { return {num_features}; }
  const char* kind() const override { return "batchnorm1d"; }
  const char* type_name() const override { return "BatchNorm1DLayer"; }
  std::vector<std::pair<std::string, int>> config() const override { return {{"num_features", num_features}}; }
};

// nn/types/loss.v:7-27, nn/loss/mse.v:30-41, nn/loss/softmax_cross_entropy.v
struct Loss {
  virtual ~Loss() = default;
  // `global_rows` = rows of the whole (unsharded) batch; equals output rows on one GPU
  virtual VarPtr loss(const VarPtr& output, const Tensor& target, int global_rows) = 0;
};
struct MSELoss : Loss {
  VarPtr loss(const VarPtr& output, const Tensor& target, int global_rows) override;
};
struct SoftmaxCrossEntropyLoss : Loss {
  VarPtr loss(const VarPtr& output, const Tensor& target, int global_rows) override;
};

class AdamOptimizer;

// nn/models/sequential.v:11-220 + sequential_info.v; checkpoints: nn/models/serialization.v
class Sequential {
 public:
  explicit Sequential(Session* s);
  Context* ctx() { return &ctx_; }
  void input(std::vector<int> shape);
  void linear(int output_size);
  void relu();
  void flatten();
  void conv2d(int in_channels, int out_channels, int kh, int kw, Conv2DConfig cfg);
  void maxpool2d(int kh, int kw, int ph, int pw, int sh, int sw);
  void softmax();
  void avgpool2d(int kh, int kw, int ph, int pw, int sh, int sw);
  void global_avgpool2d();
  void batchnorm1d(int num_features, BatchNorm1DConfig c = {});
  void mse_loss();
  void softmax_cross_entropy_loss();
  VarPtr forward(const VarPtr& train);                                  // sequential.v:204-215
  VarPtr loss(const VarPtr& output, const Tensor& target, int global_rows = -1);  // :218-220
  // serialization.v:102-262: weights (and, beyond the reference, the optimizer's moments when
  // `opt` is given) as JSON with base64 payloads; :266-276: (epoch, loss) of a file; :279-373:
  // weights into this already-constructed model, with the reference's checks and error texts.
  void save(const std::string& path);
  void save_checkpoint(const std::string& path, int epoch, double loss, const AdamOptimizer* opt = nullptr);
  static std::pair<int, double> load_checkpoint(const std::string& path);
  void load_weights(const std::string& path, AdamOptimizer* opt = nullptr);
  std::vector<std::unique_ptr<Layer>> layers;
  std::unique_ptr<Loss> loss_fn;
  bool fuse_relu = true;  // run Linear/Conv + ReLU pairs as one launch

 private:
  Context ctx_;
  std::vector<int> cur_shape() const;
};

// nn/optimizers/adam.v:19-145 and adamw.v:17-106.  With a data-parallel session the
// gradient all-reduces started during backprop are awaited before the update.
struct AdamConfig {
  double learning_rate = 0.001, beta1 = 0.9, beta2 = 0.999, epsilon = 1e-8, weight_decay = 0.01;
};
class AdamOptimizer {
 public:
  AdamOptimizer(AdamConfig c, bool decoupled_weight_decay);
  void build_params(const std::vector<std::unique_ptr<Layer>>& layers);
  void update();
  double learning_rate, beta1, beta2, epsilon, weight_decay, beta1_t, beta2_t;
  bool adamw;
  std::vector<VarPtr> params;
  std::vector<Tensor> first_moments, second_moments;
};

// nn/optimizers/sgd.v:9-52 and rmsprop.v:19-91
class SgdOptimizer {
 public:
  explicit SgdOptimizer(double lr) : learning_rate(lr) {}
  void build_params(const std::vector<std::unique_ptr<Layer>>& layers);
  void update();
  double learning_rate;
  std::vector<VarPtr> params;
};
struct RMSPropConfig {
  double learning_rate = 0.001, alpha = 0.99, epsilon = 1e-8, weight_decay = 0.0;
};
class RMSPropOptimizer {
 public:
  explicit RMSPropOptimizer(RMSPropConfig c)
      : learning_rate(c.learning_rate), epsilon(c.epsilon), alpha(c.alpha), weight_decay(c.weight_decay) {}
  void build_params(const std::vector<std::unique_ptr<Layer>>& layers);
  void update();
  double learning_rate, epsilon, alpha, weight_decay;
  std::vector<VarPtr> params;
  std::vector<Tensor> sq_avg;
};

// datasets.DataLoader (datasets/dataloader.v:19-331) over device-resident dataset and label
// tensors: same configuration, index order (LCG Fisher-Yates, seed + epoch), drop_last rules, len,
// reset and split; batch(i) gathers the rows of batch i on the device.
struct DataLoaderConfig {
  int batch_size = 32;
  bool shuffle = true, drop_last = true;
  uint64_t seed = 0;
};
class DataLoader {
 public:
  DataLoader(const Tensor& dataset, const Tensor& labels /* may be undefined */, DataLoaderConfig c);
  bool batch(int i, Tensor* features);                                   // false = none (:41-84)
  bool batch_with_labels(int i, Tensor* features, Tensor* labels_out);   // (:87-143)
  int len() const;                                                       // (:146-154)
  int total_samples() const { return (int)indices.size(); }
  int mini_batch_count() const { return len(); }
  void reset();                                                          // (:160-165)
  std::pair<std::unique_ptr<DataLoader>, std::unique_ptr<DataLoader>> split(double val_fraction) const;
  Tensor dataset, labels;
  int batch_size;
  bool shuffle, drop_last;
  uint64_t seed;
  std::vector<int> indices;
  int epoch = 0;

 private:
  void shuffle_indices();
  bool range(int i, int& start, int& end) const;
  void sync_indices();
  Tensor gather(const Tensor& src, int start, int end);
  std::shared_ptr<DeviceBuf> d_indices_;
  bool indices_dirty_ = true;
};

}  // namespace vtl
