/* C entry points of libvtl_host.so: a thin driver around the C++ host mirror
 * (vtl_host.hpp: Tensor / Variable / Context / Sequential / optimizers), so that the
 * Python tests and the benchmark can build a model the way a vtl program does
 * (input, linear, relu, ..., mse_loss; adam) and run training steps.  Not part of the
 * device boundary (that is include/vtlb.h); every function returns 0 or a negative
 * VTLB_E* code, vtlh_last_error() gives the message. */
#ifndef VTLH_H
#define VTLH_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct vtlh_session vtlh_session;
typedef struct vtlh_model vtlh_model;

const char* vtlh_last_error(void);
int vtlh_session_create(int device, vtlh_session** out);
int vtlh_session_destroy(vtlh_session* s);
void* vtlh_session_ctx(vtlh_session* s); /* the vtlb_ctx* the session owns */
int vtlh_session_comm_init(vtlh_session* s, int nranks, int rank, const void* id128);
/* Seed of the layers' Kaiming-normal weight draws (restarts the per-layer counter). */
int vtlh_session_set_seed(vtlh_session* s, unsigned long long seed);
/* Whether large Linear layers hand TF32 operand planes from producer to consumer and fold the ReLU
 * backward into the gradient product (default on; off = every product splits its own operands). */
int vtlh_session_set_pass_planes(vtlh_session* s, int on);
/* Smallest product (2*M*N*K flops) that hands its planes on; default 1e12 (see vtl_host.hpp). */
int vtlh_session_set_plane_min_flops(vtlh_session* s, double flops);
/* nn/internal/init.v: compute_fans (as written there) and variance_scaled into a host array;
 * fan_mode 0 = fan_avg, 1 = fan_in, 2 = fan_out; distribution 0 = uniform, 1 = normal. */
int vtlh_compute_fans(int ndim, const int* shape, long long* f0, long long* f1);
int vtlh_variance_scaled(vtlh_session* s, int ndim, const int* shape, double scale, int fan_mode, int distribution,
                         unsigned long long seed, float* host_out);

int vtlh_model_create(vtlh_session* s, vtlh_model** out);
int vtlh_model_destroy(vtlh_model* m);
int vtlh_model_input(vtlh_model* m, int ndim, const int* shape);
int vtlh_model_linear(vtlh_model* m, int output_size);
int vtlh_model_relu(vtlh_model* m);
int vtlh_model_flatten(vtlh_model* m);
int vtlh_model_conv2d(vtlh_model* m, int in_ch, int out_ch, int kh, int kw, int ph, int pw, int sh, int sw);
int vtlh_model_conv2d_dilated(vtlh_model* m, int in_ch, int out_ch, int kh, int kw, int ph, int pw, int sh, int sw,
                              int dh, int dw);
int vtlh_model_maxpool2d(vtlh_model* m, int kh, int kw, int ph, int pw, int sh, int sw);
int vtlh_model_mse_loss(vtlh_model* m);
int vtlh_model_softmax_cross_entropy_loss(vtlh_model* m);
int vtlh_model_set_fuse_relu(vtlh_model* m, int on);
int vtlh_model_adam(vtlh_model* m, double lr, double beta1, double beta2, double eps);
int vtlh_model_adamw(vtlh_model* m, double lr, double beta1, double beta2, double eps, double wd);

int vtlh_model_sgd(vtlh_model* m, double lr);
int vtlh_model_rmsprop(vtlh_model* m, double lr, double alpha, double eps, double wd);
int vtlh_model_softmax(vtlh_model* m);
int vtlh_model_avgpool2d(vtlh_model* m, int kh, int kw, int ph, int pw, int sh, int sw);
int vtlh_model_global_avgpool2d(vtlh_model* m);
int vtlh_model_batchnorm1d(vtlh_model* m, int num_features, double eps, double momentum);
int vtlh_model_get_running_stat(vtlh_model* m, int bn_index, int which, float* host); /* 0 mean, 1 variance */
int vtlh_model_get_sq_avg(vtlh_model* m, int i, float* host);

int vtlh_model_num_params(vtlh_model* m);
int vtlh_model_param_size(vtlh_model* m, int i, size_t* n);
int vtlh_model_set_param(vtlh_model* m, int i, const float* host);
int vtlh_model_get_param(vtlh_model* m, int i, float* host);
int vtlh_model_get_grad(vtlh_model* m, int i, float* host);           /* after a step with do_update == 0 */
int vtlh_model_get_moment(vtlh_model* m, int i, int second, float* host);

/* forward only; copies the output into d_y (device) when non-null */
int vtlh_model_forward(vtlh_model* m, const void* d_x, int ndim, const int* xshape, void* d_y);
/* forward, loss, backprop and (do_update != 0) optimizer update on device-resident x and
 * target; global_rows = rows of the whole batch when rows are sharded over ranks (0: local);
 * h_loss (may be null) receives the loss value, which makes the call synchronous */
int vtlh_model_train_step(vtlh_model* m, const void* d_x, int ndim, const int* xshape, const void* d_t,
                          int tdim, const int* tshape, int global_rows, int do_update, float* h_loss);
/* resets every parameter gradient to zero (what AdamOptimizer.update does after stepping) */
int vtlh_model_zero_grad(vtlh_model* m);
/* gradient of the loss w.r.t. the input of the last train_step (device -> host) */
int vtlh_model_get_input_grad(vtlh_model* m, float* host);
/* Variable.matmul on its own tape: C = A[M,K].B[K,N], loss = MSE(C, T), backprop; copies the loss,
 * C and the gradients of A and B to the host (any of the outputs may be null) */
int vtlh_matmul_mse_backprop(vtlh_session* s, const void* d_A, int M, int K, const void* d_B, int N,
                             const void* d_T, float* h_loss, float* h_C, float* h_dA, float* h_dB);
/* Checkpoints in the reference's file format (nn/models/serialization.v): save_checkpoint writes
 * the weights and, with_optimizer != 0, the optimizer's moments; load_weights restores them into a
 * model of the same architecture (with_optimizer != 0: the moments too); load_checkpoint reads
 * (epoch, loss) of a file. */
int vtlh_model_save_checkpoint(vtlh_model* m, const char* path, int epoch, double loss, int with_optimizer);
int vtlh_model_load_weights(vtlh_model* m, const char* path, int with_optimizer);
int vtlh_load_checkpoint(const char* path, int* epoch, double* loss);
/* datasets.DataLoader over device-resident tensors the caller owns (d_dataset [n, ...] f32;
 * d_labels [n, ...] f32 or null).  batch copies batch i into d_features (and d_labels_out when the
 * loader has labels and it is non-null) and returns its row count in *rows, 0 meaning "none". */
typedef struct vtlh_loader vtlh_loader;
int vtlh_loader_create(vtlh_session* s, const void* d_dataset, int ndim, const int* shape, const void* d_labels,
                       int lndim, const int* lshape, int batch_size, int shuffle, int drop_last,
                       unsigned long long seed, vtlh_loader** out);
int vtlh_loader_destroy(vtlh_loader* l);
int vtlh_loader_len(vtlh_loader* l);
int vtlh_loader_total_samples(vtlh_loader* l);
int vtlh_loader_reset(vtlh_loader* l);
int vtlh_loader_indices(vtlh_loader* l, int* out); /* total_samples() entries */
int vtlh_loader_batch(vtlh_loader* l, int i, void* d_features, void* d_labels_out, int* rows);
int vtlh_loader_split(vtlh_loader* l, double val_fraction, vtlh_loader** train, vtlh_loader** val);
#ifdef __cplusplus
}
#endif
#endif
