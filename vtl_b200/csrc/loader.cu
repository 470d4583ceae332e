// Batch assembly on the device for a dataset that lives in HBM (180 GB hold every dataset of the
// reference's examples many times over): the loader's per-batch row gather
// (datasets/dataloader.v:41-143: result.set_nth(dst_base + k, dataset.get_nth(src_base + k)) for
// every index of the batch) and the one-hot expansion of integer labels
// (examples build [N, num_classes] label tensors on the host).  Both are bound by HBM.
#include "common.cuh"

namespace {

// dst[j, :] = src[idx[j], :]; one warp per row, 16-byte pieces when the rows allow it
__global__ void __launch_bounds__(256) gather_rows_kernel(const float* __restrict__ src, size_t row_elems,
                                                          const int32_t* __restrict__ idx, int n_rows,
                                                          int src_rows, float* __restrict__ dst, int vec,
                                                          uint32_t* __restrict__ bad) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int j = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; j < n_rows; j += warps) {
    const int r = idx[j];
    if (r < 0 || r >= src_rows) {  // never read outside the dataset: report and leave the row
      if (lane == 0) atomicOr(bad, 1u);
      continue;
    }
    const float* s = src + (size_t)r * row_elems;
    float* d = dst + (size_t)j * row_elems;
    if (vec) {
      const float4* s4 = reinterpret_cast<const float4*>(s);
      float4* d4 = reinterpret_cast<float4*>(d);
      for (size_t k = lane; k < row_elems / 4; k += 32) d4[k] = __ldg(s4 + k);
    } else {
      for (size_t k = lane; k < row_elems; k += 32) d[k] = __ldg(s + k);
    }
  }
}

__global__ void __launch_bounds__(256) one_hot_kernel(const int32_t* __restrict__ labels, size_t n, int classes,
                                                      float* __restrict__ out, uint32_t* __restrict__ bad) {
  const size_t total = n * (size_t)classes;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / classes;
    const int c = (int)(i - row * classes);
    const int l = labels[row];
    if ((l < 0 || l >= classes) && c == 0) atomicOr(bad, 1u);
    out[i] = l == c ? 1.0f : 0.0f;
  }
}

int loader_grid(vtlb_ctx* ctx, size_t blocks) {
  const size_t cap = (size_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

// reads the flag word the kernels above raise; blocks
int read_flag(vtlb_ctx* ctx, uint32_t* d_flag, uint32_t* out) {
  VTLB_CUDA(ctx, cudaMemcpyAsync(out, d_flag, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  VTLB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VTLB_OK;
}

}  // namespace

VTLB_API int vtlb_gather_rows_f32(vtlb_ctx* ctx, const void* d_src, int src_rows, size_t row_elems,
                                  const void* d_indices_i32, int n_rows, void* d_dst, int check) {
  VTLB_ENTER(ctx);
  if (src_rows < 0 || n_rows < 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_gather_rows_f32: negative row count");
  if (n_rows == 0 || row_elems == 0) return VTLB_OK;
  if (!d_src || !d_indices_i32 || !d_dst) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_gather_rows_f32: null pointer");
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, 256, &scr);
  if (rc) return rc;
  uint32_t* d_flag = (uint32_t*)scr;
  VTLB_CUDA(ctx, cudaMemsetAsync(d_flag, 0, sizeof(uint32_t), ctx->stream));
  const int vec = (row_elems % 4 == 0) && vtlb_aligned16(d_src) && vtlb_aligned16(d_dst);
  gather_rows_kernel<<<loader_grid(ctx, ((size_t)n_rows + 7) / 8), 256, 0, ctx->stream>>>(
      (const float*)d_src, row_elems, (const int32_t*)d_indices_i32, n_rows, src_rows, (float*)d_dst, vec, d_flag);
  VTLB_LAUNCHED(ctx);
  if (check) {
    uint32_t flag = 0;
    if ((rc = read_flag(ctx, d_flag, &flag))) return rc;
    if (flag) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_gather_rows_f32: an index is outside [0, %d)", src_rows);
  }
  return VTLB_OK;
}

VTLB_API int vtlb_one_hot_f32(vtlb_ctx* ctx, const void* d_labels_i32, size_t n, int classes, void* d_out, int check) {
  VTLB_ENTER(ctx);
  if (classes <= 0) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_one_hot_f32: classes must be positive");
  if (n == 0) return VTLB_OK;
  if (!d_labels_i32 || !d_out) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_one_hot_f32: null pointer");
  void* scr = nullptr;
  int rc = vtlb_scratch(ctx, 256, &scr);
  if (rc) return rc;
  uint32_t* d_flag = (uint32_t*)scr;
  VTLB_CUDA(ctx, cudaMemsetAsync(d_flag, 0, sizeof(uint32_t), ctx->stream));
  one_hot_kernel<<<loader_grid(ctx, (n * classes + 1023) / 1024), 256, 0, ctx->stream>>>(
      (const int32_t*)d_labels_i32, n, classes, (float*)d_out, d_flag);
  VTLB_LAUNCHED(ctx);
  if (check) {
    uint32_t flag = 0;
    if ((rc = read_flag(ctx, d_flag, &flag))) return rc;
    if (flag) return vtlb_fail(ctx, VTLB_EINVAL, "vtlb_one_hot_f32: a label is outside [0, %d)", classes);
  }
  return VTLB_OK;
}
