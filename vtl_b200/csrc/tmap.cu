// Tensor-map (TMA descriptor) construction for the GEMM operands.
#include "gemm_tc.cuh"

namespace gemm {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn g_encode = nullptr;

// 2-D row-major operand: `inner` contiguous elements per row, `outer` rows,
// rows `row_stride_bytes` apart (a multiple of 16).  Box = box_inner x box_outer
// elements with the 128-byte swizzle; out-of-range elements read as zero, which
// is what makes ragged M, N and K tails correct without any masking.
int encode_tmap_2d(vtlb_ctx* ctx, CUtensorMap* out, bool f32, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                   uint32_t box_outer) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
      return vtlb_fail(ctx, VTLB_ECUDA, "cuTensorMapEncodeTiled unavailable (%s)",
                       e == cudaSuccess ? "not found" : cudaGetErrorString(e));
    g_encode = (EncodeTiledFn)fn;
  }
  if (!vtlb_aligned16(base) || (row_stride_bytes & 15u))
    return vtlb_fail(ctx, VTLB_EINVAL,
                     "GEMM operand must be 16-byte aligned with a 16-byte-multiple row stride "
                     "(base %p, stride %llu)",
                     base, (unsigned long long)row_stride_bytes);
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                        2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return vtlb_fail(ctx, VTLB_ECUDA,
                     "cuTensorMapEncodeTiled failed (%d) for %llu x %llu, stride %llu", (int)r,
                     (unsigned long long)inner, (unsigned long long)outer,
                     (unsigned long long)row_stride_bytes);
  return VTLB_OK;
}

// 3-D byte operand: `planes` dense [rows, inner] matrices one after another; box =
// box_inner x box_rows x 1 with the 128-byte swizzle.
int encode_tmap_3d_u8(vtlb_ctx* ctx, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows,
                      uint64_t planes, uint64_t row_stride_bytes, uint64_t plane_stride_bytes,
                      uint32_t box_inner, uint32_t box_rows) {
  CUtensorMap probe;
  int rc = encode_tmap_2d(ctx, &probe, false, base, inner, rows, row_stride_bytes, box_inner, box_rows);
  if (rc) return rc;  // also resolves the driver entry point and checks alignment
  if (plane_stride_bytes & 15u)
    return vtlb_fail(ctx, VTLB_EINVAL, "GEMM operand shard stride %llu is not a multiple of 16 bytes",
                     (unsigned long long)plane_stride_bytes);
  cuuint64_t dims[3] = {inner, rows, planes};
  cuuint64_t strides[2] = {row_stride_bytes, plane_stride_bytes};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return vtlb_fail(ctx, VTLB_ECUDA, "cuTensorMapEncodeTiled (3-D) failed (%d)", (int)r);
  return VTLB_OK;
}

// 3-D f32 tensor [planes][rows][inner] without swizzle, for tiled stores of box_inner x box_rows x 1
// boxes out of a plain row-major shared-memory tile.
int encode_tmap_3d_f32_plain(vtlb_ctx* ctx, CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows,
                             uint64_t planes, uint32_t box_inner, uint32_t box_rows) {
  CUtensorMap probe;
  int rc = encode_tmap_2d(ctx, &probe, true, base, inner, rows, inner * 4, 32, 1);
  if (rc) return rc;  // resolves the driver entry point and checks alignment
  cuuint64_t dims[3] = {inner, rows, planes};
  cuuint64_t strides[2] = {inner * 4, inner * rows * 4};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return vtlb_fail(ctx, VTLB_ECUDA, "cuTensorMapEncodeTiled (3-D f32) failed (%d)", (int)r);
  return VTLB_OK;
}

}  // namespace gemm
