#include "tmap.h"

#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <mutex>

namespace evo {
namespace {

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_once;

void resolve() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

uint64_t fix_stride(long long stride_elems, int esize, uint64_t fallback_bytes, int dim) {
  // A dimension of extent 1 never advances; any legal stride will do.
  if (dim == 1) return fallback_bytes;
  return static_cast<uint64_t>(stride_elems) * esize;
}

}  // namespace

bool make_qkv_map(CUtensorMap* out, const void* base, const Str4& st, int B, int H, int S, int R, int D, int box_d,
                  int box_r) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  const uint64_t row = static_cast<uint64_t>(D) * 2;
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)R, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[4] = {fix_stride(st.r, 2, row, R), fix_stride(st.s, 2, row, S), fix_stride(st.h, 2, row, H),
                           fix_stride(st.b, 2, row, B)};
  cuuint32_t box[5] = {(cuuint32_t)box_d, (cuuint32_t)box_r, 1, 1, 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const int row_bytes = box_d * 2;
  CUtensorMapSwizzle swz = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                           : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                             : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_bias_map(CUtensorMap* out, const float* base, const Str3& st, int B, int H, int R, int box_i, int box_j) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  const uint64_t row = static_cast<uint64_t>(R) * 4;
  cuuint64_t dims[4] = {(cuuint64_t)R, (cuuint64_t)R, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {fix_stride(st.c, 4, row, R), fix_stride(st.b, 4, row, H), fix_stride(st.a, 4, row, B)};
  cuuint32_t box[4] = {(cuuint32_t)box_j, (cuuint32_t)box_i, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        box_j == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_rows_f32_map(CUtensorMap* out, const float* base, int D, int R, long long slabs, int box_d, int box_r) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)R, (cuuint64_t)slabs};
  cuuint64_t strides[2] = {(cuuint64_t)D * 4, (cuuint64_t)D * 4 * (cuuint64_t)R};
  cuuint32_t box[3] = {(cuuint32_t)box_d, (cuuint32_t)box_r, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const int row_bytes = box_d * 4;
  CUtensorMapSwizzle swz = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                           : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                             : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_rows_f32_plain_map(CUtensorMap* out, const float* base, int D, int R, long long slabs, int box_d, int box_r) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)R, (cuuint64_t)slabs};
  cuuint64_t strides[2] = {(cuuint64_t)D * 4, (cuuint64_t)D * 4 * (cuuint64_t)R};
  cuuint32_t box[3] = {(cuuint32_t)box_d, (cuuint32_t)box_r, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_bias_plain_map(CUtensorMap* out, const float* base, const Str3& st, int B, int H, int R, int box_i,
                         int box_j) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  const uint64_t row = static_cast<uint64_t>(R) * 4;
  cuuint64_t dims[4] = {(cuuint64_t)R, (cuuint64_t)R, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {fix_stride(st.c, 4, row, R), fix_stride(st.b, 4, row, H), fix_stride(st.a, 4, row, B)};
  cuuint32_t box[4] = {(cuuint32_t)box_j, (cuuint32_t)box_i, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_bias16_map(CUtensorMap* out, const void* base, const Str3& st, int B, int H, int R, int box_i, int box_j,
                     bool swizzle) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  const uint64_t row = static_cast<uint64_t>(R) * 2;
  cuuint64_t dims[4] = {(cuuint64_t)R, (cuuint64_t)R, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {fix_stride(st.c, 2, row, R), fix_stride(st.b, 2, row, H), fix_stride(st.a, 2, row, B)};
  cuuint32_t box[4] = {(cuuint32_t)box_j, (cuuint32_t)box_i, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const int row_bytes = box_j * 2;
  CUtensorMapSwizzle swz = !swizzle ? CU_TENSOR_MAP_SWIZZLE_NONE
                           : row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                           : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                             : CU_TENSOR_MAP_SWIZZLE_32B;
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_stats_map(CUtensorMap* out, const float* base, int BH, int S, int R, int box_r) {
  std::call_once(g_once, resolve);
  if (!g_encode) return false;
  cuuint64_t dims[3] = {(cuuint64_t)R, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)R * 4, (cuuint64_t)R * 4 * (cuuint64_t)S};
  cuuint32_t box[3] = {(cuuint32_t)box_r, 1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace evo
