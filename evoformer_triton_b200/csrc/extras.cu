// Small device passes around the attention kernels: the backward half of the gated output, and the
// conversion of a pair bias (and its gradient) between the layout a linear layer emits,
// [B, R, R, H], and the [B, H, R, R] the kernels (and dsevoformer-triton/evoformer.py:638,652) use.
// None of this exists in the reference: its op ends at O and takes the bias heads-first.
#include <string.h>

#include "common.cuh"
#include "launch.h"

namespace evo {
namespace {

// Gated output Og = sigmoid(gate) * O.  With G = dOg (gradient of the gated output):
//   dO    = G * sigmoid(gate)                      (what the attention backward needs)
//   delta = sum_d dO * O = sum_d G * Og            (so the un-gated O is never needed)
//   dgate = G * O * sigmoid'(gate) = G * Og * (1 - sigmoid(gate))
// One warp per (b,h,s,i) row.  dO is written contiguously ([rows][D]) into scratch.
template <class T>
__global__ void __launch_bounds__(256) gate_backward_kernel(Args a, T* __restrict__ d_o_eff, void* __restrict__ dgate,
                                                            Str4 sdgate) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + warp;
  const long long rows = (long long)a.B * a.H * a.S * a.R;
  if (row >= rows) return;
  const int i = (int)(row % a.R);
  long long sl = row / a.R;
  const int s = (int)(sl % a.S); sl /= a.S;
  const int h = (int)(sl % a.H);
  const int b = (int)(sl / a.H);
  const T* og = reinterpret_cast<const T*>(a.o) + off4(a.so, b, h, s, i);
  const T* g = reinterpret_cast<const T*>(a.d_o) + off4(a.sdo, b, h, s, i);
  const T* gt = reinterpret_cast<const T*>(a.gate) + off4(a.sgate, b, h, s, i);
  T* dg = reinterpret_cast<T*>(dgate) + off4(sdgate, b, h, s, i);
  float acc = 0.f;
  for (int d = lane; d < a.D; d += 32) {
    const float G = to_float<T>(g[d]), O = to_float<T>(og[d]);
    const float sg = sigmoidf_fast(to_float<T>(gt[d]));
    acc += G * O;
    d_o_eff[row * a.D + d] = from_float<T>(G * sg);
    dg[d] = from_float<T>(G * O * (1.f - sg));
  }
  acc = warp_sum(acc);
  if (lane == 0) a.delta[row] = acc;
}

// [B,R,R,H] -> [B,H,R,R]: a block takes 128 keys of one (b, i) row: 128*H contiguous elements in,
// H runs of 128 contiguous elements out.
template <class E>
__global__ void __launch_bounds__(256) heads_first_kernel(const E* __restrict__ src, E* __restrict__ dst, int H, int R) {
  extern __shared__ unsigned char sm_raw[];
  E* sm = reinterpret_cast<E*>(sm_raw);
  const int j0 = blockIdx.x * 128, i = blockIdx.y, b = blockIdx.z;
  const int nj = min(128, R - j0);
  const E* in = src + (((long long)b * R + i) * R + j0) * H;
  for (int e = threadIdx.x; e < nj * H; e += 256) sm[e] = in[e];
  __syncthreads();
  for (int e = threadIdx.x; e < nj * H; e += 256) {
    const int h = e / nj, j = e - h * nj;
    dst[(((long long)b * H + h) * R + i) * R + j0 + j] = sm[j * H + h];
  }
}

// fp32 [B,H,R,R] -> [B,R,R,H] in type E (the one cast of the gradient happens here).
template <class E>
__global__ void __launch_bounds__(256) heads_last_kernel(const float* __restrict__ src, E* __restrict__ dst, int H, int R) {
  extern __shared__ unsigned char sm_raw[];
  float* sm = reinterpret_cast<float*>(sm_raw);
  const int j0 = blockIdx.x * 128, i = blockIdx.y, b = blockIdx.z;
  const int nj = min(128, R - j0);
  for (int e = threadIdx.x; e < nj * H; e += 256) {
    const int h = e / nj, j = e - h * nj;
    sm[j * H + h] = src[(((long long)b * H + h) * R + i) * R + j0 + j];
  }
  __syncthreads();
  E* out = dst + (((long long)b * R + i) * R + j0) * H;
  for (int e = threadIdx.x; e < nj * H; e += 256) out[e] = from_float<E>(sm[e]);
}

}  // namespace

size_t gate_backward_scratch_bytes(int dtype, const Args& a) {
  const size_t es = dtype == EVOATTN_FP32 ? 4 : 2;
  return ((size_t)a.B * a.H * a.S * a.R * a.D * es + 255) / 256 * 256;
}

// Runs the gate pass and redirects `a` to the effective dO; `scratch` holds gate_backward_scratch_bytes().
int launch_gate_backward(int dtype, Args* a, void* scratch, void* dgate, const Str4& sdgate, cudaStream_t st, int* launches) {
  const long long rows = (long long)a->B * a->H * a->S * a->R;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  switch (dtype) {
    case EVOATTN_BF16: gate_backward_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(*a, reinterpret_cast<__nv_bfloat16*>(scratch), dgate, sdgate); break;
    case EVOATTN_FP16: gate_backward_kernel<__half><<<grid, 256, 0, st>>>(*a, reinterpret_cast<__half*>(scratch), dgate, sdgate); break;
    default: gate_backward_kernel<float><<<grid, 256, 0, st>>>(*a, reinterpret_cast<float*>(scratch), dgate, sdgate); break;
  }
  *launches += 1;
  a->d_o = scratch;
  a->sdo = Str4{(long long)a->H * a->S * a->R * a->D, (long long)a->S * a->R * a->D, (long long)a->R * a->D, (long long)a->D};
  a->delta_ready = 1;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

}  // namespace evo

extern "C" {

int evoattn_bias_to_heads_first(const void* src, void* dst, int dtype, int B, int H, int R, void* cuda_stream) {
  if (!src || !dst) return EVOATTN_ERR_NULL;
  if (B <= 0 || H <= 0 || R <= 0 || H > 96 || B > 65535 || R > 65535) return EVOATTN_ERR_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  dim3 grid((R + 127) / 128, R, B);
  if (dtype == EVOATTN_FP32)
    evo::heads_first_kernel<float><<<grid, 256, (size_t)128 * H * 4, st>>>(static_cast<const float*>(src), static_cast<float*>(dst), H, R);
  else if (dtype == EVOATTN_BF16 || dtype == EVOATTN_FP16)
    evo::heads_first_kernel<uint16_t><<<grid, 256, (size_t)128 * H * 2, st>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), H, R);
  else
    return EVOATTN_ERR_DTYPE;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

int evoattn_dbias_to_heads_last(const float* src, void* dst, int dtype, int B, int H, int R, void* cuda_stream) {
  if (!src || !dst) return EVOATTN_ERR_NULL;
  if (B <= 0 || H <= 0 || R <= 0 || H > 96 || B > 65535 || R > 65535) return EVOATTN_ERR_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  dim3 grid((R + 127) / 128, R, B);
  const size_t smem = (size_t)128 * H * 4;
  if (dtype == EVOATTN_FP32) evo::heads_last_kernel<float><<<grid, 256, smem, st>>>(src, static_cast<float*>(dst), H, R);
  else if (dtype == EVOATTN_BF16) evo::heads_last_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(src, static_cast<__nv_bfloat16*>(dst), H, R);
  else if (dtype == EVOATTN_FP16) evo::heads_last_kernel<__half><<<grid, 256, smem, st>>>(src, static_cast<__half*>(dst), H, R);
  else return EVOATTN_ERR_DTYPE;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

}  // extern "C"
