// Shared device-side definitions for the Evoformer attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "evoattn.h"

namespace evo {

// Device status codes written to evoattn_fwd_params::status.
enum : int {
  DEV_OK = 0,
  DEV_TIMEOUT_TMA = 1,   // a wait for a TMA copy ran out
  DEV_TIMEOUT_MMA = 2,   // a wait for tcgen05.commit ran out
  DEV_TIMEOUT_SYNC = 3   // a wait between warps ran out
};

struct Str4 {
  long long b, h, s, r;
};
struct Str3 {
  long long a, b, c;
};

// Kernel arguments (by value).  Attention view [B,H,S,R,D]; D contiguous.
struct Args {
  int B, H, S, R, D;
  float scale;
  const void* q;
  const void* k;
  const void* v;
  void* o;          // forward: out; backward: in
  float* lse;       // [B,H,S,R]
  Str4 sq, sk, sv, so;
  const void* mask; // [B,S,R]
  int mask_kind;
  Str3 smask;       // (b,s,r)
  const float* bias;  // [B,H,R,R]; fp32, or (bias16 != 0) the q/k/v 16-bit type behind this pointer
  Str3 sbias;         // (b,h,i), in elements of the bias type
  int bias16;
  // backward only
  const void* d_o;
  void* dq;
  void* dk;
  void* dv;
  float* dbias;     // [B,H,R,R] contiguous
  float* delta;     // [B,H,S,R] (workspace)
  Str4 sdo, sdq, sdk, sdv;
  int* status;
  // gated output (optional): forward multiplies O by sigmoid(gate); backward gets dO of the gated output
  const void* gate;
  Str4 sgate;
  int delta_ready;  // backward: delta has been written already (gated path), the kernels must not recompute it
  const void* exchange;  // backward: evoattn_peer_allreduce_params of the d(pair_bias) exchange, or null
  float* dmask;     // backward (CUDA-core kernels only): gradient of an additive mask, [B,S,R] fp32
};

template <class T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }

template <class T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

// Two floats rounded to the 16-bit storage type, packed into one 32-bit word (first value low).
template <class T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

__device__ __forceinline__ long long off4(const Str4& s, int b, int h, int ss, int r) {
  return (long long)b * s.b + (long long)h * s.h + (long long)ss * s.s + (long long)r * s.r;
}

// Residue mask applied to one score.  BOOL replaces (evoformer.py:69), the others add.
template <class T>
__device__ __forceinline__ float apply_mask(float x, const void* mask, int kind, long long idx, bool& replaced) {
  replaced = false;
  if (kind == EVOATTN_MASK_BOOL) {
    if (reinterpret_cast<const unsigned char*>(mask)[idx] == 0) {
      replaced = true;
      return -FLT_MAX;
    }
    return x;
  }
  if (kind == EVOATTN_MASK_ADD_F32) return x + reinterpret_cast<const float*>(mask)[idx];
  if (kind == EVOATTN_MASK_ADD_SAME) return x + to_float<T>(reinterpret_cast<const T*>(mask)[idx]);
  return x;
}

// Residue mask of key j for batch b, MSA row s as the float the tcgen05 kernels combine with a
// score: MIN mode (boolean keep-mask or none) gives +FLT_MAX (keep) or -FLT_MAX (drop) for
// `min(score, m)`; ADD mode gives the additive value.  Keys beyond R are always dropped.
template <class T, int MIN_MODE>
__device__ __forceinline__ float mask_value(const Args& a, int b, int s, int j) {
  if (j >= a.R) return -FLT_MAX;
  if (a.mask_kind == EVOATTN_MASK_NONE) return MIN_MODE ? FLT_MAX : 0.f;
  const long long mi = (long long)b * a.smask.a + (long long)s * a.smask.b + (long long)j * a.smask.c;
  if (MIN_MODE) return reinterpret_cast<const unsigned char*>(a.mask)[mi] ? FLT_MAX : -FLT_MAX;
  if (a.mask_kind == EVOATTN_MASK_ADD_F32) return reinterpret_cast<const float*>(a.mask)[mi];
  return to_float<T>(reinterpret_cast<const T*>(a.mask)[mi]);
}

// Pair-bias element (b, h, i, j) in either storage type.
template <class T>
__device__ __forceinline__ float load_bias(const Args& a, int b, int h, int i, int j) {
  const long long idx = (long long)b * a.sbias.a + (long long)h * a.sbias.b + (long long)i * a.sbias.c + j;
  if (a.bias16) return to_float<T>(reinterpret_cast<const T*>(a.bias)[idx]);
  return a.bias[idx];
}
template <>
__device__ __forceinline__ float load_bias<float>(const Args& a, int b, int h, int i, int j) {
  return a.bias[(long long)b * a.sbias.a + (long long)h * a.sbias.b + (long long)i * a.sbias.c + j];
}

__device__ __forceinline__ float sigmoidf_fast(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace evo
