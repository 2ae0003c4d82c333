// CUDA-core Evoformer attention kernels: any dtype (fp32 included), any D <= 128, any R.
//
// These serve fp32 inputs (tensor cores would lose bits there) and every shape the
// tcgen05 kernels do not cover.  They are written for clarity and determinism, not
// speed: one warp owns one score row, every sum has a fixed order, and the pair-bias
// gradient is produced by one owner per element instead of the reference's fp32
// atomics (dsevoformer-triton/evoformer.py:458).
//
// Math (evoformer.py:68-89 forward, :450-462 and :594-614 backward), fp32 throughout:
//   x_ij = scale * <q_i,k_j> + bias_ij ;  mask ;  P = softmax_j(x) ;  O = P V
//   delta_i = <dO_i,O_i> ; dP_ij = <dO_i,v_j> ; dS = P (dP - delta)
//   dV_j = sum_i P_ij dO_i ; dQ_i = scale sum_j dS_ij k_j ; dK_j = scale sum_i dS_ij q_i
//   dBias_ij = sum_s dS_ij
#include "common.cuh"
#include "launch.h"

namespace evo {

constexpr int GW = 8;   // warps per CTA = score rows per CTA
constexpr int GT = 32;  // rows staged in shared memory per step (one per lane)

struct Slab {
  int b, h, s;
};
__device__ __forceinline__ Slab slab_of(int idx, const Args& a) {
  Slab r;
  r.s = idx % a.S;
  r.h = (idx / a.S) % a.H;
  r.b = idx / (a.S * a.H);
  return r;
}

template <class T>
__device__ __forceinline__ void stage_rows(float* dst, int DP, const T* base, const Str4& st, int b, int h, int s,
                                           int r0, int R, int D) {
  for (int idx = threadIdx.x; idx < GT * D; idx += blockDim.x) {
    int rr = idx / D, d = idx - rr * D;
    int r = r0 + rr;
    dst[rr * DP + d] = (r < R) ? to_float<T>(base[off4(st, b, h, s, r) + d]) : 0.f;
  }
}

// Score of (i, j) before the softmax, with mask applied.  `replaced` tells the caller
// that the score is a constant (boolean mask dropped the key).
template <class T>
__device__ __forceinline__ float score(const Args& a, int b, int h, int s, int i, int j, float dot, bool& replaced) {
  float x = dot * a.scale;
  if (a.bias) x += load_bias<T>(a, b, h, i, j);
  replaced = false;
  if (a.mask_kind != EVOATTN_MASK_NONE)
    x = apply_mask<T>(x, a.mask, a.mask_kind, (long long)b * a.smask.a + (long long)s * a.smask.b + (long long)j * a.smask.c,
                      replaced);
  return x;
}

// P_ij from a stored log-sum-exp.  A row whose keys were all dropped has lse == -FLT_MAX
// exactly (the log of the row sum is absorbed); its softmax is uniform over the R keys.
__device__ __forceinline__ float prob_from_lse(float x, float lse, int R) {
  if (lse == -FLT_MAX) return 1.f / (float)R;
  return expf(x - lse);
}

template <class T>
__global__ void __launch_bounds__(GW * 32) generic_fwd_kernel(Args a) {
  extern __shared__ float sm[];
  const int D = a.D, DP = D + 1;
  float* Ks = sm;
  float* Vs = Ks + GT * DP;
  float* Qs = Vs + GT * DP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Slab sl = slab_of(blockIdx.x, a);
  const int i = blockIdx.y * GW + warp;
  const bool row_ok = i < a.R;
  const int ic = row_ok ? i : 0;
  const T* q = reinterpret_cast<const T*>(a.q) + off4(a.sq, sl.b, sl.h, sl.s, ic);
  for (int d = lane; d < D; d += 32) Qs[warp * DP + d] = to_float<T>(q[d]);
  float m = -INFINITY, l = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j0 = 0; j0 < a.R; j0 += GT) {
    __syncthreads();
    stage_rows<T>(Ks, DP, reinterpret_cast<const T*>(a.k), a.sk, sl.b, sl.h, sl.s, j0, a.R, D);
    stage_rows<T>(Vs, DP, reinterpret_cast<const T*>(a.v), a.sv, sl.b, sl.h, sl.s, j0, a.R, D);
    __syncthreads();
    const int j = j0 + lane;
    float x = -INFINITY;
    if (j < a.R) {
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot += Qs[warp * DP + d] * Ks[lane * DP + d];
      bool rep;
      x = score<T>(a, sl.b, sl.h, sl.s, ic, j, dot, rep);
    }
    const float mn = fmaxf(m, warp_max(x));
    const float alpha = expf(m - mn);
    const float p = (j < a.R) ? expf(x - mn) : 0.f;
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[t] *= alpha;
    for (int jj = 0; jj < GT; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int d = lane + 32 * t;
        if (d < D) acc[t] += pj * Vs[jj * DP + d];
      }
    }
    m = mn;
  }
  if (row_ok) {
    T* o = reinterpret_cast<T*>(a.o) + off4(a.so, sl.b, sl.h, sl.s, i);
    const T* gate = a.gate ? reinterpret_cast<const T*>(a.gate) + off4(a.sgate, sl.b, sl.h, sl.s, i) : nullptr;
    const float inv = 1.f / l;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int d = lane + 32 * t;
      if (d < D) o[d] = from_float<T>(acc[t] * inv * (gate ? sigmoidf_fast(to_float<T>(gate[d])) : 1.f));
    }
    if (lane == 0) a.lse[((long long)blockIdx.x) * a.R + i] = m + logf(l);
  }
}

// delta[b,h,s,i] = <dO_i, O_i>   (evoformer.py:299-326)
template <class T>
__global__ void __launch_bounds__(GW * 32) generic_delta_kernel(Args a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * GW + warp;
  const long long rows = (long long)a.B * a.H * a.S * a.R;
  if (row >= rows) return;
  const int i = (int)(row % a.R);
  const Slab sl = slab_of((int)(row / a.R), a);
  const T* o = reinterpret_cast<const T*>(a.o) + off4(a.so, sl.b, sl.h, sl.s, i);
  const T* g = reinterpret_cast<const T*>(a.d_o) + off4(a.sdo, sl.b, sl.h, sl.s, i);
  float acc = 0.f;
  for (int d = lane; d < a.D; d += 32) acc += to_float<T>(o[d]) * to_float<T>(g[d]);
  acc = warp_sum(acc);
  if (lane == 0) a.delta[row] = acc;
}

// dQ: one warp per query row, lanes over keys.
template <class T>
__global__ void __launch_bounds__(GW * 32) generic_dq_kernel(Args a) {
  extern __shared__ float sm[];
  const int D = a.D, DP = D + 1;
  float* Ks = sm;
  float* Vs = Ks + GT * DP;
  float* Qs = Vs + GT * DP;
  float* Gs = Qs + GW * DP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Slab sl = slab_of(blockIdx.x, a);
  const int i = blockIdx.y * GW + warp;
  const bool row_ok = i < a.R;
  const int ic = row_ok ? i : 0;
  const T* q = reinterpret_cast<const T*>(a.q) + off4(a.sq, sl.b, sl.h, sl.s, ic);
  const T* g = reinterpret_cast<const T*>(a.d_o) + off4(a.sdo, sl.b, sl.h, sl.s, ic);
  for (int d = lane; d < D; d += 32) {
    Qs[warp * DP + d] = to_float<T>(q[d]);
    Gs[warp * DP + d] = to_float<T>(g[d]);
  }
  const float lse = a.lse[(long long)blockIdx.x * a.R + ic];
  const float delta = a.delta[(long long)blockIdx.x * a.R + ic];
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int j0 = 0; j0 < a.R; j0 += GT) {
    __syncthreads();
    stage_rows<T>(Ks, DP, reinterpret_cast<const T*>(a.k), a.sk, sl.b, sl.h, sl.s, j0, a.R, D);
    stage_rows<T>(Vs, DP, reinterpret_cast<const T*>(a.v), a.sv, sl.b, sl.h, sl.s, j0, a.R, D);
    __syncthreads();
    const int j = j0 + lane;
    float ds = 0.f;
    if (j < a.R) {
      float dot = 0.f, dp = 0.f;
      for (int d = 0; d < D; ++d) {
        dot += Qs[warp * DP + d] * Ks[lane * DP + d];
        dp += Gs[warp * DP + d] * Vs[lane * DP + d];
      }
      bool rep;
      const float x = score<T>(a, sl.b, sl.h, sl.s, ic, j, dot, rep);
      const float p = prob_from_lse(x, lse, a.R);
      ds = rep ? 0.f : p * (dp - delta);
    }
    for (int jj = 0; jj < GT; ++jj) {
      const float dj = __shfl_sync(0xffffffffu, ds, jj);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int d = lane + 32 * t;
        if (d < D) acc[t] += dj * Ks[jj * DP + d];
      }
    }
  }
  if (row_ok) {
    T* o = reinterpret_cast<T*>(a.dq) + off4(a.sdq, sl.b, sl.h, sl.s, i);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int d = lane + 32 * t;
      if (d < D) o[d] = from_float<T>(acc[t] * a.scale);
    }
  }
}

// dK, dV: one warp per key row, lanes over queries.
template <class T>
__global__ void __launch_bounds__(GW * 32) generic_dkdv_kernel(Args a) {
  extern __shared__ float sm[];
  const int D = a.D, DP = D + 1;
  float* Qs = sm;                  // [GT][DP]
  float* Gs = Qs + GT * DP;        // [GT][DP]
  float* Kw = Gs + GT * DP;        // [GW][DP]
  float* Vw = Kw + GW * DP;        // [GW][DP]
  float* Ls = Vw + GW * DP;        // [GT] lse
  float* Ds = Ls + GT;             // [GT] delta
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Slab sl = slab_of(blockIdx.x, a);
  const int j = blockIdx.y * GW + warp;
  const bool row_ok = j < a.R;
  const int jc = row_ok ? j : 0;
  const T* k = reinterpret_cast<const T*>(a.k) + off4(a.sk, sl.b, sl.h, sl.s, jc);
  const T* v = reinterpret_cast<const T*>(a.v) + off4(a.sv, sl.b, sl.h, sl.s, jc);
  for (int d = lane; d < D; d += 32) {
    Kw[warp * DP + d] = to_float<T>(k[d]);
    Vw[warp * DP + d] = to_float<T>(v[d]);
  }
  float accK[4] = {0.f, 0.f, 0.f, 0.f}, accV[4] = {0.f, 0.f, 0.f, 0.f};
  float dmask_acc = 0.f;  // this lane's share of sum_i dS_ij (gradient of an additive mask)
  for (int i0 = 0; i0 < a.R; i0 += GT) {
    __syncthreads();
    stage_rows<T>(Qs, DP, reinterpret_cast<const T*>(a.q), a.sq, sl.b, sl.h, sl.s, i0, a.R, D);
    stage_rows<T>(Gs, DP, reinterpret_cast<const T*>(a.d_o), a.sdo, sl.b, sl.h, sl.s, i0, a.R, D);
    if (threadIdx.x < GT) {
      const int i = i0 + threadIdx.x;
      Ls[threadIdx.x] = (i < a.R) ? a.lse[(long long)blockIdx.x * a.R + i] : 0.f;
      Ds[threadIdx.x] = (i < a.R) ? a.delta[(long long)blockIdx.x * a.R + i] : 0.f;
    }
    __syncthreads();
    const int i = i0 + lane;
    float p = 0.f, ds = 0.f;
    if (i < a.R) {
      float dot = 0.f, dp = 0.f;
      for (int d = 0; d < D; ++d) {
        dot += Qs[lane * DP + d] * Kw[warp * DP + d];
        dp += Gs[lane * DP + d] * Vw[warp * DP + d];
      }
      bool rep;
      const float x = score<T>(a, sl.b, sl.h, sl.s, i, jc, dot, rep);
      p = prob_from_lse(x, Ls[lane], a.R);
      ds = rep ? 0.f : p * (dp - Ds[lane]);
      dmask_acc += ds;
    }
    for (int ii = 0; ii < GT; ++ii) {
      const float pi = __shfl_sync(0xffffffffu, p, ii);
      const float di = __shfl_sync(0xffffffffu, ds, ii);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int d = lane + 32 * t;
        if (d < D) {
          accV[t] += pi * Gs[ii * DP + d];
          accK[t] += di * Qs[ii * DP + d];
        }
      }
    }
  }
  if (a.dmask != nullptr) {  // one addition per (b,h,s,j): the sum over heads
    const float tot = warp_sum(dmask_acc);
    if (row_ok && lane == 0) atomicAdd(a.dmask + ((long long)sl.b * a.S + sl.s) * a.R + j, tot);
  }
  if (row_ok) {
    T* ok = reinterpret_cast<T*>(a.dk) + off4(a.sdk, sl.b, sl.h, sl.s, j);
    T* ov = reinterpret_cast<T*>(a.dv) + off4(a.sdv, sl.b, sl.h, sl.s, j);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int d = lane + 32 * t;
      if (d < D) {
        ok[d] = from_float<T>(accK[t] * a.scale);
        ov[d] = from_float<T>(accV[t]);
      }
    }
  }
}

// dBias[b,h,i,j] = sum over the S rows of dS_ij.  One warp owns one (b,h,i) row and
// walks s in order, so the sum order is fixed.
template <class T>
__global__ void __launch_bounds__(GW * 32) generic_dbias_kernel(Args a) {
  extern __shared__ float sm[];
  const int D = a.D, DP = D + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* Qw = sm + warp * 2 * DP;
  float* Gw = Qw + DP;
  const int i = blockIdx.y * GW + warp;
  if (i >= a.R) return;  // warps are independent here (only __syncwarp below)
  const int h = blockIdx.x % a.H, b = blockIdx.x / a.H;
  for (int j0 = 0; j0 < a.R; j0 += 32) {
    const int j = j0 + lane;
    float acc = 0.f;
    for (int s = 0; s < a.S; ++s) {
      __syncwarp();
      const T* q = reinterpret_cast<const T*>(a.q) + off4(a.sq, b, h, s, i);
      const T* g = reinterpret_cast<const T*>(a.d_o) + off4(a.sdo, b, h, s, i);
      for (int d = lane; d < D; d += 32) {
        Qw[d] = to_float<T>(q[d]);
        Gw[d] = to_float<T>(g[d]);
      }
      __syncwarp();
      const long long row = (((long long)b * a.H + h) * a.S + s) * a.R + i;
      const float lse = a.lse[row], delta = a.delta[row];
      if (j < a.R) {
        const T* k = reinterpret_cast<const T*>(a.k) + off4(a.sk, b, h, s, j);
        const T* v = reinterpret_cast<const T*>(a.v) + off4(a.sv, b, h, s, j);
        float dot = 0.f, dp = 0.f;
        for (int d = 0; d < D; ++d) {
          dot += Qw[d] * to_float<T>(k[d]);
          dp += Gw[d] * to_float<T>(v[d]);
        }
        bool rep;
        const float x = score<T>(a, b, h, s, i, j, dot, rep);
        const float p = prob_from_lse(x, lse, a.R);
        acc += rep ? 0.f : p * (dp - delta);
      }
    }
    if (j < a.R) a.dbias[(((long long)b * a.H + h) * a.R + i) * a.R + j] = acc;
  }
}

template <class T>
static cudaError_t launch_fwd_t(const Args& a, cudaStream_t st, int* launches) {
  const int DP = a.D + 1;
  dim3 grid(a.B * a.H * a.S, (a.R + GW - 1) / GW);
  size_t smem = (size_t)(2 * GT + GW) * DP * sizeof(float);
  generic_fwd_kernel<T><<<grid, GW * 32, smem, st>>>(a);
  *launches += 1;
  return cudaGetLastError();
}

template <class T>
static cudaError_t launch_bwd_t(const Args& a, cudaStream_t st, int* launches) {
  const int DP = a.D + 1;
  const long long rows = (long long)a.B * a.H * a.S * a.R;
  if (!a.delta_ready) generic_delta_kernel<T><<<(unsigned)((rows + GW - 1) / GW), GW * 32, 0, st>>>(a);
  dim3 grid(a.B * a.H * a.S, (a.R + GW - 1) / GW);
  generic_dq_kernel<T><<<grid, GW * 32, (size_t)(2 * GT + 2 * GW) * DP * sizeof(float), st>>>(a);
  generic_dkdv_kernel<T><<<grid, GW * 32, ((size_t)(2 * GT + 2 * GW) * DP + 2 * GT) * sizeof(float), st>>>(a);
  *launches += 3;
  if (a.dbias) {
    dim3 g2(a.B * a.H, (a.R + GW - 1) / GW);
    generic_dbias_kernel<T><<<g2, GW * 32, (size_t)GW * 2 * DP * sizeof(float), st>>>(a);
    *launches += 1;
  }
  return cudaGetLastError();
}

cudaError_t launch_generic_fwd(int dtype, const Args& a, cudaStream_t st, int* launches) {
  switch (dtype) {
    case EVOATTN_BF16: return launch_fwd_t<__nv_bfloat16>(a, st, launches);
    case EVOATTN_FP16: return launch_fwd_t<__half>(a, st, launches);
    default: return launch_fwd_t<float>(a, st, launches);
  }
}

cudaError_t launch_generic_bwd(int dtype, const Args& a, cudaStream_t st, int* launches) {
  switch (dtype) {
    case EVOATTN_BF16: return launch_bwd_t<__nv_bfloat16>(a, st, launches);
    case EVOATTN_FP16: return launch_bwd_t<__half>(a, st, launches);
    default: return launch_bwd_t<float>(a, st, launches);
  }
}

}  // namespace evo
