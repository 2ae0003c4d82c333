// Evoformer attention backward for sm_100a, head dimensions 33..64 (smaller ones are served by
// the kernel with transposed score tiles in bwdt_sm100.cu): one fused kernel recomputes P and produces
// dQ, dK, dV and d(pair_bias) with tcgen05 MMAs (accumulators in TMEM) and TMA-staged tiles.
//
// Replaces dsevoformer-triton/evoformer.py:299-326 (_attn_bwd_preprocess), :479-630
// (_attn_bwd_dk_dv) and :329-476 (_attn_bwd_dq).  The reference recomputes S and dP in two
// kernels and adds every dS tile to d_pair_bias with fp32 atomics (:458); here S and dP are
// computed once, and a CTA sums dS over a group of G MSA rows in registers before it
// touches memory, so d(pair_bias) sees one reduction per CTA tile.
//
// Decomposition: a work item is a 128-key tile j of G consecutive MSA rows s of one (b,h), one CTA
// per item.  For an item:
//   for each 128-query tile i:             (pair-bias tile (i,j) is the same for all s)
//     for each of the G rows s:
//       S  = Q_i K_j^T, dP = dO_i V_j^T                      (2 MMAs -> TMEM)
//       P  = exp(scale*S + bias, masked - lse_i),  dS = P (dP - delta_i)   (registers)
//       d_bias_acc += dS                                      (registers, fp32)
//       dV_j[s] += P^T dO_i,  dK_j[s] += dS^T Q_i             (MMAs, TMEM accumulators per s)
//       dQ_i[s] partial = dS K_j  -> fp32 reduction into the dQ scratch buffer
//     d_bias[i-tile, j-tile] += d_bias_acc                    (one vector reduction per tile)
//   write dK_j[s], dV_j[s] for the G rows.
// P and dS (rounded to the storage type, as evoformer.py:459,603,611 do) are written once to
// shared memory as [i][j] tiles in the 128B-swizzled layout and are read by the tensor core
// both K-major (dQ = dS K) and MN-major (dV = P^T dO, dK = dS^T Q).
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace evo {
namespace {

using namespace ptx;

constexpr int BT = 128;  // tile edge (queries and keys)
constexpr int kThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int MASK_MIN = 0;
constexpr int MASK_ADD = 1;

// G = MSA rows per CTA (each needs 2*DP TMEM columns for its dK/dV accumulators).  For DP <= 32
// three rows leave 32+ columns for a dQ partial of its own, which lets the next step's S/dP
// MMAs start while this step's dV/dK/dQ MMAs are still running; at DP = 64 the dQ partial has to
// reuse the S columns.
template <int DP> struct GroupOf {
  static constexpr int G = (DP == 64) ? 2 : 3;
  static constexpr bool kOwnDQ = (DP != 64);
};

template <int DP, int G>
struct BwdSmem {
  static constexpr int RB = DP * 2;
  static constexpr int kTile = BT * RB;
  static constexpr int kPS = BT * BT * 2;       // one P or dS tile
  static constexpr int kBiasChunk = BT * 128;
  static constexpr int offK = 0;                      // G tiles
  static constexpr int offV = offK + G * kTile;       // G tiles
  static constexpr int offQ = offV + G * kTile;        // 2 buffers
  static constexpr int offDO = offQ + 2 * kTile;       // 2 buffers
  static constexpr int offP = offDO + 2 * kTile;
  static constexpr int offDS = offP + kPS;
  static constexpr int offB = offDS + kPS;            // 2 chunk buffers
  static constexpr int offMask = offB + 2 * kBiasChunk;  // G x 128 floats
  static constexpr int offBars = offMask + G * BT * 4;
  static constexpr size_t bytes = offBars + 128 + 1024;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// delta[b,h,s,i] = <dO_i, O_i> (evoformer.py:299-326), one thread per row.
template <class T>
__global__ void __launch_bounds__(256) delta_kernel(Args a) {
  const long long row = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long rows = (long long)a.B * a.H * a.S * a.R;
  if (row >= rows) return;
  const int i = (int)(row % a.R);
  long long sl = row / a.R;
  const int s = (int)(sl % a.S); sl /= a.S;
  const int h = (int)(sl % a.H);
  const int b = (int)(sl / a.H);
  const uint4* o = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.o) + off4(a.so, b, h, s, i));
  const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.d_o) + off4(a.sdo, b, h, s, i));
  float acc = 0.f;
  for (int d8 = 0; d8 < a.D / 8; ++d8) {
    const uint4 ov = o[d8], gv = g[d8];
    const T* op = reinterpret_cast<const T*>(&ov);
    const T* gp = reinterpret_cast<const T*>(&gv);
#pragma unroll
    for (int u = 0; u < 8; ++u) acc += to_float<T>(op[u]) * to_float<T>(gp[u]);
  }
  a.delta[row] = acc;
}

// Dense fp32 copy [B,H,R,R] of a pair bias stored in the 16-bit type (these kernels stage the
// bias as fp32 tiles; the copy lives in the backward's scratch).
template <class T>
__global__ void __launch_bounds__(256) widen_bias_kernel(Args a, float* __restrict__ dst) {
  const long long n = (long long)a.B * a.H * a.R * a.R;
  for (long long e = (long long)blockIdx.x * 256 + threadIdx.x; e < n; e += (long long)gridDim.x * 256) {
    const int j = (int)(e % a.R);
    long long r = e / a.R;
    const int i = (int)(r % a.R); r /= a.R;
    const int h = (int)(r % a.H);
    const int b = (int)(r / a.H);
    dst[e] = load_bias<T>(a, b, h, i, j);
  }
}

// dq = scale * dq_acc, cast to the storage type (dq_acc: contiguous fp32 [B,H,S,R,D]).
template <class T>
__global__ void __launch_bounds__(256) dq_convert_kernel(Args a, const float* __restrict__ acc) {
  const int d8n = a.D / 8;
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  const long long total = (long long)a.B * a.H * a.S * a.R * d8n;
  if (idx >= total) return;
  const int d8 = (int)(idx % d8n);
  const long long row = idx / d8n;
  const int i = (int)(row % a.R);
  long long sl = row / a.R;
  const int s = (int)(sl % a.S); sl /= a.S;
  const int h = (int)(sl % a.H);
  const int b = (int)(sl / a.H);
  const float4* src = reinterpret_cast<const float4*>(acc + row * a.D + d8 * 8);
  const float4 x = src[0], y = src[1];
  uint4 pk;
  pk.x = Pack2<T>::pack(x.x * a.scale, x.y * a.scale);
  pk.y = Pack2<T>::pack(x.z * a.scale, x.w * a.scale);
  pk.z = Pack2<T>::pack(y.x * a.scale, y.y * a.scale);
  pk.w = Pack2<T>::pack(y.z * a.scale, y.w * a.scale);
  *reinterpret_cast<uint4*>(reinterpret_cast<T*>(a.dq) + off4(a.sdq, b, h, s, i) + d8 * 8) = pk;
}

template <class T, int DP, int MASKMODE>
__global__ void __launch_bounds__(kThreads, 1)
evo_bwd_sm100_kernel(const Args a, float* __restrict__ dq_acc, const __grid_constant__ CUtensorMap tmQ,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmB) {
  constexpr int G = GroupOf<DP>::G;
  using L = BwdSmem<DP, G>;
  constexpr int RB = L::RB;
  constexpr uint32_t SWZ = swizzle_code_for_row_bytes(RB);
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int HALF_D = DP / 2;
  constexpr int kTmemCols = 512;
  constexpr int colS = 0, colDP = BT, colDV = 2 * BT, colDK = 2 * BT + G * DP;
  constexpr bool kOwnDQ = GroupOf<DP>::kOwnDQ;
  // the dQ partial has columns of its own, or reuses the S columns once S has been read
  constexpr int colDQ = kOwnDQ ? (2 * BT + 2 * G * DP) : colS;
  static_assert(colDQ + DP <= kTmemCols, "TMEM budget");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + L::offK;
  uint8_t* sV = smem + L::offV;
  uint8_t* sQ = smem + L::offQ;
  uint8_t* sDO = smem + L::offDO;
  uint8_t* sP = smem + L::offP;
  uint8_t* sDS = smem + L::offDS;
  uint8_t* sB = smem + L::offB;
  float* sMask = reinterpret_cast<float*>(smem + L::offMask);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBars);
  uint64_t* bar_kv = bars + 0;
  uint64_t* bar_ld = bars + 6;  // [2], one per Q/dO buffer
  uint64_t* bar_sdp = bars + 2;
  uint64_t* bar_out = bars + 3;
  uint64_t* bar_b = bars + 4;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 9);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;
  const int row = (warp & 3) * 32 + lane;

  const int NT = (a.R + BT - 1) / BT;
  const int NC = (a.S + G - 1) / G;
  int idx = blockIdx.x;
  const int chunk = idx % NC; idx /= NC;
  const int jt = idx % NT; idx /= NT;
  const int h = idx % a.H;
  const int b = idx / a.H;
  const int s0 = chunk * G;
  const int ng = min(G, a.S - s0);
  const int j0 = jt * BT;
  const bool has_bias = a.bias != nullptr;

  if (tid == 0) *abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    mbar_init(bar_kv, 1); mbar_init(bar_ld, 1); mbar_init(bar_ld + 1, 1); mbar_init(bar_sdp, 1); mbar_init(bar_out, 1);
    mbar_init(bar_b + 0, 1); mbar_init(bar_b + 1, 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
    if (has_bias) prefetch_tmap(&tmB);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  // Mask values of the G rows for this key tile.
  for (int t = tid; t < G * BT; t += kThreads) {
    const int g = t / BT, j = j0 + (t % BT);
    float m;
    if (j >= a.R || g >= ng) {
      m = -FLT_MAX;
    } else if (a.mask_kind == EVOATTN_MASK_NONE) {
      m = (MASKMODE == MASK_MIN) ? FLT_MAX : 0.f;
    } else {
      const long long mi = (long long)b * a.smask.a + (long long)(s0 + g) * a.smask.b + (long long)j * a.smask.c;
      if (MASKMODE == MASK_MIN) m = reinterpret_cast<const unsigned char*>(a.mask)[mi] ? FLT_MAX : -FLT_MAX;
      else if (a.mask_kind == EVOATTN_MASK_ADD_F32) m = reinterpret_cast<const float*>(a.mask)[mi];
      else m = to_float<T>(reinterpret_cast<const T*>(a.mask)[mi]);
    }
    sMask[t] = m;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  constexpr uint32_t kIdescS = make_idesc(kBf16, false, false, BT, BT);    // S, dP: both operands K-major
  constexpr uint32_t kIdescT = make_idesc(kBf16, true, true, BT, DP);      // dV, dK: A = P^T / dS^T (MN-major)
  constexpr uint32_t kIdescQ = make_idesc(kBf16, false, true, BT, DP);     // dQ: A = dS K-major, B = K MN-major

  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * ng * L::kTile);
    for (int g = 0; g < ng; ++g) {
      tma_load_5d(sK + g * L::kTile, &tmK, bar_kv, 0, j0, s0 + g, h, b);
      tma_load_5d(sV + g * L::kTile, &tmV, bar_kv, 0, j0, s0 + g, h, b);
    }
  }
  auto issue_bias = [&](int it, int c) {
    mbar_expect_tx(bar_b + wg, L::kBiasChunk);
    tma_load_4d(sB + wg * L::kBiasChunk, &tmB, bar_b + wg, j0 + c * 32, it * BT, h, b);
  };
  if (has_bias && (tid & 127) == 0) issue_bias(0, wg * 2);
  mbar_wait(bar_kv, 0, abort_flag, a.status, DEV_TIMEOUT_TMA);

  const float scale = a.scale;
  const float inv_r = 1.f / (float)a.R;
  uint32_t step = 0, bias_phase = 0;
  const int total_steps = NT * ng;

  // Step n = (query tile n / ng, MSA row n % ng).  Q and dO of step n live in buffer n & 1 and
  // are fetched two steps ahead; S and dP of step n+1 are issued as soon as step n's have been
  // read (right after step n's dV/dK/dQ MMAs when the dQ partial has TMEM columns of its own).
  auto load_q_do = [&](int n) {
    const int buf = n & 1;
    mbar_expect_tx(bar_ld + buf, 2 * L::kTile);
    tma_load_5d(sQ + buf * L::kTile, &tmQ, bar_ld + buf, 0, (n / ng) * BT, s0 + n % ng, h, b);
    tma_load_5d(sDO + buf * L::kTile, &tmDO, bar_ld + buf, 0, (n / ng) * BT, s0 + n % ng, h, b);
  };
  auto issue_s_dp = [&](int n) {
    const int buf = n & 1, g = n % ng;
    mbar_wait(bar_ld + buf, (n >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
    tc_fence_after();
    const uint32_t qa = smem_u32(sQ + buf * L::kTile), ka = smem_u32(sK + g * L::kTile);
    const uint32_t da = smem_u32(sDO + buf * L::kTile), va = smem_u32(sV + g * L::kTile);
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk)
      mma_ss(tmem + colS, make_sdesc(qa + kk * 32, 16, 8 * RB, SWZ), make_sdesc(ka + kk * 32, 16, 8 * RB, SWZ),
             kIdescS, kk > 0 ? 1u : 0u);
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk)
      mma_ss(tmem + colDP, make_sdesc(da + kk * 32, 16, 8 * RB, SWZ), make_sdesc(va + kk * 32, 16, 8 * RB, SWZ),
             kIdescS, kk > 0 ? 1u : 0u);
    mma_commit(bar_sdp);
  };
  if (tid == 0) {
    load_q_do(0);
    if (total_steps > 1) load_q_do(1);
    issue_s_dp(0);
  }

  for (int it = 0; it < NT; ++it) {
    const int i0 = it * BT;
    const int i = i0 + row;
    float bacc[64];
#pragma unroll
    for (int e = 0; e < 64; ++e) bacc[e] = 0.f;

    for (int g = 0; g < ng; ++g, ++step) {
      const int s = s0 + g;
      const uint32_t ph = step & 1;
      // row statistics of my query row
      float lse = 1e30f, delta = 0.f;
      if (i < a.R) {
        const long long ri = (((long long)b * a.H + h) * a.S + s) * a.R + i;
        lse = a.lse[ri];
        delta = a.delta[ri];
      }
      const bool dead = (lse == -FLT_MAX);  // every key of this row was dropped: P is uniform
      const float nlse = -lse * kLog2e;
      mbar_wait(bar_sdp, ph, abort_flag, a.status, DEV_TIMEOUT_MMA);
      tc_fence_after();

#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col0 = wg * 64 + c * 32;
        uint32_t sr[32], dr[32];
        tmem_ld32(t_lane + colS + col0, sr);
        tmem_ld32(t_lane + colDP + col0, dr);
        float bv[32];
        if (has_bias) {
          mbar_wait(bar_b + wg, bias_phase, abort_flag, a.status, DEV_TIMEOUT_TMA);
          bias_phase ^= 1;
          const uint8_t* brow = sB + wg * L::kBiasChunk + row * 128;
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {
            const float4 f = *reinterpret_cast<const float4*>(brow + ((q4 ^ (row & 7)) << 4));
            bv[q4 * 4 + 0] = f.x; bv[q4 * 4 + 1] = f.y; bv[q4 * 4 + 2] = f.z; bv[q4 * 4 + 3] = f.w;
          }
          named_bar_sync(1 + wg, 128);
          if ((tid & 127) == 0) {
            // next chunk in consumption order: (same step, second chunk) or (next step, first chunk)
            if (c == 0) issue_bias(it, wg * 2 + 1);
            else if (step + 1 < (uint32_t)total_steps) issue_bias((g + 1 < ng) ? it : it + 1, wg * 2);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) bv[e] = 0.f;
        }
        tmem_wait_ld();
        const float* mrow = sMask + g * BT + col0;
        uint8_t* prow = sP + wg * (BT * 128) + row * 128;
        uint8_t* drow = sDS + wg * (BT * 128) + row * 128;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float p[8], ds[8];
          const float4 mk0 = *reinterpret_cast<const float4*>(mrow + c8 * 8);
          const float4 mk1 = *reinterpret_cast<const float4*>(mrow + c8 * 8 + 4);
          const float mkv[8] = {mk0.x, mk0.y, mk0.z, mk0.w, mk1.x, mk1.y, mk1.z, mk1.w};
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int e = c8 * 8 + u;
            float x = fmaf(__uint_as_float(sr[e]), scale, bv[e]);
            x = (MASKMODE == MASK_MIN) ? fminf(x, mkv[u]) : (x + mkv[u]);
            if (!dead) {
              p[u] = ex2(fmaf(x, kLog2e, nlse));
              ds[u] = p[u] * (__uint_as_float(dr[e]) - delta);
            } else {
              p[u] = (j0 + col0 + e < a.R) ? inv_r : 0.f;
              ds[u] = 0.f;  // replaced scores are constants: no gradient flows through them
            }
            bacc[c * 32 + e] += ds[u];
          }
          uint4 pk, dk;
          pk.x = Pack2<T>::pack(p[0], p[1]); pk.y = Pack2<T>::pack(p[2], p[3]);
          pk.z = Pack2<T>::pack(p[4], p[5]); pk.w = Pack2<T>::pack(p[6], p[7]);
          dk.x = Pack2<T>::pack(ds[0], ds[1]); dk.y = Pack2<T>::pack(ds[2], ds[3]);
          dk.z = Pack2<T>::pack(ds[4], ds[5]); dk.w = Pack2<T>::pack(ds[6], ds[7]);
          const int chunk16 = ((c * 4 + c8) ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(prow + chunk16) = pk;
          *reinterpret_cast<uint4*>(drow + chunk16) = dk;
        }
      }
      tc_fence_before();
      fence_async_shared();
      __syncthreads();  // P, dS complete in shared memory; S and dP fully read
      if (tid == 0) {
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), dsa = smem_u32(sDS);
        const uint32_t qa = smem_u32(sQ + (step & 1) * L::kTile), da = smem_u32(sDO + (step & 1) * L::kTile);
        const uint32_t ka = smem_u32(sK + g * L::kTile);
        const uint32_t first = (it == 0) ? 0u : 1u;
        // dV_j[s] += P^T dO_i : A = P as MN-major (M = j), K runs over the 128 query rows
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          mma_ss(tmem + colDV + g * DP, make_sdesc(pa + kk * 2048, BT * 128, 1024, SWZ_128B),
                 make_sdesc(da + kk * 16 * RB, 16, 8 * RB, SWZ), kIdescT, (kk > 0) ? 1u : first);
        // dK_j[s] += dS^T Q_i
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          mma_ss(tmem + colDK + g * DP, make_sdesc(dsa + kk * 2048, BT * 128, 1024, SWZ_128B),
                 make_sdesc(qa + kk * 16 * RB, 16, 8 * RB, SWZ), kIdescT, (kk > 0) ? 1u : first);
        // dQ_i[s] partial = dS K_j : A = dS K-major (K runs over the 128 keys)
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          mma_ss(tmem + colDQ, make_sdesc(dsa + (kk >> 2) * (BT * 128) + (kk & 3) * 32, 16, 1024, SWZ_128B),
                 make_sdesc(ka + kk * 16 * RB, 16, 8 * RB, SWZ), kIdescQ, kk > 0 ? 1u : 0u);
        mma_commit(bar_out);
        // S and dP of this step have been read by everyone (barrier above): the next step's can
        // start now, behind the MMAs just issued, unless its dQ partial shares the S columns.
        if (kOwnDQ && step + 1 < (uint32_t)total_steps) issue_s_dp(step + 1);
      }
      mbar_wait(bar_out, ph, abort_flag, a.status, DEV_TIMEOUT_MMA);
      tc_fence_after();
      {
        uint32_t qr[HALF_D];
        tmem_ld<HALF_D>(t_lane + colDQ + wg * HALF_D, qr);
        tmem_wait_ld();
        if (i < a.R) {
          float* dst = dq_acc + ((((long long)b * a.H + h) * a.S + s) * a.R + i) * a.D + wg * HALF_D;
#pragma unroll
          for (int d4 = 0; d4 < HALF_D / 4; ++d4)
            if (wg * HALF_D + d4 * 4 < a.D)
              red_add_v4(dst + d4 * 4, __uint_as_float(qr[d4 * 4]), __uint_as_float(qr[d4 * 4 + 1]),
                         __uint_as_float(qr[d4 * 4 + 2]), __uint_as_float(qr[d4 * 4 + 3]));
        }
      }
      // this step's MMAs are complete: its Q/dO buffer can take the step after next
      if (tid == 0 && step + 2 < (uint32_t)total_steps) load_q_do(step + 2);
      if (!kOwnDQ) {
        tc_fence_before();
        __syncthreads();  // the dQ partial (in the S columns) has been read by everyone
        if (tid == 0 && step + 1 < (uint32_t)total_steps) issue_s_dp(step + 1);
      }
    }

    // one reduction of this CTA's d_bias tile (i-tile, j-tile)
    if (a.dbias != nullptr && i < a.R) {
      float* dst = a.dbias + (((long long)b * a.H + h) * a.R + i) * a.R + j0 + wg * 64;
#pragma unroll
      for (int e4 = 0; e4 < 16; ++e4)
        if (j0 + wg * 64 + e4 * 4 < a.R)
          red_add_v4(dst + e4 * 4, bacc[e4 * 4], bacc[e4 * 4 + 1], bacc[e4 * 4 + 2], bacc[e4 * 4 + 3]);
    }
  }

  // ---- dK, dV of the G rows: TMEM -> registers -> global
  tc_fence_after();
  const int j = j0 + row;
  for (int g = 0; g < ng; ++g) {
    uint32_t kr[HALF_D], vr[HALF_D];
    tmem_ld<HALF_D>(t_lane + colDK + g * DP + wg * HALF_D, kr);
    tmem_ld<HALF_D>(t_lane + colDV + g * DP + wg * HALF_D, vr);
    tmem_wait_ld();
    if (j < a.R) {
      T* kd = reinterpret_cast<T*>(a.dk) + off4(a.sdk, b, h, s0 + g, j) + wg * HALF_D;
      T* vd = reinterpret_cast<T*>(a.dv) + off4(a.sdv, b, h, s0 + g, j) + wg * HALF_D;
#pragma unroll
      for (int d8 = 0; d8 < HALF_D / 8; ++d8) {
        if (wg * HALF_D + d8 * 8 < a.D) {
          uint4 pk, pv;
          pk.x = Pack2<T>::pack(__uint_as_float(kr[d8 * 8 + 0]) * scale, __uint_as_float(kr[d8 * 8 + 1]) * scale);
          pk.y = Pack2<T>::pack(__uint_as_float(kr[d8 * 8 + 2]) * scale, __uint_as_float(kr[d8 * 8 + 3]) * scale);
          pk.z = Pack2<T>::pack(__uint_as_float(kr[d8 * 8 + 4]) * scale, __uint_as_float(kr[d8 * 8 + 5]) * scale);
          pk.w = Pack2<T>::pack(__uint_as_float(kr[d8 * 8 + 6]) * scale, __uint_as_float(kr[d8 * 8 + 7]) * scale);
          pv.x = Pack2<T>::pack(__uint_as_float(vr[d8 * 8 + 0]), __uint_as_float(vr[d8 * 8 + 1]));
          pv.y = Pack2<T>::pack(__uint_as_float(vr[d8 * 8 + 2]), __uint_as_float(vr[d8 * 8 + 3]));
          pv.z = Pack2<T>::pack(__uint_as_float(vr[d8 * 8 + 4]), __uint_as_float(vr[d8 * 8 + 5]));
          pv.w = Pack2<T>::pack(__uint_as_float(vr[d8 * 8 + 6]), __uint_as_float(vr[d8 * 8 + 7]));
          *reinterpret_cast<uint4*>(kd + d8 * 8) = pk;
          *reinterpret_cast<uint4*>(vd + d8 * 8) = pv;
        }
      }
    }
  }
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}


size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <class T, int DP>
int launch_t(const Args& a0, void* ws, size_t ws_bytes, cudaStream_t st, int* launches) {
  constexpr int G = GroupOf<DP>::G;
  using L = BwdSmem<DP, G>;
  Args a = a0;
  const size_t rows = (size_t)a.B * a.H * a.S * a.R;
  const size_t delta_bytes = align_up(rows * sizeof(float), 256);
  const size_t dq_bytes = rows * a.D * sizeof(float);
  const size_t wide_bytes = (a.bias && a.bias16) ? (size_t)a.B * a.H * a.R * a.R * sizeof(float) : 0;
  if (ws_bytes < delta_bytes + align_up(dq_bytes, 256) + wide_bytes) return EVOATTN_ERR_WORKSPACE;
  a.delta = reinterpret_cast<float*>(ws);
  float* dq_acc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + delta_bytes);
  if (wide_bytes) {
    float* wide = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + delta_bytes + align_up(dq_bytes, 256));
    const long long n = (long long)a.B * a.H * a.R * a.R;
    widen_bias_kernel<T><<<(unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096), 256, 0, st>>>(a, wide);
    a.bias = wide;
    a.sbias = Str3{(long long)a.H * a.R * a.R, (long long)a.R * a.R, (long long)a.R};
    a.bias16 = 0;
    *launches += 1;
  }

  CUtensorMap tq, tk, tv, tdo, tb;
  if (!make_qkv_map(&tq, a.q, a.sq, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tk, a.k, a.sk, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tv, a.v, a.sv, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tdo, a.d_o, a.sdo, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  CUtensorMap tdb;
  if (a.bias) {
    if (!make_bias_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, BT, 32)) return EVOATTN_ERR_CUDA;
    const Str3 dense{(long long)a.H * a.R * a.R, (long long)a.R * a.R, (long long)a.R};
    if (!a.dbias) tdb = tq;  // the bias needs no gradient
    else if (!make_bias_map(&tdb, a.dbias, dense, a.B, a.H, a.R, BT, 32)) return EVOATTN_ERR_CUDA;
  } else {
    tb = tq;
    tdb = tq;
  }
  if (cudaMemsetAsync(dq_acc, 0, dq_bytes, st) != cudaSuccess) return EVOATTN_ERR_CUDA;
  if (a.dbias &&
      cudaMemsetAsync(a.dbias, 0, (size_t)a.B * a.H * a.R * a.R * sizeof(float), st) != cudaSuccess)
    return EVOATTN_ERR_CUDA;
  if (!a.delta_ready) delta_kernel<T><<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(a);

  const int NT = (a.R + BT - 1) / BT;
  const bool add = a.mask_kind == EVOATTN_MASK_ADD_F32 || a.mask_kind == EVOATTN_MASK_ADD_SAME;
  {
    const long long ctas = (long long)a.B * a.H * NT * ((a.S + G - 1) / G);
    auto kern = add ? evo_bwd_sm100_kernel<T, DP, MASK_ADD> : evo_bwd_sm100_kernel<T, DP, MASK_MIN>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::bytes) != cudaSuccess)
      return EVOATTN_ERR_CUDA;
    kern<<<(unsigned)ctas, kThreads, L::bytes, st>>>(a, dq_acc, tq, tk, tv, tdo, tb);
  }
  const long long n8 = (long long)rows * (a.D / 8);
  dq_convert_kernel<T><<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(a, dq_acc);
  *launches += 3;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

template <class T>
int launch_d(const Args& a, void* ws, size_t ws_bytes, cudaStream_t st, int* launches) {
#ifdef EVO_D64_T
  if (a.D <= 64)
#else
  if (a.D <= 32)  // the kernel with transposed score tiles (bwdt_sm100.cu)
#endif
    return launch_sm100_bwdt(std::is_same<T, __nv_bfloat16>::value ? EVOATTN_BF16 : EVOATTN_FP16, a, ws, ws_bytes, st,
                             launches);
  return launch_t<T, 64>(a, ws, ws_bytes, st, launches);
}

}  // namespace

bool sm100_bwd_supported(int dtype, const Args& a) {
  if (!sm100_fwd_supported(dtype, a)) return false;
  const long long NT = (a.R + BT - 1) / BT;
  if ((long long)a.B * a.H * NT * a.S > 2147483647LL) return false;
  return true;
}

size_t sm100_bwd_workspace_bytes(int, const Args& a) {
#ifdef EVO_D64_T
  if (a.D <= 64) return sm100_bwdt_workspace_bytes(a);
#endif
  if (a.D <= 32) return sm100_bwdt_workspace_bytes(a);
  const size_t rows = (size_t)a.B * a.H * a.S * a.R;
  const size_t wide_bytes = (a.bias && a.bias16) ? (size_t)a.B * a.H * a.R * a.R * sizeof(float) : 0;
  return align_up(rows * sizeof(float), 256) + align_up(rows * a.D * sizeof(float), 256) + wide_bytes;
}

int launch_sm100_bwd(int dtype, const Args& a, void* workspace, size_t workspace_bytes, cudaStream_t st,
                     int* launches) {
  if (dtype == EVOATTN_BF16) return launch_d<__nv_bfloat16>(a, workspace, workspace_bytes, st, launches);
  return launch_d<__half>(a, workspace, workspace_bytes, st, launches);
}

}  // namespace evo
