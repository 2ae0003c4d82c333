// Evoformer attention forward for sm_100a: TMA-staged tiles, tcgen05 MMAs with the
// accumulators in TMEM, online softmax with pair bias and residue mask in registers.
//
// Computes what dsevoformer-triton/evoformer.py:23-100 (_attn_fwd_inner) and :103-297
// (_attn_fwd) compute:  O = softmax(scale*Q K^T + bias, masked) V  and the row
// log-sum-exp, without ever writing the R x R scores to memory.
//
// One CTA = one 128-row query tile of one (b,h,s) slab, 256 threads:
//   * thread 0 issues the TMA loads of Q, K, V and all tcgen05.mma instructions;
//   * all 8 warps run the softmax: thread (warp w, lane l) owns score row 32*(w%4)+l
//     (= its TMEM lane) and the 64 columns of half w/4 of each 128-key tile;
//   * S = Q K^T lands in TMEM columns [0,128); P (rounded to the storage type, as
//     evoformer.py:84 does) goes to shared memory in the K-major 128B-swizzled layout
//     and P V lands in TMEM columns [128,128+DP); the running O lives in registers.
//   * the pair-bias tile arrives by TMA in 128x32 fp32 chunks (128B swizzle) so that a
//     thread can read "its" row with conflict-free 16-byte shared loads.
#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace evo {
namespace {

using namespace ptx;

constexpr int BM = 128;        // query rows per CTA
constexpr int BN = 128;        // keys per tile
constexpr int kThreads = 256;
constexpr int kTmemCols = 256; // S [0,128) + PV [128,128+DP)
constexpr float kLog2e = 1.4426950408889634f;
constexpr int MASK_MIN = 0;    // boolean keep-mask (or none): score = min(score, m) with m = +-FLT_MAX
constexpr int MASK_ADD = 1;    // additive mask

template <int DP>
struct FwdSmem {
  static constexpr int RB = DP * 2;            // bytes per staged Q/K/V row
  static constexpr int kTile = BM * RB;        // bytes per Q/K/V tile
  static constexpr int kP = BM * BN * 2;       // 32 KB
  static constexpr int kBiasChunk = BM * 128;  // 128 rows x 32 fp32
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + kTile;
  static constexpr int offV = offK + kTile;
  static constexpr int offP = offV + kTile;
  static constexpr int offB = offP + kP;       // two chunk buffers, one per warpgroup
  static constexpr int offMask = offB + 2 * kBiasChunk;
  static size_t bytes(int r_pad) {
    return (size_t)offMask + (size_t)r_pad * 4 /*mask*/ + 4 * BM * 4 /*pmax,psum*/ + 128 /*barriers*/ + 1024 /*align*/;
  }
};

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

template <class T, int DP, int MASKMODE>
__global__ void __launch_bounds__(kThreads, 1)
evo_fwd_sm100_kernel(const Args a, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmB) {
  using L = FwdSmem<DP>;
  constexpr int RB = L::RB;
  constexpr uint32_t SWZ = swizzle_code_for_row_bytes(RB);
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int HALF_D = DP / 2;  // PV columns each thread accumulates

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::offQ;
  uint8_t* sK = smem + L::offK;
  uint8_t* sV = smem + L::offV;
  uint8_t* sP = smem + L::offP;
  uint8_t* sB = smem + L::offB;
  float* sMask = reinterpret_cast<float*>(smem + L::offMask);
  const int NT = (a.R + BN - 1) / BN;
  const int r_pad = NT * BN;
  float* sPmax = sMask + r_pad;          // [2][BM]
  float* sPsum = sPmax + 2 * BM;         // [2][BM]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sPsum + 2 * BM);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_k = bars + 1;
  uint64_t* bar_v = bars + 2;
  uint64_t* bar_s = bars + 3;
  uint64_t* bar_o = bars + 4;
  uint64_t* bar_b = bars + 5;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 9);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;                  // column half
  const int row = (warp & 3) * 32 + lane;    // score row inside the tile == TMEM lane

  // CTA -> (b, h, q-tile, s); s fastest so neighbouring CTAs share the same bias rows in L2.
  const int NQT = (a.R + BM - 1) / BM;
  int idx = blockIdx.x;
  const int s = idx % a.S; idx /= a.S;
  const int qt = idx % NQT; idx /= NQT;
  const int h = idx % a.H;
  const int b = idx / a.H;
  const int i0 = qt * BM;
  const bool has_bias = a.bias != nullptr;

  // A launch that follows a failed one returns at once (one reader, so the CTA agrees).
  if (tid == 0) *abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_o, 1);
    mbar_init(bar_b + 0, 1); mbar_init(bar_b + 1, 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
    if (has_bias) prefetch_tmap(&tmB);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  // Mask row of this (b, s) as one float per key.  Keys beyond R are always excluded.
  for (int j = tid; j < r_pad; j += kThreads) {
    float m;
    if (j >= a.R) {
      m = -FLT_MAX;
    } else if (a.mask_kind == EVOATTN_MASK_NONE) {
      m = (MASKMODE == MASK_MIN) ? FLT_MAX : 0.f;
    } else {
      const long long mi = (long long)b * a.smask.a + (long long)s * a.smask.b + (long long)j * a.smask.c;
      if (MASKMODE == MASK_MIN) m = reinterpret_cast<const unsigned char*>(a.mask)[mi] ? FLT_MAX : -FLT_MAX;
      else if (a.mask_kind == EVOATTN_MASK_ADD_F32) m = reinterpret_cast<const float*>(a.mask)[mi];
      else m = to_float<T>(reinterpret_cast<const T*>(a.mask)[mi]);
    }
    sMask[j] = m;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  const uint32_t tS = t_lane;              // columns [0,128)
  const uint32_t tO = t_lane + BN;         // columns [128,128+DP)

  constexpr uint32_t kIdescS = make_idesc(kBf16, false, false, BM, BN);
  constexpr uint32_t kIdescO = make_idesc(kBf16, false, true, BM, DP);

  auto issue_s_mma = [&]() {
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      const uint64_t ad = make_sdesc(qa + kk * 32, 16, 8 * RB, SWZ);
      const uint64_t bd = make_sdesc(ka + kk * 32, 16, 8 * RB, SWZ);
      mma_ss(tmem, ad, bd, kIdescS, kk > 0 ? 1u : 0u);
    }
    mma_commit(bar_s);
  };
  auto issue_o_mma = [&]() {
    const uint32_t pa = smem_u32(sP), va = smem_u32(sV);
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      const uint64_t ad = make_sdesc(pa + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024, SWZ_128B);
      const uint64_t bd = make_sdesc(va + kk * 16 * RB, 16, 8 * RB, SWZ);
      mma_ss(tmem + BN, ad, bd, kIdescO, kk > 0 ? 1u : 0u);
    }
    mma_commit(bar_o);
  };
  // Pair-bias chunk c (0..3) of key tile jt -> this warpgroup's buffer.
  auto issue_bias = [&](int jt, int c) {
    mbar_expect_tx(bar_b + wg, L::kBiasChunk);
    tma_load_4d(sB + wg * L::kBiasChunk, &tmB, bar_b + wg, jt * BN + c * 32, i0, h, b);
  };

  if (tid == 0) {
    mbar_expect_tx(bar_q, L::kTile);
    tma_load_5d(sQ, &tmQ, bar_q, 0, i0, s, h, b);
    mbar_expect_tx(bar_k, L::kTile);
    tma_load_5d(sK, &tmK, bar_k, 0, 0, s, h, b);
    mbar_expect_tx(bar_v, L::kTile);
    tma_load_5d(sV, &tmV, bar_v, 0, 0, s, h, b);
  }
  if (has_bias && (tid & 127) == 0) issue_bias(0, wg * 2);
  if (tid == 0) {
    mbar_wait(bar_q, 0, abort_flag, a.status, DEV_TIMEOUT_TMA);
    mbar_wait(bar_k, 0, abort_flag, a.status, DEV_TIMEOUT_TMA);
    tc_fence_after();
    issue_s_mma();
  }

  float m_run = -FLT_MAX, l_run = 0.f;
  float acc[HALF_D];
#pragma unroll
  for (int d = 0; d < HALF_D; ++d) acc[d] = 0.f;
  uint32_t bias_phase = 0;
  const float scale = a.scale;

  for (int jt = 0; jt < NT; ++jt) {
    const uint32_t ph = jt & 1;
    mbar_wait(bar_s, ph, abort_flag, a.status, DEV_TIMEOUT_MMA);
    tc_fence_after();
    if (tid == 0 && jt + 1 < NT) {  // S MMA is done with the K tile
      mbar_expect_tx(bar_k, L::kTile);
      tma_load_5d(sK, &tmK, bar_k, 0, (jt + 1) * BN, s, h, b);
    }

    // ---- scores of my 64 columns: x = scale*S + bias, then the mask
    float x[64];
    float mx = -FLT_MAX;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t sr[32];
      tmem_ld32(tS + wg * 64 + c * 32, sr);
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
        named_bar_sync(1 + wg, 128);  // the whole warpgroup has read the chunk
        if ((tid & 127) == 0) {
          if (c == 0) issue_bias(jt, wg * 2 + 1);
          else if (jt + 1 < NT) issue_bias(jt + 1, wg * 2);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) bv[e] = 0.f;
      }
      tmem_wait_ld();
      const float* mrow = sMask + jt * BN + wg * 64 + c * 32;
#pragma unroll
      for (int e4 = 0; e4 < 8; ++e4) {
        const float4 mk = *reinterpret_cast<const float4*>(mrow + e4 * 4);
        const float mkv[4] = {mk.x, mk.y, mk.z, mk.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int e = e4 * 4 + u;
          float v = fmaf(__uint_as_float(sr[e]), scale, bv[e]);
          v = (MASKMODE == MASK_MIN) ? fminf(v, mkv[u]) : (v + mkv[u]);
          x[c * 32 + e] = v;
          mx = fmaxf(mx, v);
        }
      }
    }
    sPmax[wg * BM + row] = mx;
    tc_fence_before();
    __syncthreads();  // (1) all S reads done; partial row maxima visible
    if (tid == 0 && jt + 1 < NT) {
      mbar_wait(bar_k, (jt + 1) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
      tc_fence_after();
      issue_s_mma();  // next tile's scores overlap this tile's exponentials
    }
    const float m_new = fmaxf(m_run, fmaxf(sPmax[row], sPmax[BM + row]));
    // A row whose keys are all dropped so far has every score at -FLT_MAX: its
    // probabilities are uniform over the real keys (test.py:54-55 semantics).
    const bool dead = (m_new == -FLT_MAX);
    const float alpha = dead ? 1.f : ex2((m_run - m_new) * kLog2e);
    const float nm2 = -m_new * kLog2e;
    float lsum = 0.f;
    uint8_t* prow = sP + wg * (BM * 128) + row * 128;
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
      float p[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = c8 * 8 + u;
        if (!dead) p[u] = ex2(fmaf(x[e], kLog2e, nm2));
        else p[u] = (jt * BN + wg * 64 + e < a.R) ? 1.f : 0.f;
        lsum += p[u];
      }
      uint4 pk;
      pk.x = Pack2<T>::pack(p[0], p[1]);
      pk.y = Pack2<T>::pack(p[2], p[3]);
      pk.z = Pack2<T>::pack(p[4], p[5]);
      pk.w = Pack2<T>::pack(p[6], p[7]);
      *reinterpret_cast<uint4*>(prow + ((c8 ^ (row & 7)) << 4)) = pk;
    }
    l_run = l_run * alpha + lsum;
    m_run = m_new;
    fence_async_shared();
    __syncthreads();  // (2) P is complete in shared memory
    if (tid == 0) {
      mbar_wait(bar_v, ph, abort_flag, a.status, DEV_TIMEOUT_TMA);
      tc_fence_after();
      issue_o_mma();
    }
#pragma unroll
    for (int d = 0; d < HALF_D; ++d) acc[d] *= alpha;
    mbar_wait(bar_o, ph, abort_flag, a.status, DEV_TIMEOUT_MMA);
    tc_fence_after();
    if (tid == 0 && jt + 1 < NT) {  // P V is done with the V tile
      mbar_expect_tx(bar_v, L::kTile);
      tma_load_5d(sV, &tmV, bar_v, 0, (jt + 1) * BN, s, h, b);
    }
    uint32_t orr[HALF_D];
    tmem_ld<HALF_D>(tO + wg * HALF_D, orr);
    tmem_wait_ld();
#pragma unroll
    for (int d = 0; d < HALF_D; ++d) acc[d] += __uint_as_float(orr[d]);
  }

  // ---- epilogue: combine the two column halves' row sums, normalise, store
  sPsum[wg * BM + row] = l_run;
  tc_fence_before();
  __syncthreads();
  const float l_tot = sPsum[row] + sPsum[BM + row];
  const float inv = 1.f / l_tot;
  const int i = i0 + row;
  if (i < a.R) {
    T* orow = reinterpret_cast<T*>(a.o) + off4(a.so, b, h, s, i) + wg * HALF_D;
#pragma unroll
    for (int d8 = 0; d8 < HALF_D / 8; ++d8) {
      if (wg * HALF_D + d8 * 8 < a.D) {
        uint4 pk;
        pk.x = Pack2<T>::pack(acc[d8 * 8 + 0] * inv, acc[d8 * 8 + 1] * inv);
        pk.y = Pack2<T>::pack(acc[d8 * 8 + 2] * inv, acc[d8 * 8 + 3] * inv);
        pk.z = Pack2<T>::pack(acc[d8 * 8 + 4] * inv, acc[d8 * 8 + 5] * inv);
        pk.w = Pack2<T>::pack(acc[d8 * 8 + 6] * inv, acc[d8 * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(orow + d8 * 8) = pk;
      }
    }
    if (wg == 0) {
      const long long li = (((long long)b * a.H + h) * a.S + s) * a.R + i;
      a.lse[li] = (m_run == -FLT_MAX) ? -FLT_MAX : (m_run + logf(l_tot));
    }
  }
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA retires
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

template <class T, int DP>
int launch_t(const Args& a, cudaStream_t st, int* launches) {
  using L = FwdSmem<DP>;
  CUtensorMap tq, tk, tv, tb;
  if (!make_qkv_map(&tq, a.q, a.sq, a.B, a.H, a.S, a.R, a.D, DP, BM)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tk, a.k, a.sk, a.B, a.H, a.S, a.R, a.D, DP, BN)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tv, a.v, a.sv, a.B, a.H, a.S, a.R, a.D, DP, BN)) return EVOATTN_ERR_CUDA;
  if (a.bias) {
    if (!make_bias_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, BM)) return EVOATTN_ERR_CUDA;
  } else {
    tb = tq;
  }
  const int NT = (a.R + BN - 1) / BN;
  const size_t smem = L::bytes(NT * BN);
  const long long ctas = (long long)a.B * a.H * a.S * ((a.R + BM - 1) / BM);
  const bool add = a.mask_kind == EVOATTN_MASK_ADD_F32 || a.mask_kind == EVOATTN_MASK_ADD_SAME;
  auto kern = add ? evo_fwd_sm100_kernel<T, DP, MASK_ADD> : evo_fwd_sm100_kernel<T, DP, MASK_MIN>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return EVOATTN_ERR_CUDA;
  kern<<<(unsigned)ctas, kThreads, smem, st>>>(a, tq, tk, tv, tb);
  *launches += 1;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

template <class T>
int launch_d(const Args& a, cudaStream_t st, int* launches) {
  if (a.D <= 16) return launch_t<T, 16>(a, st, launches);
  if (a.D <= 32) return launch_t<T, 32>(a, st, launches);
  return launch_t<T, 64>(a, st, launches);
}

}  // namespace

bool sm100_fwd_supported(int dtype, const Args& a) {
  if (dtype != EVOATTN_BF16 && dtype != EVOATTN_FP16) return false;
  if (a.D % 8 != 0 || a.D > 64) return false;
  if (a.R > 8192) return false;  // the mask row is staged in shared memory
  if (a.bias) {
    if ((reinterpret_cast<uintptr_t>(a.bias) & 15) != 0) return false;
    if ((a.sbias.a * 4) % 16 || (a.sbias.b * 4) % 16 || (a.sbias.c * 4) % 16) return false;
  }
  if ((long long)a.B * a.H * a.S * ((a.R + BM - 1) / BM) > 2147483647LL) return false;
  return true;
}

int launch_sm100_fwd(int dtype, const Args& a, cudaStream_t st, int* launches) {
  if (dtype == EVOATTN_BF16) return launch_d<__nv_bfloat16>(a, st, launches);
  return launch_d<__half>(a, st, launches);
}

}  // namespace evo
