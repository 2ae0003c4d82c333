// d(pair_bias) for sm_100a as a kernel of its own: dBias[b,h,i,j] = sum over the MSA rows s of
// dS_ij(s), with dS = P (dP - delta) recomputed from Q, K, V, dO, lse and delta.
//
// The reference produces this sum with one fp32 atomic per score and row
// (dsevoformer-triton/evoformer.py:458).  Global fp32 reductions are a scarce resource on the
// GPU (about 16 bytes per clock and SM), so this kernel keeps the whole sum on chip: a CTA owns
// ONE 128x128 tile (i-tile, j-tile) of one (b,h) and walks over a range of MSA rows with the
// running sum in registers; the tile leaves the CTA once.  The price is that S and dP are
// computed here a second time (the fused backward kernel computes them for dQ, dK, dV).
//
// 384 threads: warps 0-7 compute (thread = query row i, 64 of the 128 keys), warp 8 issues TMA
// loads and tcgen05.mma, warp 9 stages the residue-mask values of the coming rows.
//   * the pair-bias tile of the CTA is loaded into shared memory once (64 KB, 128B swizzle);
//   * Q_i, dO_i, K_j, V_j of a row arrive in a ring of kStages stages;
//   * S = Q K^T and dP = dO V^T of row n+1 are computed into the second half of TMEM while the
//     compute warps work on row n (no accumulators live in TMEM here, so S/dP are double buffered).
#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace evo {
namespace {

using namespace ptx;

constexpr int BT = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int MASK_MIN = 0;
constexpr int MASK_ADD = 1;

template <int N> __device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int DP>
struct DbSmem {
  static constexpr int kStages = (DP == 64) ? 2 : 4;
  static constexpr int RB = DP * 2;
  static constexpr int kTile = BT * RB;
  static constexpr int kStage = 4 * kTile;            // Q, dO, K, V of one row
  static constexpr int kBias = BT * BT * 4;           // resident pair-bias tile: four 128x32 boxes
  static constexpr int offStage = 0;
  static constexpr int offBias = offStage + kStages * kStage;
  static constexpr int offMask = offBias + kBias;      // [kStages][128] floats
  static constexpr int offBars = offMask + kStages * BT * 4;
  static constexpr size_t bytes = offBars + 256 + 1024;
};

template <class T, int DP, int MASKMODE>
__global__ void __launch_bounds__(384, 1)
evo_dbias_kernel(const Args a, const int rows_per_cta, const __grid_constant__ CUtensorMap tmQ,
                 const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmB) {
  using L = DbSmem<DP>;
  constexpr int NST = L::kStages;
  constexpr int RB = L::RB;
  constexpr uint32_t SWZ = swizzle_code_for_row_bytes(RB);
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int kTmemCols = 512;  // two buffers of (S 128 + dP 128)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sBias = smem + L::offBias;
  float* sMask = reinterpret_cast<float*>(smem + L::offMask);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBars);
  uint64_t* bar_ld = bars + 0;        // [NST] tiles of a row landed
  uint64_t* bar_free = bars + 4;      // [NST] stage consumed by its MMAs
  uint64_t* bar_mfull = bars + 8;     // [NST] mask values of a row staged
  uint64_t* bar_mfree = bars + 12;    // [NST] mask values consumed (8 warps)
  uint64_t* bar_sdp = bars + 16;      // [2] S, dP of a row complete
  uint64_t* bar_cdone = bars + 18;    // [2] the 8 compute warps have read a TMEM buffer
  uint64_t* bar_bias = bars + 20;     // resident bias tile landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 22);
  volatile uint32_t* scratch = reinterpret_cast<volatile uint32_t*>(bars + 23);  // written, never read

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = (a.R + BT - 1) / BT;
  const int NCH = (a.S + rows_per_cta - 1) / rows_per_cta;
  int idx = blockIdx.x;
  const int ch = idx % NCH; idx /= NCH;
  const int jt = idx % NT; idx /= NT;
  const int it = idx % NT; idx /= NT;
  const int h = idx % a.H;
  const int b = idx / a.H;
  const int s0 = ch * rows_per_cta;
  const int nrows = min(rows_per_cta, a.S - s0);
  const int i0 = it * BT, j0 = jt * BT;
  const bool has_bias = a.bias != nullptr;

  if (tid == 0) *abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(bar_ld + i, 1); mbar_init(bar_free + i, 1);
      mbar_init(bar_mfull + i, 1); mbar_init(bar_mfree + i, 8);
    }
    mbar_init(bar_sdp, 1); mbar_init(bar_sdp + 1, 1);
    mbar_init(bar_cdone, 8); mbar_init(bar_cdone + 1, 8);
    mbar_init(bar_bias, 1);
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
    if (has_bias) prefetch_tmap(&tmB);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= 8) {
    setmaxnreg_dec<24>();
    if (warp == 8) {
      // =============================== control: TMA + MMA ===============================
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      constexpr uint32_t kIdescS = make_idesc(kBf16, false, false, BT, BT);
      constexpr uint32_t kHiOp = static_cast<uint32_t>(make_sdesc_const(16, 8 * RB, SWZ) >> 32);
      constexpr uint32_t kLoLbo = static_cast<uint32_t>(make_sdesc_const(16, 0, 0) & 0xffffffffu);
      const uint32_t st_lo = smem_u32(smem + L::offStage) >> 4;
      auto load_row = [&](int n) {
        const int st = n % NST, s = s0 + n;
        mbar_wait(bar_free + st, ((n / NST) & 1) ^ 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
        uint8_t* dst = smem + L::offStage + st * L::kStage;
        mbar_expect_tx_if(leader, bar_ld + st, L::kStage);
        tma_load_5d_if(leader, dst, &tmQ, bar_ld + st, 0, i0, s, h, b);
        tma_load_5d_if(leader, dst + L::kTile, &tmDO, bar_ld + st, 0, i0, s, h, b);
        tma_load_5d_if(leader, dst + 2 * L::kTile, &tmK, bar_ld + st, 0, j0, s, h, b);
        tma_load_5d_if(leader, dst + 3 * L::kTile, &tmV, bar_ld + st, 0, j0, s, h, b);
      };
      if (has_bias) {
        mbar_expect_tx_if(leader, bar_bias, L::kBias);
        for (int c = 0; c < 4; ++c)
          tma_load_4d_if(leader, sBias + c * (BT * 128), &tmB, bar_bias, j0 + c * 32, i0, h, b);
      }
      for (int n = 0; n < NST && n < nrows; ++n) load_row(n);
      for (int n = 0; n < nrows; ++n) {
        const int st = n % NST, u = n & 1;
        mbar_wait(bar_ld + st, (n / NST) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
        // TMEM buffer u was last read for row n-2
        if (n >= 2) mbar_wait(bar_cdone + u, ((n - 2) >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
        tc_fence_after();
        const uint32_t base = (st_lo + st * (L::kStage >> 4)) | kLoLbo;
        const uint32_t qa = base, da = base + (L::kTile >> 4), ka = base + 2 * (L::kTile >> 4),
                       va = base + 3 * (L::kTile >> 4);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk)
          mma_ss_if(leader, tmem + u * 256, pack_desc(qa + kk * 2, kHiOp), pack_desc(ka + kk * 2, kHiOp), kIdescS,
                    kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk)
          mma_ss_if(leader, tmem + u * 256 + BT, pack_desc(da + kk * 2, kHiOp), pack_desc(va + kk * 2, kHiOp), kIdescS,
                    kk > 0 ? 1u : 0u);
        mma_commit_if(leader, bar_free + st);
        mma_commit_if(leader, bar_sdp + u);
        if (n + NST < nrows) load_row(n + NST);  // waits for the commit above
      }
    } else if (warp == 9) {
      // =============================== residue-mask stager ===============================
      for (int n = 0; n < nrows; ++n) {
        const int st = n % NST, s = s0 + n;
        mbar_wait(bar_mfree + st, ((n / NST) & 1) ^ 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
        float m[4];  // four independent loads per lane, then the stores
#pragma unroll
        for (int u = 0; u < 4; ++u) m[u] = mask_value<T, MASKMODE == MASK_MIN>(a, b, s, j0 + u * 32 + lane);
#pragma unroll
        for (int u = 0; u < 4; ++u) sMask[st * BT + u * 32 + lane] = m[u];
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_mfull + st);
      }
    }
  } else {
    // =============================== compute warps ===============================
    setmaxnreg_inc<240>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int i = i0 + row;
    const uint32_t t_lane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const F2 scale2 = f2_make(a.scale, a.scale), l2e2 = f2_make(kLog2e, kLog2e);

    float bacc[64];
#pragma unroll
    for (int e = 0; e < 64; ++e) bacc[e] = 0.f;

    float lse_next = 1e30f, delta_next = 0.f;
    auto load_row_stats = [&](int n) {  // out-of-range rows get a huge lse so that their P is exactly 0
      lse_next = 1e30f;
      delta_next = 0.f;
      if (n < nrows && i < a.R) {
        const long long ri = (((long long)b * a.H + h) * a.S + s0 + n) * a.R + i;
        lse_next = a.lse[ri];
        delta_next = a.delta[ri];
      }
    };
    load_row_stats(0);
    if (has_bias) mbar_wait(bar_bias, 0, abort_flag, a.status, DEV_TIMEOUT_TMA);
    const uint8_t* brow = sBias + (wg * 2) * (BT * 128) + row * 128;  // my row in my two 32-column boxes

    for (int n = 0; n < nrows; ++n) {
      const int st = n % NST, u = n & 1;
      const float lse = lse_next, delta = delta_next;
      load_row_stats(n + 1);
      const bool dead = (lse == -FLT_MAX);  // every key of this row was dropped: dS = 0
      const float nlse = -lse * kLog2e;
      const F2 nlse2 = f2_make(nlse, nlse), delta2 = f2_make(delta, delta);
      mbar_wait(bar_mfull + st, (n / NST) & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
      mbar_wait(bar_sdp + u, (n >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
      tc_fence_after();
      if (!dead) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = wg * 64 + c * 32;
          uint32_t sr[32], dr[32];
          tmem_ld32(t_lane + u * 256 + col0, sr);
          tmem_ld32(t_lane + u * 256 + BT + col0, dr);
          tmem_wait_ld();
          const float* mrow = sMask + st * BT + col0;
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
            if (has_bias) {
              b0 = *reinterpret_cast<const float4*>(brow + c * (BT * 128) + (((q8 * 2) ^ (row & 7)) << 4));
              b1 = *reinterpret_cast<const float4*>(brow + c * (BT * 128) + (((q8 * 2 + 1) ^ (row & 7)) << 4));
            }
            const float4 k0 = *reinterpret_cast<const float4*>(mrow + q8 * 8);
            const float4 k1 = *reinterpret_cast<const float4*>(mrow + q8 * 8 + 4);
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            const float mkv[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
            const int e0 = q8 * 8;
            float x[8], p[8];
#pragma unroll
            for (int v = 0; v < 8; v += 2)
              f2_get(f2_fma(f2_from_bits(sr[e0 + v], sr[e0 + v + 1]), scale2, f2_make(bv[v], bv[v + 1])), x[v], x[v + 1]);
#pragma unroll
            for (int v = 0; v < 8; ++v) x[v] = (MASKMODE == MASK_MIN) ? fminf(x[v], mkv[v]) : (x[v] + mkv[v]);
#pragma unroll
            for (int v = 0; v < 8; v += 2) f2_get(f2_fma(f2_make(x[v], x[v + 1]), l2e2, nlse2), x[v], x[v + 1]);
#pragma unroll
            for (int v = 0; v < 8; ++v) p[v] = ex2(x[v]);
#pragma unroll
            for (int v = 0; v < 8; v += 2) {
              const F2 t = f2_mul(f2_make(p[v], p[v + 1]), f2_sub(f2_from_bits(dr[e0 + v], dr[e0 + v + 1]), delta2));
              f2_get(f2_add(f2_make(bacc[c * 32 + e0 + v], bacc[c * 32 + e0 + v + 1]), t), bacc[c * 32 + e0 + v],
                     bacc[c * 32 + e0 + v + 1]);
            }
          }
        }
      }
      // The mask stage is handed back only after the loads from it have returned: the store needs
      // a sum that every one of them fed (an mbarrier arrival by itself does not wait for shared
      // loads that are still queued).
      {
        uint32_t dep = 0;
#pragma unroll
        for (int e = 0; e < 64; e += 4) dep ^= __float_as_uint(bacc[e]);
        *scratch = dep;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_cdone + u);
        mbar_arrive(bar_mfree + st);
      }
    }

    // the tile leaves the CTA once: plain stores when this CTA saw every MSA row, else a reduction
    if (i < a.R) {
      float* dst = a.dbias + (((long long)b * a.H + h) * a.R + i) * a.R + j0 + wg * 64;
#pragma unroll
      for (int e4 = 0; e4 < 16; ++e4) {
        if (j0 + wg * 64 + e4 * 4 < a.R) {
          if (NCH == 1)
            *reinterpret_cast<float4*>(dst + e4 * 4) =
                make_float4(bacc[e4 * 4], bacc[e4 * 4 + 1], bacc[e4 * 4 + 2], bacc[e4 * 4 + 3]);
          else
            red_add_v4(dst + e4 * 4, bacc[e4 * 4], bacc[e4 * 4 + 1], bacc[e4 * 4 + 2], bacc[e4 * 4 + 3]);
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

int g_sms = 0;

template <class T, int DP>
int launch_t(const Args& a, cudaStream_t st, int* launches) {
  using L = DbSmem<DP>;
  CUtensorMap tq, tk, tv, tdo, tb;
  if (!make_qkv_map(&tq, a.q, a.sq, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tk, a.k, a.sk, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tv, a.v, a.sv, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tdo, a.d_o, a.sdo, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_bias_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, BT, 32)) return EVOATTN_ERR_CUDA;
  if (g_sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      return EVOATTN_ERR_CUDA;
    g_sms = n;
  }
  // Split the MSA rows into as many chunks as it takes to give every SM about two CTAs, but keep
  // at least 8 rows per CTA so that the one-off costs (bias tile, pipeline fill) stay small.
  const int NT = (a.R + BT - 1) / BT;
  const long long tiles = (long long)a.B * a.H * NT * NT;
  int nch = (int)((2LL * g_sms + tiles - 1) / tiles);
  if (nch < 1) nch = 1;
  int rows = (a.S + nch - 1) / nch;
  if (rows < 8) rows = a.S < 8 ? a.S : 8;
  nch = (a.S + rows - 1) / rows;
  if (nch > 1 &&
      cudaMemsetAsync(a.dbias, 0, (size_t)a.B * a.H * a.R * a.R * sizeof(float), st) != cudaSuccess)
    return EVOATTN_ERR_CUDA;
  const bool add = a.mask_kind == EVOATTN_MASK_ADD_F32 || a.mask_kind == EVOATTN_MASK_ADD_SAME;
  auto kern = add ? evo_dbias_kernel<T, DP, MASK_ADD> : evo_dbias_kernel<T, DP, MASK_MIN>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::bytes) != cudaSuccess)
    return EVOATTN_ERR_CUDA;
  kern<<<(unsigned)(tiles * nch), 384, L::bytes, st>>>(a, rows, tq, tk, tv, tdo, tb);
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

// Needs a.delta (fp32 [B,H,S,R]) filled and a.dbias non-null.  Writes a.dbias in full.
int launch_sm100_dbias(int dtype, const Args& a, cudaStream_t st, int* launches) {
  if (dtype == EVOATTN_BF16) return launch_d<__nv_bfloat16>(a, st, launches);
  return launch_d<__half>(a, st, launches);
}

}  // namespace evo
