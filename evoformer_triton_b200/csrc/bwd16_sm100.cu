// Evoformer attention backward for sm_100a, head dimension 32 (D <= 32 padded to 32): the fused
// dQ/dK/dV/d(pair_bias) kernel of bwd_sm100.cu with sixteen compute warps instead of eight.
//
// Replaces dsevoformer-triton/evoformer.py:479-630 (_attn_bwd_dk_dv) and :329-476 (_attn_bwd_dq);
// the decomposition into work items and steps, the TMEM budget and the shared-memory layout are
// those of the warp-specialised kernel in bwd_sm100.cu.  What differs is who does the arithmetic:
//   * 640 threads: warps 0-15 compute, warp 16 issues every tcgen05.mma and the dQ reductions,
//     warps 17 and 18 feed the pair bias and send the d_bias blocks off, warp 19 loads the
//     Q/dO/K/V tiles.
//   * Compute warp w owns query rows 32*(w%4).. (the TMEM lanes a warp may read) and the 32 key
//     columns of quarter w/4.  A step of the eight-warp kernel is a serial chain of waits, loads,
//     arithmetic and stores per warp with two warps per scheduler; here each chain is half as
//     long and four warps per scheduler fill each other's gaps.
//   * The element-wise block stays in packed fp32 pairs from the scores to the exponent:
//     x = S*(scale*log2e) + (bias*log2e - lse*log2e) + mask, two fused multiply-adds and one add
//     per pair.  The residue mask is staged already multiplied by log2e as 0 (keep) or -inf
//     (drop): a dropped score becomes -inf and its P exactly 0, which is what exp(-FLT_MAX - lse)
//     gives in the reference (evoformer.py:69 replaces the score by the most negative float).
//     Rows whose every key is dropped carry the lse sentinel and take the uniform branch.
//   * 112 registers per compute thread: the d_bias accumulator of a thread is 32 floats, the
//     rest is worked through sixteen columns at a time.
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace evo {
namespace {

using namespace ptx;

constexpr int BT = 128;   // tile edge (queries and keys)
constexpr int DP = 32;    // padded head dimension
constexpr int G = 3;      // MSA rows per work item
constexpr int RB = DP * 2;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kThreads16 = 640;
constexpr int kComputeWarps = 16;

// Shared memory.  P and dS have one buffer each: the dV/dK/dQ MMAs of a step are issued the
// moment its last compute warp is done and have completed before the next step's first P/dS
// stores (which wait for them anyway).  That leaves room for the pair bias of a whole step (one
// block of 32 key columns per column quarter) and for two staging tiles from which the dQ partials
// leave as bulk tensor reductions.  Q, dO, K, V of a step arrive two steps ahead in a two-deep ring.
struct Smem16 {
  static constexpr int kTile = BT * RB;                   // one Q, dO, K or V tile
  static constexpr int kPS = BT * BT * 2;                 // the P or the dS tile
  static constexpr int kBiasBlock = BT * 128;             // 128 rows x 32 fp32, 128-byte swizzle
  static constexpr int kStage = 4 * kTile;                // Q, dO, K, V of one step
  static constexpr int kStages = 2;
  static constexpr int offStage = 0;
  static constexpr int offP = offStage + kStages * kStage;
  static constexpr int offDS = offP + kPS;
  static constexpr int offB = offDS + kPS;                // one block per column quarter
  static constexpr int kDQ = BT * DP * 4;                 // a dQ partial: 128 rows x 32 fp32, 128-byte swizzle
  static constexpr int offDQ = offB + 4 * kBiasBlock;     // 2 buffers
  static constexpr int offMask = offDQ + 2 * kDQ;         // G x 128 floats
  static constexpr int offBars = offMask + G * BT * 4;
  static constexpr size_t bytes = offBars + 256 + 1024;
};

struct StepId16 {
  int b, h, s, it, g, j0;
};

template <class T>
__global__ void __launch_bounds__(kThreads16, 1)
evo_bwd16_kernel(const Args a, float* __restrict__ dq_acc, const int n_items, const __grid_constant__ CUtensorMap tmQ,
                 const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmDB, const __grid_constant__ CUtensorMap tmDQ) {
  using L = Smem16;
  constexpr uint32_t SWZ = swizzle_code_for_row_bytes(RB);
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int QD = DP / 4;  // dQ / dK / dV columns handled by one column quarter
  constexpr int kTmemCols = 512;
  constexpr int colS = 0, colDP = BT, colDV = 2 * BT, colDK = 2 * BT + G * DP, colDQ = 2 * BT + 2 * G * DP;
  static_assert(colDQ + DP <= kTmemCols, "TMEM budget");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sP = smem + L::offP;
  uint8_t* sDS = smem + L::offDS;
  uint8_t* sB = smem + L::offB;
  uint8_t* sDQ = smem + L::offDQ;
  float* sMask = reinterpret_cast<float*>(smem + L::offMask);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBars);
  uint64_t* bar_ld = bars + 0;       // [2] tiles of a step landed
  uint64_t* bar_sdp = bars + 3;      // S, dP of a step complete
  uint64_t* bar_out = bars + 4;      // dV, dK, dQ MMAs of a step complete
  uint64_t* bar_bfull = bars + 5;    // [4 quarters] that quarter's pair-bias block (32 key columns) landed
  uint64_t* bar_bempty = bars + 13;  // [4 quarters] ... may be refilled (one arrival per warp): it has been read,
                                     // or, after a row group's last step, holds the quarter's d_bias values instead
  uint64_t* bar_sread = bars + 21;   // the 16 compute warps hold their S, dP columns of a step in registers
  uint64_t* bar_cdone = bars + 22;   // the 16 compute warps finished a step (P, dS written; dQ read)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 24);
  volatile uint32_t* scratch = reinterpret_cast<volatile uint32_t*>(bars + 25);  // written, never read

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = (a.R + BT - 1) / BT;
  const int NC = (a.S + G - 1) / G;
  const bool has_bias = a.bias != nullptr;
  const bool add_mask = a.mask_kind == EVOATTN_MASK_ADD_F32 || a.mask_kind == EVOATTN_MASK_ADD_SAME;
  // Persistent CTAs: CTA c owns the items c, c + gridDim.x, ... and walks them as one flat list of
  // steps, SPI per item.  A short last row group (S % G != 0) is padded with rows >= S: their
  // tiles arrive as zeros and their mask is -inf, so P = dS = 0, and nothing of them is stored.
  const int SPI = NT * G;
  const int my_items = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int total_steps = my_items * SPI;
  auto decode = [&](int N) {
    StepId16 d;
    const int k = N / SPI, n = N - k * SPI;
    d.it = n / G;
    d.g = n - d.it * G;
    int idx = (int)blockIdx.x + k * (int)gridDim.x;
    const int chunk = idx % NC; idx /= NC;
    d.j0 = (idx % NT) * BT; idx /= NT;
    d.h = idx % a.H;
    d.b = idx / a.H;
    d.s = chunk * G + d.g;
    return d;
  };
  // The residue mask of MSA row s, key j in two halves, so that the load can be issued long
  // before its value is needed: the raw element (0 where there is none to read) ...
  auto mask_fetch = [&](int b, int s, int j, bool wanted) -> uint32_t {
    const bool ok = wanted && s < a.S && j < a.R && a.mask_kind != EVOATTN_MASK_NONE;
    const long long mi = (long long)b * a.smask.a + (long long)s * a.smask.b + (long long)j * a.smask.c;
    if (a.mask_kind == EVOATTN_MASK_BOOL) return ldg_u8_if(reinterpret_cast<const unsigned char*>(a.mask) + mi, ok);
    if (a.mask_kind == EVOATTN_MASK_ADD_F32) return ldg_u32_if(reinterpret_cast<const uint32_t*>(a.mask) + mi, ok);
    return ldg_u16_if(reinterpret_cast<const uint16_t*>(a.mask) + mi, ok);
  };
  // ... and the float that is added to a score in the log2 domain: 0 keeps it, -inf drops it
  auto mask_decode = [&](uint32_t raw, int s, int j) -> float {
    const float ninf = __int_as_float(0xff800000);
    if (s >= a.S || j >= a.R) return ninf;
    if (a.mask_kind == EVOATTN_MASK_NONE) return 0.f;
    if (a.mask_kind == EVOATTN_MASK_BOOL) return raw ? 0.f : ninf;
    if (a.mask_kind == EVOATTN_MASK_ADD_F32) return __uint_as_float(raw) * kLog2e;
    const uint16_t h16 = (uint16_t)raw;
    return to_float<T>(*reinterpret_cast<const T*>(&h16)) * kLog2e;
  };

  if (tid == 0) *abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    for (int i = 0; i < L::kStages; ++i) mbar_init(bar_ld + i, 1);
    mbar_init(bar_sdp, 1);
    mbar_init(bar_out, 1);
    mbar_init(bar_cdone, kComputeWarps);  // one arrival per compute warp
    mbar_init(bar_sread, kComputeWarps);
    for (int i = 0; i < 4; ++i) { mbar_init(bar_bfull + i, 1); mbar_init(bar_bempty + i, 4); }
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
    if (has_bias) prefetch_tmap(&tmB);
    if (a.dbias != nullptr) prefetch_tmap(&tmDB);
    prefetch_tmap(&tmDQ);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  {
    const StepId16 d0 = decode(0);  // the first item's mask; later items are staged by the compute warps
    for (int t = tid; t < G * BT; t += kThreads16) {
      const int s = d0.s + t / BT, j = d0.j0 + (t % BT);
      sMask[t] = mask_decode(mask_fetch(d0.b, s, j, true), s, j);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  (void)add_mask;

  if (warp >= kComputeWarps) {
    setmaxnreg_dec<24>();
    if (warp == kComputeWarps) {
      const uint32_t leader = (lane == 0) ? 1u : 0u;  // the lane that issues; everything else is warp-uniform
      // =============================== control: TMA + MMA ===============================
      constexpr uint32_t kIdescS = make_idesc(kBf16, false, false, BT, BT);      // S, dP: K-major operands
      constexpr uint32_t kIdescT = make_idesc(kBf16, true, true, BT, DP);        // dV, dK: A = P^T / dS^T (MN-major)
      constexpr uint32_t kIdescQ = make_idesc(kBf16, false, true, BT, DP);       // dQ: A = dS K-major, B = K MN-major
      constexpr uint32_t kHiOp = static_cast<uint32_t>(make_sdesc_const(16, 8 * RB, SWZ) >> 32);
      constexpr uint32_t kHiPS = static_cast<uint32_t>(make_sdesc_const(16, 1024, SWZ_128B) >> 32);
      constexpr uint32_t kLoLbo = static_cast<uint32_t>(make_sdesc_const(16, 0, 0) & 0xffffffffu);
      constexpr uint32_t kLoLboT = static_cast<uint32_t>(make_sdesc_const(BT * 128, 0, 0) & 0xffffffffu);
      const uint32_t st_lo = smem_u32(smem + L::offStage) >> 4;
      const uint32_t p_lo0 = smem_u32(sP) >> 4, ds_lo0 = smem_u32(sDS) >> 4;

      // S and dP of step n: issued as soon as the compute warps hold the previous step's in
      // registers, which is about half a step before they need these.  (Issuing the two halves of
      // the key columns separately, each as soon as its warps are done, costs more than it gains:
      // an MMA takes about as long for 64 columns as for 128, and the issuing thread waits for it.)
      auto issue_s_dp = [&](int n) {
        const int buf = n % L::kStages;
        const uint32_t base = (st_lo + buf * (L::kStage >> 4)) | kLoLbo;
        const uint32_t qa = base, da = base + (L::kTile >> 4), ka = base + 2 * (L::kTile >> 4),
                       va = base + 3 * (L::kTile >> 4);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk)
          mma_ss_if(leader, tmem + colS, pack_desc(qa + kk * 2, kHiOp), pack_desc(ka + kk * 2, kHiOp), kIdescS, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk)
          mma_ss_if(leader, tmem + colDP, pack_desc(da + kk * 2, kHiOp), pack_desc(va + kk * 2, kHiOp), kIdescS, kk > 0 ? 1u : 0u);
        mma_commit_if(leader, bar_sdp);
      };
      auto issue_out = [&](int n) {
        const int buf = n % L::kStages, nn = n % SPI, g = nn % G;
        const uint32_t first = (nn < G) ? 0u : 1u;  // the item's first query tile overwrites the accumulators
        const uint32_t base = (st_lo + buf * (L::kStage >> 4)) | kLoLbo;
        const uint32_t qa = base, da = base + (L::kTile >> 4), ka = base + 2 * (L::kTile >> 4);
        const uint32_t p_lo = p_lo0, ds_lo = ds_lo0;
#ifndef EVO_OUT_INTERLEAVE
#define EVO_OUT_INTERLEAVE 1
#endif
#if EVO_OUT_INTERLEAVE
        // The three accumulators are independent chains: their MMAs are issued round-robin so that
        // an MMA never follows one it depends on.
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {
          // dV_j[s] += P^T dO_i : A = P read MN-major (M = j); K runs over the 128 query rows
          mma_ss_if(leader, tmem + colDV + g * DP, pack_desc((p_lo + kk * 128) | kLoLboT, kHiPS), pack_desc(da + kk * RB, kHiOp),
                    kIdescT, (kk > 0) ? 1u : first);
          // dK_j[s] += dS^T Q_i
          mma_ss_if(leader, tmem + colDK + g * DP, pack_desc((ds_lo + kk * 128) | kLoLboT, kHiPS), pack_desc(qa + kk * RB, kHiOp),
                    kIdescT, (kk > 0) ? 1u : first);
          // dQ_i[s] partial = dS K_j : A = dS K-major (K runs over the 128 keys)
          mma_ss_if(leader, tmem + colDQ, pack_desc((ds_lo + (kk >> 2) * (BT * 128 >> 4) + (kk & 3) * 2) | kLoLbo, kHiPS),
                    pack_desc(ka + kk * RB, kHiOp), kIdescQ, kk > 0 ? 1u : 0u);
        }
#else
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          mma_ss_if(leader, tmem + colDV + g * DP, pack_desc((p_lo + kk * 128) | kLoLboT, kHiPS), pack_desc(da + kk * RB, kHiOp),
                    kIdescT, (kk > 0) ? 1u : first);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          mma_ss_if(leader, tmem + colDK + g * DP, pack_desc((ds_lo + kk * 128) | kLoLboT, kHiPS), pack_desc(qa + kk * RB, kHiOp),
                    kIdescT, (kk > 0) ? 1u : first);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          mma_ss_if(leader, tmem + colDQ, pack_desc((ds_lo + (kk >> 2) * (BT * 128 >> 4) + (kk & 3) * 2) | kLoLbo, kHiPS),
                    pack_desc(ka + kk * RB, kHiOp), kIdescQ, kk > 0 ? 1u : 0u);
#endif
        mma_commit_if(leader, bar_out);
      };

      mbar_wait(bar_ld, 0, abort_flag, a.status, DEV_TIMEOUT_TMA);
      tc_fence_after();
      issue_s_dp(0);
      for (int n = 0; n < total_steps; ++n) {
        if (n + 1 < total_steps) {
          mbar_wait(bar_ld + (n + 1) % L::kStages, ((n + 1) / L::kStages) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
          mbar_wait(bar_sread, n & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
          tc_fence_after();
          issue_s_dp(n + 1);
        }
        const StepId16 dp = decode(n > 0 ? n - 1 : 0);  // before the wait: off the critical path
        mbar_wait(bar_cdone, n & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
        tc_fence_after();
        // The reduction issued one step ago has read its staging tile: placed before the commit
        // below, that is what lets the compute warps reuse the tile after their wait on bar_out.
        if (lane == 0) tma_wait_group_read0();
        issue_out(n);  // runs underneath step n+1's arithmetic
        // the dQ partial of step n-1, staged by the compute warps during step n
        if (n > 0 && dp.s < a.S && lane == 0) {
          tma_reduce_add_3d(&tmDQ, sDQ + (n & 1) * L::kDQ, 0, dp.it * BT, (dp.b * a.H + dp.h) * a.S + dp.s);
          tma_commit_group();
        }
        __syncwarp();
      }
      if (total_steps > 0) {
        // the last step's partial: staged after the loop, announced by one more round of arrivals
        const StepId16 dp = decode(total_steps - 1);
        mbar_wait(bar_cdone, total_steps & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
        if (lane == 0) {
          if (dp.s < a.S) {
            tma_reduce_add_3d(&tmDQ, sDQ + (total_steps & 1) * L::kDQ, 0, dp.it * BT, (dp.b * a.H + dp.h) * a.S + dp.s);
            tma_commit_group();
          }
          tma_wait_group0();
        }
        __syncwarp();
      }
    } else if (warp == kComputeWarps + 3) {
      // =============================== Q, dO, K, V loader ===============================
      // The tiles of a step arrive two steps ahead in a two-deep ring; the stage of step n is
      // free once the dV/dK/dQ MMAs of step n have completed.
      const uint32_t leader = (lane == 0) ? 1u : 0u;
      auto load_step = [&](int n, const StepId16& d) {
        const int buf = n % L::kStages;
        uint8_t* dst = smem + L::offStage + buf * L::kStage;
        mbar_expect_tx_if(leader, bar_ld + buf, L::kStage);
        tma_load_5d_if(leader, dst, &tmQ, bar_ld + buf, 0, d.it * BT, d.s, d.h, d.b);
        tma_load_5d_if(leader, dst + L::kTile, &tmDO, bar_ld + buf, 0, d.it * BT, d.s, d.h, d.b);
        tma_load_5d_if(leader, dst + 2 * L::kTile, &tmK, bar_ld + buf, 0, d.j0, d.s, d.h, d.b);
        tma_load_5d_if(leader, dst + 3 * L::kTile, &tmV, bar_ld + buf, 0, d.j0, d.s, d.h, d.b);
      };
      for (int n = 0; n < L::kStages && n < total_steps; ++n) load_step(n, decode(n));
      for (int n = 0; n + L::kStages < total_steps; ++n) {
        const StepId16 d = decode(n + L::kStages);  // before the wait: the divisions are off the critical path
        mbar_wait(bar_out, n & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
        load_step(n + L::kStages, d);
      }
    } else if (warp <= kComputeWarps + 2 && has_bias) {
      // ====== pair-bias loaders: warp 17 feeds column quarters 0 and 1, warp 18 quarters 2 and 3 ======
      // A quarter's buffer holds the bias of its 32 key columns for one step (rows of 128 bytes:
      // half as many rows for the copy engine as two 16-column chunks would be) and is refilled
      // as soon as the quarter's warps have read it, most of a step before it is needed again.
      // After the last step of a row group the compute warps hand the buffer back holding the
      // quarter's d_bias block instead of the bias they read from it: this warp then adds it to
      // d_bias in global memory with a bulk tensor reduction and refills the buffer once the
      // reduction has read it.
      const int q0 = (warp - kComputeWarps - 1) * 2;
      StepId16 pd = decode(0);
      bool prev_flush = false;
      for (int n = 0; n <= total_steps; ++n) {
        const bool load = n < total_steps;
        if (!load && !prev_flush) break;
        const StepId16 d = decode(load ? n : 0);
#pragma unroll
        for (int qq = 0; qq < 2; ++qq) {
          const int qd = q0 + qq;
          mbar_wait(bar_bempty + qd, (n & 1) ^ 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
          if (prev_flush && lane == 0) {
            tma_reduce_add_4d(&tmDB, sB + qd * L::kBiasBlock, pd.j0 + qd * 32, pd.it * BT, pd.h, pd.b);
            tma_commit_group();
            if (load) tma_wait_group_read0(); else tma_wait_group0();
          }
          __syncwarp();
          if (load && lane == 0) {
            mbar_expect_tx(bar_bfull + qd, L::kBiasBlock);
            tma_load_4d(sB + qd * L::kBiasBlock, &tmB, bar_bfull + qd, d.j0 + qd * 32, d.it * BT, d.h, d.b);
          }
          __syncwarp();
        }
        prev_flush = load && (d.g == G - 1) && (a.dbias != nullptr);
        pd = d;
      }
      // every reduction of this warp has completed before the CTA may exit
      if (lane == 0) tma_wait_group0();
    }
  } else {
    // =============================== compute warps ===============================
    setmaxnreg_inc<112>();
    const int qd = warp >> 2;    // column quarter: key columns qd*32 .. qd*32+31 of the tile
    const int half = qd >> 1;    // the half of S / dP (and of the P / dS tiles) those columns lie in
    const int row = (warp & 3) * 32 + lane;
    const uint32_t t_lane = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float scale = a.scale;
    const float inv_r = 1.f / (float)a.R;
    const F2 c2 = f2_make(scale * kLog2e, scale * kLog2e), l2e2 = f2_make(kLog2e, kLog2e);

    // The dQ partial of step n-1 (its MMAs ran underneath step n's loads and arithmetic) leaves
    // TMEM during step n: this quarter's 8 columns of every row go into the staging tile of step n
    // (128-byte-swizzled rows), and the control warp adds the tile to the fp32 accumulator in
    // global memory with one bulk tensor reduction once every warp has finished step n.  Plain
    // reductions from registers (16 bytes per row and instruction) drain at half the rate and,
    // worse, hold up every later global access of the warp while they do.
    auto stage_dq = [&](int n) {  // n = the step during which the partial is staged
      uint32_t qr[QD];
      tmem_ld<QD>(t_lane + colDQ + qd * QD, qr);
      tmem_wait_ld();
      uint8_t* dst = sDQ + (n & 1) * L::kDQ + row * 128;
#pragma unroll
      for (int c = 0; c < QD / 4; ++c)
        *reinterpret_cast<uint4*>(dst + (((qd * (QD / 4) + c) ^ (row & 7)) << 4)) =
            make_uint4(qr[c * 4], qr[c * 4 + 1], qr[c * 4 + 2], qr[c * 4 + 3]);
    };

    // dK, dV of row-group slot g (MSA row s of (b,h), keys j0..): TMEM -> registers -> global
    auto drain_dkdv = [&](int b, int h, int s, int j0, int g) {
      const int j = j0 + row;
      uint32_t kr[QD], vr[QD];
      tmem_ld<QD>(t_lane + colDK + g * DP + qd * QD, kr);
      tmem_ld<QD>(t_lane + colDV + g * DP + qd * QD, vr);
      tmem_wait_ld();
      if (j < a.R && s < a.S && qd * QD < a.D) {
        T* kd = reinterpret_cast<T*>(a.dk) + off4(a.sdk, b, h, s, j) + qd * QD;
        T* vd = reinterpret_cast<T*>(a.dv) + off4(a.sdv, b, h, s, j) + qd * QD;
        uint4 pk, pv;
        pk.x = Pack2<T>::pack(__uint_as_float(kr[0]) * scale, __uint_as_float(kr[1]) * scale);
        pk.y = Pack2<T>::pack(__uint_as_float(kr[2]) * scale, __uint_as_float(kr[3]) * scale);
        pk.z = Pack2<T>::pack(__uint_as_float(kr[4]) * scale, __uint_as_float(kr[5]) * scale);
        pk.w = Pack2<T>::pack(__uint_as_float(kr[6]) * scale, __uint_as_float(kr[7]) * scale);
        pv.x = Pack2<T>::pack(__uint_as_float(vr[0]), __uint_as_float(vr[1]));
        pv.y = Pack2<T>::pack(__uint_as_float(vr[2]), __uint_as_float(vr[3]));
        pv.z = Pack2<T>::pack(__uint_as_float(vr[4]), __uint_as_float(vr[5]));
        pv.w = Pack2<T>::pack(__uint_as_float(vr[6]), __uint_as_float(vr[7]));
        *reinterpret_cast<uint4*>(kd) = pk;
        *reinterpret_cast<uint4*>(vd) = pv;
      }
    };

    // log-sum-exp and delta of this thread's query row for a step (rows that do not exist get a
    // huge lse so that their P is exactly 0)
    float lse_next = 1e30f, delta_next = 0.f;
    // `slab` = index of the [R] row of (b, h, row-group start) in the [B,H,S,R] statistics: the
    // 64-bit index arithmetic is done once per item, a step adds small offsets to it
    long long slab = 0;
    auto set_slab = [&](const StepId16& d) { slab = (((long long)d.b * a.H + d.h) * a.S + (d.s - d.g)) * a.R; };
    auto load_row_stats = [&](const StepId16& d, bool in_range) {
      const int i = d.it * BT + row;
      const bool ok = in_range && i < a.R && d.s < a.S;
      const long long ri = slab + d.g * a.R + i;
      lse_next = ldg_f32_if(a.lse + ri, ok, 1e30f);
      delta_next = ldg_f32_if(a.delta + ri, ok, 0.f);
    };
    // The compute warps step their position instead of decoding it: the divisions of `decode` are a
    // dependent chain of several hundred cycles, paid only when an item ends.
    StepId16 cur = decode(0);
    auto advance = [&](const StepId16& c, int n) {  // position of step n = the one after c
      StepId16 d = c;
      if (++d.g == G) {
        d.g = 0;
        if (++d.it == NT) return decode(n);
      }
      d.s = c.s - c.g + d.g;
      return d;
    };
    set_slab(cur);
    load_row_stats(cur, total_steps > 0);
    int pb = 0, ph = 0, ps0 = 0, pj0 = 0;     // the item whose dK/dV still sit in TMEM
    float bacc[32];
    bool out_seen = true;  // the dV/dK/dQ MMAs of the previous step are known to have completed

    for (int step = 0; step < total_steps; ++step) {
      const StepId16 nxt = advance(cur, step + 1);
      const bool more = step + 1 < total_steps;
      const bool item_ends = (cur.it == NT - 1) && (cur.g == G - 1);
      const int g = cur.g;
      const int j0 = cur.j0;
      if (g == 0) {
#pragma unroll
        for (int e = 0; e < 32; ++e) bacc[e] = 0.f;
      }
      // Fetched during the previous step.  They are pinned in registers before the next fetch is
      // issued: the same load instruction reuses its scoreboard slot, and a wait for the old value
      // placed after the new load would wait for the new one as well.
      float lse = lse_next, delta = delta_next;
      asm volatile("" : "+f"(lse), "+f"(delta)::"memory");
      // the next item's residue mask, fetched under this item's last step (G*128 = 384 values)
      uint32_t mnext = 0u;
      if (item_ends) {  // warp-uniform: the index arithmetic is skipped on the other steps
        set_slab(nxt);
        mnext = mask_fetch(nxt.b, nxt.s + tid / BT, nxt.j0 + (tid % BT), more && tid < G * BT);
      }
      load_row_stats(nxt, more);  // in flight during this step
      const bool dead = (lse == -FLT_MAX);  // every key of this row was dropped: P is uniform
      const float nlse = -lse * kLog2e;
      const F2 nlse2 = f2_make(nlse, nlse), delta2 = f2_make(delta, delta);
      mbar_wait(bar_sdp, step & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
      tc_fence_after();

      const bool flush = (g == G - 1) && a.dbias != nullptr;  // the row group's last step: d_bias leaves
      uint8_t* prow = sP + half * (BT * 128) + row * 128;
      uint8_t* drow = sDS + half * (BT * 128) + row * 128;
      out_seen = (step == 0);
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        const int col0 = qd * 32 + sub * 16;
        uint32_t sr[16], dr[16];
        tmem_ld16(t_lane + colS + col0, sr);
        tmem_ld16(t_lane + colDP + col0, dr);
        // pair bias: 16 of my row's 32 floats (rows of 128 bytes, 128-byte swizzle)
        float bv[16];
        uint8_t* brow = sB + qd * L::kBiasBlock + row * 128;
        if (has_bias) {
          if (sub == 0) mbar_wait(bar_bfull + qd, step & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const float4 f = *reinterpret_cast<const float4*>(brow + (((sub * 4 + q4) ^ (row & 7)) << 4));
            bv[q4 * 4 + 0] = f.x; bv[q4 * 4 + 1] = f.y; bv[q4 * 4 + 2] = f.z; bv[q4 * 4 + 3] = f.w;
          }
          if (!flush && sub == 1) {
            // The buffer is handed back only after the loads from it have returned: a store that
            // needs one word of each of this block's loads is issued first, and the first block's
            // values have been used by then (an mbarrier arrival does not wait for shared loads
            // still queued, and the refill would overwrite what they are about to read).
            *scratch = __float_as_uint(bv[0]) ^ __float_as_uint(bv[4]) ^ __float_as_uint(bv[8]) ^ __float_as_uint(bv[12]);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_bempty + qd);  // one arrival per warp
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) bv[e] = 0.f;
        }
        tmem_wait_ld();
        if (sub == 1) {  // this warp holds its S, dP columns in registers: the next step's may be issued
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_sread);
        }
        const float* mrow = sMask + g * BT + col0;
        float p[16], ds[16];
        if (!dead) {
#pragma unroll
          for (int u = 0; u < 16; u += 4) {
            const float4 mk = *reinterpret_cast<const float4*>(mrow + u);
            // x = S*(scale*log2e) + (bias*log2e - lse*log2e) + mask, in packed pairs
            F2 t0 = f2_add(f2_fma(f2_make(bv[u], bv[u + 1]), l2e2, nlse2), f2_make(mk.x, mk.y));
            F2 t1 = f2_add(f2_fma(f2_make(bv[u + 2], bv[u + 3]), l2e2, nlse2), f2_make(mk.z, mk.w));
            float x0, x1, x2, x3;
            f2_get(f2_fma(f2_from_bits(sr[u], sr[u + 1]), c2, t0), x0, x1);
            f2_get(f2_fma(f2_from_bits(sr[u + 2], sr[u + 3]), c2, t1), x2, x3);
            p[u] = ex2(x0); p[u + 1] = ex2(x1); p[u + 2] = ex2(x2); p[u + 3] = ex2(x3);
          }
#pragma unroll
          for (int u = 0; u < 16; u += 2) {  // dS = P (dP - delta); d_bias_acc += dS
            const F2 t = f2_mul(f2_make(p[u], p[u + 1]), f2_sub(f2_from_bits(dr[u], dr[u + 1]), delta2));
            f2_get(t, ds[u], ds[u + 1]);
            f2_get(f2_add(f2_make(bacc[sub * 16 + u], bacc[sub * 16 + u + 1]), t), bacc[sub * 16 + u],
                   bacc[sub * 16 + u + 1]);
          }
        } else {
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            p[u] = (j0 + col0 + u < a.R) ? inv_r : 0.f;
            ds[u] = 0.f;  // replaced scores are constants: no gradient flows through them
          }
        }
        if (flush && has_bias) {
          // These 16 columns of the quarter's d_bias block are final: they go where their bias
          // values were (same rows, same swizzle); after the second block the buffer goes back to
          // the loader warp, which adds it to d_bias in global memory before it refills it.
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<float4*>(brow + (((sub * 4 + q4) ^ (row & 7)) << 4)) =
                make_float4(bacc[sub * 16 + q4 * 4], bacc[sub * 16 + q4 * 4 + 1], bacc[sub * 16 + q4 * 4 + 2],
                            bacc[sub * 16 + q4 * 4 + 3]);
          if (sub == 1) {
            fence_async_shared();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_bempty + qd);
          }
        }
        if (!out_seen) {
          // P and dS have one buffer each: the previous step's dV/dK/dQ MMAs must have read them.
          // They were issued when that step's last warp finished and ran underneath this step's
          // loads and arithmetic.
          mbar_wait(bar_out, (step - 1) & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
          tc_fence_after();
          out_seen = true;
          stage_dq(step);  // and their dQ partial leaves TMEM
        }
#pragma unroll
        for (int c8 = 0; c8 < 2; ++c8) {
          uint4 pk, dk;
          pk.x = Pack2<T>::pack(p[c8 * 8 + 0], p[c8 * 8 + 1]); pk.y = Pack2<T>::pack(p[c8 * 8 + 2], p[c8 * 8 + 3]);
          pk.z = Pack2<T>::pack(p[c8 * 8 + 4], p[c8 * 8 + 5]); pk.w = Pack2<T>::pack(p[c8 * 8 + 6], p[c8 * 8 + 7]);
          dk.x = Pack2<T>::pack(ds[c8 * 8 + 0], ds[c8 * 8 + 1]); dk.y = Pack2<T>::pack(ds[c8 * 8 + 2], ds[c8 * 8 + 3]);
          dk.z = Pack2<T>::pack(ds[c8 * 8 + 4], ds[c8 * 8 + 5]); dk.w = Pack2<T>::pack(ds[c8 * 8 + 6], ds[c8 * 8 + 7]);
          const int chunk16 = (((qd & 1) * 4 + sub * 2 + c8) ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(prow + chunk16) = pk;
          *reinterpret_cast<uint4*>(drow + chunk16) = dk;
        }
      }
      // dK/dV of the previous item's slot g: complete (the wait above covers every earlier MMA),
      // and about to be overwritten by this step's MMAs
      if (cur.it == 0 && step >= SPI) drain_dkdv(pb, ph, ps0 + g, pj0, g);
      tc_fence_before();
      fence_async_shared();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_cdone);  // P, dS of this step are in shared memory; dQ has been read
      if (item_ends) {
        pb = cur.b; ph = cur.h; ps0 = cur.s - g; pj0 = j0;
        if (more) {
          named_bar_sync(7, kComputeWarps * 32);  // every compute warp has read this item's mask for the last time
          if (tid < G * BT) sMask[tid] = mask_decode(mnext, nxt.s + tid / BT, nxt.j0 + (tid % BT));
          named_bar_sync(7, kComputeWarps * 32);
        }
      }
      cur = nxt;
    }

    if (total_steps > 0) {
      mbar_wait(bar_out, (total_steps - 1) & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);  // every MMA of this CTA has completed
      tc_fence_after();
      stage_dq(total_steps);
      fence_async_shared();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_cdone);  // the control warp sends the last partial off
      for (int g = 0; g < G; ++g) drain_dkdv(pb, ph, ps0 + g, pj0, g);
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

}  // namespace

// The sixteen-warp kernel on the work list of `items` items (tensor maps and the fp32 dQ
// accumulator are those the caller built for the eight-warp kernel).
int launch_sm100_bwd16(int dtype, const Args& a, float* dq_acc, long long items, int ctas, const CUtensorMap& tq,
                       const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tb,
                       const CUtensorMap& tdb, cudaStream_t st) {
  CUtensorMap tdq;
  if (!make_rows_f32_map(&tdq, dq_acc, a.D, a.R, (long long)a.B * a.H * a.S, DP, BT)) return EVOATTN_ERR_CUDA;
  if (dtype == EVOATTN_BF16) {
    auto kern = evo_bwd16_kernel<__nv_bfloat16>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem16::bytes) != cudaSuccess)
      return EVOATTN_ERR_CUDA;
    kern<<<(unsigned)ctas, kThreads16, Smem16::bytes, st>>>(a, dq_acc, (int)items, tq, tk, tv, tdo, tb, tdb, tdq);
  } else {
    auto kern = evo_bwd16_kernel<__half>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem16::bytes) != cudaSuccess)
      return EVOATTN_ERR_CUDA;
    kern<<<(unsigned)ctas, kThreads16, Smem16::bytes, st>>>(a, dq_acc, (int)items, tq, tk, tv, tdo, tb, tdb, tdq);
  }
  return EVOATTN_OK;
}

}  // namespace evo
