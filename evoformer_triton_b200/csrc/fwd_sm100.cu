// Evoformer attention forward for sm_100a: TMA-staged tiles, tcgen05 MMAs with the
// accumulators in TMEM, online softmax with pair bias and residue mask in registers.
//
// Computes what dsevoformer-triton/evoformer.py:23-100 (_attn_fwd_inner) and :103-297
// (_attn_fwd) compute:  O = softmax(scale*Q K^T + bias, masked) V  and the row
// log-sum-exp, without ever writing the R x R scores to memory.
//
// Persistent, warp-specialised kernel, one CTA per SM, 384 threads:
//   warp 0      TMA producer: Q tiles, K/V tiles (64 keys each) and pair-bias tiles
//   warp 1, 2   issue the tcgen05.mma of warpgroup A, B
//   warp 3      stages the residue-mask rows of the next item in shared memory
//   warps 4-7   softmax warpgroup A        warps 8-11   softmax warpgroup B
// A work item is one 128-row query tile of TWO consecutive MSA rows s of one (b,h):
// warpgroup A takes row 2p, B takes row 2p+1.  Both rows use the same pair-bias tile, so
// it is staged in shared memory once per item pair.  Inside a warpgroup thread t owns
// score row t (= TMEM lane t) and all 64 columns of the current key tile, so the row
// maximum and sum need no exchange between threads.
//
// With a single MSA row (N_seq = 1, the shape of the reference's own benchmark sweep) there is no
// second row to pair: the kernel is then instantiated in query-pair mode, where an item is two
// consecutive query tiles of the same row, the warpgroups share one K/V ring and each has its own
// pair-bias tile in a stage.
//
// Per warpgroup and key tile n:  S_n = Q K_n^T lands in TMEM (double buffered); the
// warpgroup turns it into P_n (rounded to the storage type as evoformer.py:84 does) and
// writes it back over S_n in TMEM, from where it feeds the P V MMA as the A operand;
// P_n V_n lands in a second TMEM double buffer and is folded into the
// fp32 output accumulator in registers one tile later, scaled by the softmax correction
// of that tile.  The MMA warp runs S_{n+1} while the warpgroup is busy with tile n.
#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace evo {
namespace {

using namespace ptx;

constexpr int BM = 128;  // query rows per warpgroup tile
constexpr int BN = 64;   // keys per tile
constexpr int kThreads = 384;
constexpr int kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int MASK_MIN = 0;  // boolean keep-mask (or none): score = min(score, m), m = +-FLT_MAX
constexpr int MASK_ADD = 1;  // additive mask

template <int DP, bool QP>
struct Cfg {
  static constexpr int RB = DP * 2;                    // bytes per staged row
  static constexpr int QST = (DP == 64) ? 1 : 2;       // Q stages per warpgroup
  static constexpr int NKV = (DP == 64) ? 2 : 4;       // K and V ring depth per warpgroup
  static constexpr int BST = 2;                        // pair-bias stages (shared by both warpgroups)
  static constexpr int KVW = QP ? 1 : 2;               // K/V rings: one per warpgroup, or one shared (query-pair mode)
  static constexpr int BTL = QP ? 2 : 1;               // pair-bias tiles per stage: one shared, or one per warpgroup
  static constexpr int kQ = BM * RB;
  static constexpr int kKV = BN * RB;
  static constexpr int kBias = BM * BN * 4;            // 32 KB = two 128x32 fp32 boxes
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + 2 * QST * kQ;
  static constexpr int offV = offK + KVW * NKV * kKV;
  static constexpr int offB = offV + KVW * NKV * kKV;
  static constexpr int offMask = offB + BST * BTL * kBias;
  static constexpr int kNumBars = 2 * (2 * QST + 4 * NKV + 2 + 1 + 2 + 4) + 2 * BST;
  static size_t bytes(int r_pad) {
    return (size_t)offMask + (size_t)4 * r_pad * 4 + 4 * 32 * 4 + kNumBars * 8 + 64 + 1024;
  }
  // TMEM columns of warpgroup w: S double buffer, then PV double buffer
  static constexpr int tmemWg = 2 * BN + 2 * DP;
};

// A work item: warpgroup w works on query tile qt[w] of MSA row s[w] of (b, h).  Row-pair mode: rows
// 2p and 2p+1, the same query tile; query-pair mode: one row, query tiles 2p and 2p+1.
struct Item {
  int b, h, qt[2], s[2];
};
template <bool QP>
__device__ __forceinline__ Item decode_item(int idx, int n_inner, int n_outer, int H) {
  Item it;
  const int inner = idx % n_inner; idx /= n_inner;   // row pair (row-pair mode) or row (query-pair mode)
  const int outer = idx % n_outer; idx /= n_outer;   // query tile, or pair of query tiles
  it.h = idx % H;
  it.b = idx / H;
  if (QP) {
    it.s[0] = it.s[1] = inner;
    it.qt[0] = 2 * outer; it.qt[1] = 2 * outer + 1;
  } else {
    it.s[0] = 2 * inner; it.s[1] = 2 * inner + 1;
    it.qt[0] = it.qt[1] = outer;
  }
  return it;
}

template <class T, int DP, int MASKMODE, bool BIAS16, bool QP>
__global__ void __launch_bounds__(kThreads, 1)
evo_fwd_sm100_kernel(const Args a, const int n_items, const __grid_constant__ CUtensorMap tmQ,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmB) {
  using C = Cfg<DP, QP>;
  constexpr int RB = C::RB, QST = C::QST, NKV = C::NKV, BST = C::BST;
  constexpr uint32_t SWZ = swizzle_code_for_row_bytes(RB);
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int T_TILES = (a.R + BN - 1) / BN;
  const int r_pad = T_TILES * BN;
  float* sMask = reinterpret_cast<float*>(smem + C::offMask);  // [warpgroup][stage][r_pad]
  // one word per key tile of a staged mask row: non-zero if the tile has a dropped key (a key tile
  // without one skips the mask arithmetic and the mask loads in the boolean form); R <= 2048
  uint32_t* sDirty = reinterpret_cast<uint32_t*>(sMask + 4 * r_pad);  // [warpgroup][stage][32]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDirty + 4 * 32);
  // barrier layout: per warpgroup w a block of PER, then the shared bias barriers
  constexpr int PER = 2 * QST + 4 * NKV + 2 + 1 + 2 + 4;
  auto q_full = [&](int w, int st) { return bars + w * PER + st; };
  auto q_empty = [&](int w, int st) { return bars + w * PER + QST + st; };
  auto k_full = [&](int w, int st) { return bars + w * PER + 2 * QST + st; };
  auto k_empty = [&](int w, int st) { return bars + w * PER + 2 * QST + NKV + st; };
  auto v_full = [&](int w, int st) { return bars + w * PER + 2 * QST + 2 * NKV + st; };
  auto v_empty = [&](int w, int st) { return bars + w * PER + 2 * QST + 3 * NKV + st; };
  auto s_full = [&](int w, int i) { return bars + w * PER + 2 * QST + 4 * NKV + i; };
  auto p_full = [&](int w) { return bars + w * PER + 2 * QST + 4 * NKV + 2; };
  auto o_full = [&](int w, int i) { return bars + w * PER + 2 * QST + 4 * NKV + 3 + i; };
  auto m_full = [&](int w, int st) { return bars + w * PER + 2 * QST + 4 * NKV + 5 + st; };
  auto m_empty = [&](int w, int st) { return bars + w * PER + 2 * QST + 4 * NKV + 7 + st; };
  auto b_full = [&](int st) { return bars + 2 * PER + st; };
  auto b_empty = [&](int st) { return bars + 2 * PER + BST + st; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + C::kNumBars + 1);
  volatile uint32_t* scratch = reinterpret_cast<volatile uint32_t*>(bars + C::kNumBars + 2);  // written, never read

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NQT = (a.R + BM - 1) / BM;
  // items: (b, h, outer, inner) with inner fastest
  const int n_inner = QP ? a.S : (a.S + 1) / 2;
  const int n_outer = QP ? (NQT + 1) / 2 : NQT;
  const bool has_bias = a.bias != nullptr;

  // A launch that follows a failed one returns at once (one reader, so the CTA agrees).
  if (tid == 0) *abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    for (int w = 0; w < 2; ++w) {
      for (int st = 0; st < QST; ++st) { mbar_init(q_full(w, st), 1); mbar_init(q_empty(w, st), 1); }
      for (int st = 0; st < NKV; ++st) {  // (query-pair mode: both issuers release the one shared ring)
        mbar_init(k_full(w, st), 1); mbar_init(k_empty(w, st), QP ? 2 : 1);
        mbar_init(v_full(w, st), 1); mbar_init(v_empty(w, st), QP ? 2 : 1);
      }
      mbar_init(s_full(w, 0), 1); mbar_init(s_full(w, 1), 1);
      mbar_init(p_full(w), 4);  // one arrival per softmax warp
      mbar_init(o_full(w, 0), 1); mbar_init(o_full(w, 1), 1);
      for (int st = 0; st < 2; ++st) { mbar_init(m_full(w, st), 1); mbar_init(m_empty(w, st), 4); }
    }
    for (int st = 0; st < BST; ++st) { mbar_init(b_full(st), 1); mbar_init(b_empty(st), 8); }
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
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

  if (warp < 4) {
    setmaxnreg_dec<40>();
    if (warp == 0 && lane == 0) {
      // =============================== TMA producer ===============================
      uint32_t qn[2] = {0, 0}, gt = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const Item it = decode_item<QP>(item, n_inner, n_outer, a.H);
        int srow[2];
        srow[0] = min(it.s[0], a.S - 1);
        srow[1] = min(it.s[1], a.S - 1);
        for (int w = 0; w < 2; ++w) {  // (a query tile beyond the last one loads as zeros)
          const int st = qn[w] % QST;
          mbar_wait(q_empty(w, st), ((qn[w] / QST) & 1) ^ 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
          mbar_expect_tx(q_full(w, st), C::kQ);
          tma_load_5d(smem + C::offQ + (w * QST + st) * C::kQ, &tmQ, q_full(w, st), 0, it.qt[w] * BM, srow[w], it.h, it.b);
          ++qn[w];
        }
        for (int t = 0; t < T_TILES; ++t, ++gt) {
          const int st = gt % NKV;
          const uint32_t par = ((gt / NKV) & 1) ^ 1;
          for (int w = 0; w < C::KVW; ++w) {
            mbar_wait(k_empty(w, st), par, abort_flag, a.status, DEV_TIMEOUT_SYNC);
            mbar_expect_tx(k_full(w, st), C::kKV);
            tma_load_5d(smem + C::offK + (w * NKV + st) * C::kKV, &tmK, k_full(w, st), 0, t * BN, srow[w], it.h, it.b);
          }
          if (has_bias) {
            const int bs = gt % BST;
            mbar_wait(b_empty(bs), ((gt / BST) & 1) ^ 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
            mbar_expect_tx(b_full(bs), C::BTL * (BIAS16 ? C::kBias / 2 : C::kBias));
            for (int u = 0; u < C::BTL; ++u) {  // one tile for both warpgroups, or one each
              uint8_t* dst = smem + C::offB + (bs * C::BTL + u) * C::kBias;
              if constexpr (BIAS16) {  // one box of 128 rows x 64 16-bit values (rows of 128 bytes)
                tma_load_4d(dst, &tmB, b_full(bs), t * BN, it.qt[u] * BM, it.h, it.b);
              } else {                 // two boxes of 128 rows x 32 floats
                tma_load_4d(dst, &tmB, b_full(bs), t * BN, it.qt[u] * BM, it.h, it.b);
                tma_load_4d(dst + C::kBias / 2, &tmB, b_full(bs), t * BN + 32, it.qt[u] * BM, it.h, it.b);
              }
            }
          }
          for (int w = 0; w < C::KVW; ++w) {
            mbar_wait(v_empty(w, st), par, abort_flag, a.status, DEV_TIMEOUT_SYNC);
            mbar_expect_tx(v_full(w, st), C::kKV);
            tma_load_5d(smem + C::offV + (w * NKV + st) * C::kKV, &tmV, v_full(w, st), 0, t * BN, srow[w], it.h, it.b);
          }
        }
      }
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // =============================== MMA issuer of warpgroup w ===============================
      const int w = warp - 1;
      constexpr uint32_t kIdescS = make_idesc(kBf16, false, false, BM, BN);
      constexpr uint32_t kIdescO = make_idesc(kBf16, false, true, BM, DP);
      // Descriptor halves that never change: the high word holds the stride offset, version and
      // swizzle; the low word is (address >> 4) plus the leading-offset field.
      constexpr uint32_t kHiOp = static_cast<uint32_t>(make_sdesc_const(16, 8 * RB, SWZ) >> 32);
      constexpr uint32_t kLoLbo = static_cast<uint32_t>(make_sdesc_const(16, 0, 0) & 0xffffffffu);
      const uint32_t q_lo0 = (smem_u32(smem + C::offQ + w * QST * C::kQ) >> 4) | kLoLbo;
      const int kw = QP ? 0 : w;  // the K/V ring this warpgroup reads
      const uint32_t k_lo0 = (smem_u32(smem + C::offK + kw * NKV * C::kKV) >> 4) | kLoLbo;
      const uint32_t v_lo0 = (smem_u32(smem + C::offV + kw * NKV * C::kKV) >> 4) | kLoLbo;
      const uint32_t tS = tmem + w * C::tmemWg, tO = tS + 2 * BN;
      uint32_t qn = 0, base = 0;  // items done, key tiles done
      auto issue_s = [&](uint32_t g) {  // g: running key-tile index
        const int st = g % NKV;
        mbar_wait(k_full(kw, st), (g / NKV) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
        tc_fence_after();
        const uint32_t qa = q_lo0 + (qn % QST) * (C::kQ >> 4);
        const uint32_t ka = k_lo0 + st * (C::kKV >> 4);
#pragma unroll
        for (int kk = 0; kk < DP / 16; ++kk)
          mma_ss(tS + (g & 1) * BN, pack_desc(qa + kk * 2, kHiOp), pack_desc(ka + kk * 2, kHiOp), kIdescS,
                 kk > 0 ? 1u : 0u);
        mma_commit(k_empty(kw, st));
        mma_commit(s_full(w, g & 1));
      };
      auto issue_pv = [&](uint32_t g) {
        const int st = g % NKV;
        mbar_wait(v_full(kw, st), (g / NKV) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
        mbar_wait(p_full(w), g & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
        tc_fence_after();
        const uint32_t va = v_lo0 + st * (C::kKV >> 4);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)  // 16 keys = 8 packed columns of P per step
          mma_ts(tO + (g & 1) * DP, tS + (g & 1) * BN + kk * 8, pack_desc(va + kk * RB, kHiOp), kIdescO,
                 kk > 0 ? 1u : 0u);
        mma_commit(v_empty(kw, st));
        mma_commit(o_full(w, g & 1));
      };
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        mbar_wait(q_full(w, qn % QST), (qn / QST) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
        for (int t = 0; t < 2 && t < T_TILES; ++t) issue_s(base + t);
        for (int t = 0; t < T_TILES; ++t) {
          issue_pv(base + t);
          if (t + 2 < T_TILES) issue_s(base + t + 2);  // S buffer (t&1) was read before P_t was signalled
        }
        mma_commit(q_empty(w, qn % QST));
        ++qn;
        base += T_TILES;
      }
    } else if (warp == 3) {
      // =============================== residue-mask stager ===============================
      // One float per key for each warpgroup's MSA row, one item ahead of the softmax warps.
      // Keys beyond R are always excluded.
      uint32_t n = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n) {
        const Item it = decode_item<QP>(item, n_inner, n_outer, a.H);
        const int st = n & 1;
        for (int w = 0; w < 2; ++w) {
          const int s = min(it.s[w], a.S - 1);
          mbar_wait(m_empty(w, st), ((n >> 1) & 1) ^ 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
          float* dst = sMask + (w * 2 + st) * r_pad;
          uint32_t* dirty = sDirty + (w * 2 + st) * 32;
          dirty[lane] = 0u;
          __syncwarp();
          // eight loads in flight per lane: a dependent load-convert-store chain per key would
          // make this warp the slowest stage of the pipeline
          for (int j0 = 0; j0 < r_pad; j0 += 256) {
            float m[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) m[u] = mask_value<T, MASKMODE == MASK_MIN>(a, it.b, s, j0 + u * 32 + lane);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const bool in = j0 + u * 32 + lane < r_pad;
              if (in) dst[j0 + u * 32 + lane] = m[u];
              const uint32_t any = __ballot_sync(0xffffffffu, in && m[u] < 0.f);
              if (lane == 0 && any != 0u) dirty[(j0 + u * 32) / BN] = 1u;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(m_full(w, st));
        }
      }
    }
  } else {
    // =============================== softmax warpgroups ===============================
    setmaxnreg_inc<232>();
    const int w = (warp >> 2) - 1;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t t_base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + w * C::tmemWg;
    const float scale = a.scale;
    const F2 scale2 = f2_make(scale, scale);
    uint32_t g = 0, n_item = 0;  // running key-tile and item index
    // The two warpgroups take turns in the exponential phase (named barriers 1 and 2 pass a
    // token back and forth): while one keeps the MUFU busy, the other runs its load / bias /
    // mask / max phase on the FMA, ALU and shared-memory pipes instead of both queueing on
    // the same unit.
    if (w == 1) named_bar_arrive(1, 256);

    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_item) {
      const Item it = decode_item<QP>(item, n_inner, n_outer, a.H);
      const int s_raw = it.s[w];
      const bool active = s_raw < a.S && it.qt[w] < NQT;
      const int s = s_raw < a.S ? s_raw : a.S - 1;
      const int i = it.qt[w] * BM + row;

      // residue-mask row of (b, s), staged by warp 3
      const uint32_t mst = n_item & 1;
      mbar_wait(m_full(w, mst), (n_item >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_SYNC);
      const float* mrow_base = sMask + (w * 2 + mst) * r_pad;
      const uint32_t* dirty_row = sDirty + (w * 2 + mst) * 32;

      float m_run = -FLT_MAX, l_run = 0.f, alpha_pending = 1.f;
      float acc[DP];
#pragma unroll
      for (int d = 0; d < DP; ++d) acc[d] = 0.f;

      for (int t = 0; t < T_TILES; ++t, ++g) {
        mbar_wait(s_full(w, g & 1), (g >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
        tc_fence_after();
        if (has_bias) mbar_wait(b_full(g % BST), (g / BST) & 1, abort_flag, a.status, DEV_TIMEOUT_TMA);
        const uint8_t* bstage = smem + C::offB + ((g % BST) * C::BTL + (QP ? w : 0)) * C::kBias + row * 128;
        const float* mrow = mrow_base + t * BN;

        // scores of my row: x = scale*S + bias, then the mask.  Written in groups of eight
        // independent elements (loads, FMAs, mins, then eight separate max chains) so that the
        // in-order issue never waits on the previous instruction's result.
        float x[BN];
        float mx8[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) mx8[u] = -FLT_MAX;
        uint32_t sr[BN];
        tmem_ld32(t_base + (g & 1) * BN, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
        tmem_ld32(t_base + (g & 1) * BN + 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
        tmem_wait_ld();
        // A key tile of a boolean mask without a dropped key needs neither the mask values nor
        // the `min` (most tiles: masks are mostly trailing padding); the flag is warp-uniform.
        auto scores = [&](auto with_mask) {
          constexpr bool kMask = decltype(with_mask)::value;
#pragma unroll
          for (int g8 = 0; g8 < BN / 8; ++g8) {
            const int c = g8 >> 2, q4 = (g8 & 3) * 2;
            float bvv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (has_bias) {
              if constexpr (BIAS16) {
                // eight 16-bit values of my row (rows of 128 bytes, 128-byte swizzle), widened here
                const uint4 w = *reinterpret_cast<const uint4*>(bstage + ((g8 ^ (row & 7)) << 4));
                const T* hv = reinterpret_cast<const T*>(&w);
#pragma unroll
                for (int u = 0; u < 8; ++u) bvv[u] = to_float<T>(hv[u]);
              } else {
                const float4 b0 = *reinterpret_cast<const float4*>(bstage + c * (C::kBias / 2) + ((q4 ^ (row & 7)) << 4));
                const float4 b1 = *reinterpret_cast<const float4*>(bstage + c * (C::kBias / 2) + (((q4 + 1) ^ (row & 7)) << 4));
                bvv[0] = b0.x; bvv[1] = b0.y; bvv[2] = b0.z; bvv[3] = b0.w;
                bvv[4] = b1.x; bvv[5] = b1.y; bvv[6] = b1.z; bvv[7] = b1.w;
              }
            }
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u += 2) {  // x = scale*S + bias, two elements per instruction
              const F2 t = f2_fma(f2_from_bits(sr[g8 * 8 + u], sr[g8 * 8 + u + 1]), scale2, f2_make(bvv[u], bvv[u + 1]));
              f2_get(t, v[u], v[u + 1]);
            }
            if constexpr (kMask) {
              const float4 k0 = *reinterpret_cast<const float4*>(mrow + g8 * 8);
              const float4 k1 = *reinterpret_cast<const float4*>(mrow + g8 * 8 + 4);
              const float mkv[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
#pragma unroll
              for (int u = 0; u < 8; ++u) v[u] = (MASKMODE == MASK_MIN) ? fminf(v[u], mkv[u]) : (v[u] + mkv[u]);
            }
#pragma unroll
            for (int u = 0; u < 8; u += 2) {
              x[g8 * 8 + u] = v[u];
              x[g8 * 8 + u + 1] = v[u + 1];
              mx8[u >> 1] = max3(mx8[u >> 1], v[u], v[u + 1]);
            }
          }
        };
        // (only where it measured faster: at D = 64 and D <= 16 the second copy of the loop costs
        // more than the skipped instructions save)
        if constexpr (DP == 32 && MASKMODE == MASK_MIN) {
          if (dirty_row[t] != 0u) scores(std::true_type{});
          else scores(std::false_type{});
        } else {
          scores(std::true_type{});
        }
        const float mx = fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3]));
        if (has_bias) {
          // The stage is handed back only after the bias loads above have returned: the store needs
          // the row maximum, which needs every one of them (an mbarrier arrival by itself does not
          // wait for shared loads that are still queued).
          *scratch = __float_as_uint(mx);
          __syncwarp();
          if (lane == 0) mbar_arrive(b_empty(g % BST));  // one arrival per warp
        }

        const float m_new = fmaxf(m_run, mx);
        const float alpha = ex2((m_run - m_new) * kLog2e);
        float lsum = 0.f;
        uint32_t pk[BN / 2];
        named_bar_sync(1 + w, 256);  // my turn on the exponential unit
        if (m_new != -FLT_MAX) {
          const float nm2 = -m_new * kLog2e;
          const F2 l2e2 = f2_make(kLog2e, kLog2e), nm22 = f2_make(nm2, nm2);
          F2 ls4[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) ls4[u] = f2_make(0.f, 0.f);
          // Software pipeline over groups of eight keys: the FMAs of group g+1 and the sum / pack of
          // group g-1 are placed around the eight ex2 of group g, so the results of the
          // exponential unit are not needed until a group later.
          float y[8], p[8], pp[8];
#pragma unroll
          for (int u = 0; u < 8; u += 2) f2_get(f2_fma(f2_make(x[u], x[u + 1]), l2e2, nm22), y[u], y[u + 1]);
#pragma unroll
          for (int g8 = 0; g8 < BN / 8; ++g8) {
            float yn[8];
            if (g8 + 1 < BN / 8) {
#pragma unroll
              for (int u = 0; u < 8; u += 2)
                f2_get(f2_fma(f2_make(x[(g8 + 1) * 8 + u], x[(g8 + 1) * 8 + u + 1]), l2e2, nm22), yn[u], yn[u + 1]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) p[u] = ex2(y[u]);
            if (g8 > 0) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                ls4[u] = f2_add(ls4[u], f2_make(pp[2 * u], pp[2 * u + 1]));
                pk[(g8 - 1) * 4 + u] = Pack2<T>::pack(pp[2 * u], pp[2 * u + 1]);
              }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) { pp[u] = p[u]; y[u] = yn[u]; }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            ls4[u] = f2_add(ls4[u], f2_make(pp[2 * u], pp[2 * u + 1]));
            pk[(BN / 8 - 1) * 4 + u] = Pack2<T>::pack(pp[2 * u], pp[2 * u + 1]);
          }
          float lsa[8];
#pragma unroll
          for (int u = 0; u < 4; ++u) f2_get(ls4[u], lsa[2 * u], lsa[2 * u + 1]);
          lsum = ((lsa[0] + lsa[1]) + (lsa[2] + lsa[3])) + ((lsa[4] + lsa[5]) + (lsa[6] + lsa[7]));
        } else {
          // every key seen so far was dropped: the scores are all -FLT_MAX and the softmax is
          // uniform over the real keys (test.py:54-55 semantics)
#pragma unroll
          for (int e = 0; e < BN; e += 2) {
            const float p0 = (t * BN + e < a.R) ? 1.f : 0.f;
            const float p1 = (t * BN + e + 1 < a.R) ? 1.f : 0.f;
            lsum += p0 + p1;
            pk[e / 2] = Pack2<T>::pack(p0, p1);
          }
        }
        named_bar_arrive(2 - w, 256);  // hand the turn to the other warpgroup
        l_run = l_run * alpha + lsum;
        m_run = m_new;

        // fold the previous tile's P V into the accumulator (its MMA ran while we did the exps)
        if (t > 0) {
          mbar_wait(o_full(w, (g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
          tc_fence_after();
          uint32_t orr[DP];
          tmem_ld<(DP >= 32 ? 32 : 16)>(t_base + 2 * BN + ((g - 1) & 1) * DP, *reinterpret_cast<uint32_t(*)[DP >= 32 ? 32 : 16]>(&orr[0]));
          if constexpr (DP == 64)
            tmem_ld32(t_base + 2 * BN + ((g - 1) & 1) * DP + 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[32]));
          tmem_wait_ld();
          const F2 ap2 = f2_make(alpha_pending, alpha_pending);
#pragma unroll
          for (int d = 0; d < DP; d += 2)
            f2_get(f2_fma(f2_make(acc[d], acc[d + 1]), ap2, f2_from_bits(orr[d], orr[d + 1])), acc[d], acc[d + 1]);
        }
        alpha_pending = alpha;

        // P_n -> TMEM, packed two 16-bit values per column, over the first half of the S_n
        // columns this thread has just consumed (lane = row, column j = keys 2j, 2j+1): the
        // A operand of P V comes straight from tensor memory.
        tmem_st32(t_base + (g & 1) * BN, pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full(w));
      }
      // last tile's P V
      {
        mbar_wait(o_full(w, (g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag, a.status, DEV_TIMEOUT_MMA);
        tc_fence_after();
        uint32_t orr[DP];
        tmem_ld<(DP >= 32 ? 32 : 16)>(t_base + 2 * BN + ((g - 1) & 1) * DP, *reinterpret_cast<uint32_t(*)[DP >= 32 ? 32 : 16]>(&orr[0]));
        if constexpr (DP == 64)
          tmem_ld32(t_base + 2 * BN + ((g - 1) & 1) * DP + 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[32]));
        tmem_wait_ld();
#pragma unroll
        for (int d = 0; d < DP; ++d) acc[d] = fmaf(acc[d], alpha_pending, __uint_as_float(orr[d]));
      }
      if (active && i < a.R) {
        const float inv = 1.f / l_run;
        T* orow = reinterpret_cast<T*>(a.o) + off4(a.so, it.b, it.h, s, i);
        const T* grow = a.gate ? reinterpret_cast<const T*>(a.gate) + off4(a.sgate, it.b, it.h, s, i) : nullptr;
#pragma unroll
        for (int d8 = 0; d8 < DP / 8; ++d8) {
          if (d8 * 8 < a.D) {
            float f[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) f[u] = acc[d8 * 8 + u] * inv;
            if (grow != nullptr) {  // gated output: O * sigmoid(gate), in the epilogue
              const uint4 gw = *reinterpret_cast<const uint4*>(grow + d8 * 8);
              const T* gv = reinterpret_cast<const T*>(&gw);
#pragma unroll
              for (int u = 0; u < 8; ++u) f[u] *= sigmoidf_fast(to_float<T>(gv[u]));
            }
            uint4 v4;
            v4.x = Pack2<T>::pack(f[0], f[1]);
            v4.y = Pack2<T>::pack(f[2], f[3]);
            v4.z = Pack2<T>::pack(f[4], f[5]);
            v4.w = Pack2<T>::pack(f[6], f[7]);
            *reinterpret_cast<uint4*>(orow + d8 * 8) = v4;
          }
        }
        const long long li = (((long long)it.b * a.H + it.h) * a.S + s) * a.R + i;
        a.lse[li] = (m_run == -FLT_MAX) ? -FLT_MAX : (m_run + logf(l_run));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(m_empty(w, mst));
    }
    if (w == 0) named_bar_sync(1, 256);  // consume the last token so no arrival is left pending
  }

  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA retires
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

// SM count of the current device (looked up once per device).
int num_sms_of_current_device() {
  static int table[64] = {};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (table[dev] > 0) return table[dev];
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 0;
  table[dev] = n;
  return n;
}

template <class T, int DP, bool QP>
int launch_t(const Args& a, cudaStream_t st, int* launches) {
  using C = Cfg<DP, QP>;
  CUtensorMap tq, tk, tv, tb;
  if (!make_qkv_map(&tq, a.q, a.sq, a.B, a.H, a.S, a.R, a.D, DP, BM)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tk, a.k, a.sk, a.B, a.H, a.S, a.R, a.D, DP, BN)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tv, a.v, a.sv, a.B, a.H, a.S, a.R, a.D, DP, BN)) return EVOATTN_ERR_CUDA;
  if (a.bias) {
    const bool ok = a.bias16 ? make_bias16_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, BM, BN)
                             : make_bias_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, BM, 32);
    if (!ok) return EVOATTN_ERR_CUDA;
  } else {
    tb = tq;
  }
  const int g_num_sms = num_sms_of_current_device();
  if (g_num_sms <= 0) return EVOATTN_ERR_CUDA;
  const int T_TILES = (a.R + BN - 1) / BN;
  const int NQT = (a.R + BM - 1) / BM;
  const size_t smem = C::bytes(T_TILES * BN);
  const long long items = QP ? (long long)a.B * a.H * ((NQT + 1) / 2) * a.S
                             : (long long)a.B * a.H * NQT * ((a.S + 1) / 2);
  const int grid = (int)(items < g_num_sms ? items : g_num_sms);
  const bool add = a.mask_kind == EVOATTN_MASK_ADD_F32 || a.mask_kind == EVOATTN_MASK_ADD_SAME;
  auto kern = a.bias16 ? (add ? evo_fwd_sm100_kernel<T, DP, MASK_ADD, true, QP> : evo_fwd_sm100_kernel<T, DP, MASK_MIN, true, QP>)
                       : (add ? evo_fwd_sm100_kernel<T, DP, MASK_ADD, false, QP> : evo_fwd_sm100_kernel<T, DP, MASK_MIN, false, QP>);
  if (!kernel_ready(reinterpret_cast<const void*>(kern), (int)smem, nullptr)) return EVOATTN_ERR_CUDA;
  kern<<<grid, kThreads, smem, st>>>(a, (int)items, tq, tk, tv, tb);
  *launches += 1;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

// A single MSA row with several query tiles runs in query-pair mode (both warpgroups get work);
// everything else pairs MSA rows, which shares the larger tile (the pair bias) between them.
template <class T, int DP>
int launch_mode(const Args& a, cudaStream_t st, int* launches) {
  const int r_pad = (a.R + BN - 1) / BN * BN;
  if (a.S == 1 && a.R > BM && Cfg<DP, true>::bytes(r_pad) <= 232448) return launch_t<T, DP, true>(a, st, launches);
  return launch_t<T, DP, false>(a, st, launches);
}

template <class T>
int launch_d(const Args& a, cudaStream_t st, int* launches) {
  if (a.D <= 16) return launch_mode<T, 16>(a, st, launches);
  if (a.D <= 32) return launch_mode<T, 32>(a, st, launches);
  return launch_mode<T, 64>(a, st, launches);
}

}  // namespace

bool sm100_fwd_supported(int dtype, const Args& a) {
  if (dtype != EVOATTN_BF16 && dtype != EVOATTN_FP16) return false;
  if (a.D % 8 != 0 || a.D > 64) return false;
  if (a.R > 2048) return false;  // two mask rows are staged in shared memory
  if (a.bias) {
    const int es = a.bias16 ? 2 : 4;
    if ((reinterpret_cast<uintptr_t>(a.bias) & 15) != 0) return false;
    if ((a.sbias.a * es) % 16 || (a.sbias.b * es) % 16 || (a.sbias.c * es) % 16) return false;
    if ((a.R * es) % 16 != 0) return false;  // rows of the bias tensor map are whole 16-byte pieces
  }
  if ((long long)a.B * a.H * a.S * ((a.R + BM - 1) / BM) > 2147483647LL) return false;
  return true;
}

int launch_sm100_fwd(int dtype, const Args& a, cudaStream_t st, int* launches) {
  if (dtype == EVOATTN_BF16) return launch_d<__nv_bfloat16>(a, st, launches);
  return launch_d<__half>(a, st, launches);
}

}  // namespace evo
