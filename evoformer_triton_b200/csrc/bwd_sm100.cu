// Evoformer attention backward for sm_100a: the fused dQ/dK/dV/d(pair_bias) kernel with TRANSPOSED
// score tiles, for head dimensions up to 64 (padded to 32 or 64).
//
// Replaces dsevoformer-triton/evoformer.py:299-326 (_attn_bwd_preprocess), :479-630
// (_attn_bwd_dk_dv) and :329-476 (_attn_bwd_dq).  The reference recomputes S and dP in two kernels
// and adds every dS element to d_pair_bias with an fp32 atomic (:458); here they are computed once.
// Like the reference's _attn_bwd_dk_dv (evoformer.py:594,607) the scores are computed as
// S^T = K_j Q_i^T and dP^T = V_j dO_i^T, so a thread owns one KEY j (its TMEM lane) and a run of
// queries i.  What that buys on this machine:
//   * P^T and dS^T (rounded to the storage type, evoformer.py:603,611) are written back into
//     tensor memory over the scores they came from and feed dV_j += P^T dO_i and dK_j += dS^T Q_i
//     as the A operand: P never touches shared memory, dS is stored once (for dQ_i = dS K_j).
//   * The residue mask of a key is one register per thread; the row statistics of the queries
//     (-lse*log2e and delta) are two 128-float vectors that arrive with the Q/dO tiles.
//   * The shared memory this frees holds the K/V tiles of a work item for its whole life and the
//     pair-bias tile of a whole row group.
//
// Work item = one 128-key tile j of G consecutive MSA rows of one (b,h): G = 3 at a padded head
// dimension of 32, G = 1 at 64 (the dK/dV accumulators of a row take 2*DP of the 512 TMEM columns).
// A persistent CTA walks its items as a flat list of steps (query tile i, row g); a step is two
// halves of 64 queries, each with its own TMEM score buffer and its own eight warps: while one half
// computes, the tensor core finishes the other half's dV/dK MMAs and its next S^T/dP^T.
// dS is summed over the G rows in registers and leaves once per (i, j) tile as bulk tensor
// reductions; the dQ partial of a step goes to an fp32 accumulator in global memory the same way.
//
// Warps: 0-15 compute (warp w: keys 32*(w%4).., queries 32*((w/4)%2).. of half w/8), 16-18 issue the
// tcgen05.mma (18 also loads the pair-bias tiles), 19 loads the other tiles.
#include <type_traits>

#include "common.cuh"
#include "launch.h"
#include "ptx.cuh"
#include "tmap.h"

namespace evo {
namespace {

using namespace ptx;

constexpr int BT = 128;   // tile edge (queries and keys)
constexpr int HT = 64;    // queries per half of a step (one warp group)
constexpr int QT = 32;    // queries per quarter of a step
// S^T / dP^T buffers per half: 1 = one of 64 queries shared by the half's eight warps; 2 = one of 32
// queries per group of four warps (four groups that hand over to the tensor core independently;
// measured 2 % slower on the 384-residue workloads: forty smaller MMAs per step instead of thirty-two)
constexpr int kSub = 1;
// MSA rows per work item: each keeps a dK and a dV accumulator of DP columns in tensor memory for the
// whole item, next to 256 columns of score buffers and two dQ partials
template <int DP> struct RowsPerItem { static constexpr int G = (DP == 64) ? 1 : 3; };
constexpr int kCW = 16;   // compute warps
constexpr int kThreadsT = 640;  // 16 compute + 4 service warps, five warps per scheduler
constexpr int kComputeRegs = 112, kServiceRegs = 32;  // after setmaxnreg; the launch-time pool must hold their sum
constexpr int kStages = 2;  // (three or four stages measured no faster: the loads are not what a step waits for)
constexpr float kLog2e = 1.4426950408889634f;

template <int DP>
struct SmemT {
  static constexpr int G = RowsPerItem<DP>::G;
  static constexpr int RB = DP * 2;                          // bytes per staged row
  static constexpr int kTile = BT * RB;                      // one Q, dO, K or V tile
  static constexpr int kVec = BT * 4;                        // one vector of row statistics
  static constexpr int kStage = 2 * kTile + 2 * kVec;        // Q, dO, -lse*log2e, delta of one step
  static constexpr int kDS = BT * BT * 2;                    // dS^T: two halves of [128 keys][64 queries]
  static constexpr int kBias = BT * BT * 4;                  // pair-bias tile [128 i][128 j], unswizzled (fp32; half of it for a 16-bit bias)
  static constexpr int kOutWarp = 2048;                      // per compute warp: staging of a d_bias chunk or a dQ block
  static constexpr int offKV = 0;                            // [g][K, V], resident for the whole item
  static constexpr int offStage = offKV + 2 * G * kTile;
  static constexpr int offDS = offStage + kStages * kStage;
  static constexpr int offBias = offDS + kDS;
  static constexpr int offOut = offBias + kBias;
  static constexpr int offBars = offOut + kCW * kOutWarp;
  // 64 barrier slots (see the kernel) and the slack for aligning the tiles to 1024 bytes.  At DP = 64
  // only 512 bytes of slack fit: the kernel checks what the base address needs and gives up with a
  // status code if it is more (the dynamic shared memory of a kernel without static shared memory
  // starts on a 1024-byte boundary on this architecture, so it needs none).
  static constexpr int kSlack = (DP == 64) ? 512 : 1024;
  static constexpr size_t bytes = offBars + 512 + kSlack;
  static_assert(offDS % 1024 == 0 && kStage % 1024 == 0 && offStage % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static_assert(bytes <= 232448, "shared memory budget of one CTA");
};

struct StepT {
  int b, h, s, it, g, j0;
};

// An mbarrier named by its 32-bit shared-window address (8 bytes apart in the barrier array).
struct Bar {
  uint32_t a;
};
__device__ __forceinline__ Bar operator+(Bar b, int i) { return Bar{b.a + 8u * static_cast<uint32_t>(i)}; }
__device__ __forceinline__ bool mbar_wait(Bar b, uint32_t parity, uint32_t abort_s, int* status, int code) {
  return mbar_wait_s(b.a, parity, abort_s, status, code);
}
__device__ __forceinline__ void mbar_arrive(Bar b) { mbar_arrive_s(b.a); }
__device__ __forceinline__ void mbar_expect_tx(Bar b, uint32_t bytes) { mbar_expect_tx_s(b.a, bytes); }
__device__ __forceinline__ void mma_commit_if(uint32_t leader, Bar b) { mma_commit_if_s(leader, b.a); }


// delta[b,h,s,i] = <dO_i, O_i> (evoformer.py:299-326) and nl = -lse*log2e, one thread per row.
// A row whose keys were all dropped carries lse = -FLT_MAX from the forward; its nl is +inf, which
// the fused kernel recognises.  The block also clears its 256 rows of the fp32 dQ accumulator
// (contiguous in memory), which saves a separate pass over that buffer.
template <class T>
__global__ void __launch_bounds__(256) prep_kernel(Args a, float* __restrict__ nl, float* __restrict__ dq_acc) {
  const long long rows = (long long)a.B * a.H * a.S * a.R;
  {
    const long long f4_first = (long long)blockIdx.x * 256 * (a.D / 4);
    const long long f4_end = min(rows, (long long)(blockIdx.x + 1) * 256) * (a.D / 4);
    float4* dst = reinterpret_cast<float4*>(dq_acc);
    for (long long e = f4_first + threadIdx.x; e < f4_end; e += 256) dst[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const long long row = (long long)blockIdx.x * 256 + threadIdx.x;
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
  if (!a.delta_ready) a.delta[row] = acc;
  const float lse = a.lse[row];
  nl[row] = (lse == -FLT_MAX) ? __int_as_float(0x7f800000) : -lse * kLog2e;
}

// dq = scale * dq_acc, cast to the storage type (dq_acc: contiguous fp32 [B,H,S,R,D]).
template <class T>
__global__ void __launch_bounds__(256) dq_store_kernel(Args a, const float* __restrict__ acc) {
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

template <class T, int DP, bool kHasBias, bool kBias16>
__global__ void __launch_bounds__(kThreadsT, 1)
evo_bwd_sm100_kernel(const Args a, const int n_items, const __grid_constant__ CUtensorMap tmQ,
                const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmDB, const __grid_constant__ CUtensorMap tmDQ,
                const __grid_constant__ CUtensorMap tmNL, const __grid_constant__ CUtensorMap tmDL) {
  using L = SmemT<DP>;
  constexpr int RB = L::RB;
  constexpr uint32_t SWZ = swizzle_code_for_row_bytes(RB);
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  static_assert(DP == 32 || DP == 64, "padded head dimension");
  constexpr int G = RowsPerItem<DP>::G;
  constexpr int kTmemCols = 512;
  // TMEM: two (S^T, dP^T) half-tile buffers, the per-row dV and dK accumulators, two dQ partials
  constexpr int colS0 = 0, colDP0 = HT, colS1 = 2 * HT, colDP1 = 3 * HT;
  constexpr int colDV = 4 * HT, colDK = colDV + G * DP, colDQ = colDK + G * DP;
  static_assert(colDQ + 2 * DP <= kTmemCols, "TMEM budget");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (static_cast<int>(smem - smem_raw) > L::kSlack) {  // the same for every thread of every CTA
    if (threadIdx.x == 0 && a.status) atomicCAS(a.status, 0, DEV_TIMEOUT_SYNC);
    return;
  }
  uint8_t* sKV = smem + L::offKV;
  uint8_t* sStage = smem + L::offStage;
  uint8_t* sDS = smem + L::offDS;
  uint8_t* sBias = smem + L::offBias;
  uint8_t* sOut = smem + L::offOut;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBars);
  const uint32_t bars_s = smem_u32(bars);
  const Bar kv_full{bars_s + 8 * 0};     // [G] K and V of row g of the current item landed
  const Bar kv_empty{bars_s + 8 * 3};    // [G] ... and every MMA that reads them has completed
  const Bar st_full{bars_s + 8 * 32};     // [2] Q, dO and the statistics vectors of a step landed
  const Bar st_empty{bars_s + 8 * 40};    // [2] ... the step's last dV/dK MMAs have completed
  const Bar sd_full{bars_s + 8 * 48};    // [2][kSub] S^T and dP^T of score buffer (h, sub) of a step are in TMEM
  const Bar cdone{bars_s + 8 * 52};      // [2][kSub] the warps of that buffer have its P^T and dS^T in TMEM (for the dV/dK MMAs)
  const Bar sdone{bars_s + 8 * 23};      // [2] ... and have stored their half of dS in shared memory (for the dQ MMAs)
  const Bar b_full{bars_s + 8 * 14};     // [2] half h (64 queries) of the pair-bias tile landed
  const Bar b_done{bars_s + 8 * 16};     // [2] ... has been read for the last time
  const Bar ds_empty{bars_s + 8 * 18};   // the dQ MMAs of a step have read the dS tile
  const Bar dq_full{bars_s + 8 * 19};    // [2] the dQ partial of a step is complete in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 22);  // (bars 23, 24: sdone)
  const uint32_t abort_s = smem_u32(const_cast<int*>(abort_flag));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NT = (a.R + BT - 1) / BT;
  const int NC = (a.S + G - 1) / G;
  constexpr bool has_bias = kHasBias;
  constexpr int kBRow = kBias16 ? BT * 2 : BT * 4;  // bytes per row (one query, 128 keys) of the staged bias tile
  const bool flush_dbias = has_bias && a.dbias != nullptr;
  // Persistent CTAs: CTA c owns the items c, c + gridDim.x, ..., SPI steps per item.  A short last
  // row group (S % G != 0) is padded with rows >= S: their tiles and statistics arrive as zeros and
  // their mask is -inf, so P = dS = 0, and nothing of them is stored.
  const int SPI = NT * G;
  const int my_items = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int total_steps = my_items * SPI;
  auto decode = [&](int N) {
    StepT d;
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
  auto advance = [&](const StepT& c, int n) {  // position of step n = the one after c (no divisions inside an item)
    StepT d = c;
    if (++d.g == G) {
      d.g = 0;
      if (++d.it == NT) return decode(n);
    }
    d.s = c.s - c.g + d.g;
    return d;
  };

  if (tid == 0) *abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (*abort_flag) return;

  if (tid == 0) {
    for (int i = 0; i < G; ++i) { mbar_init(bars + 0 + i, 1); mbar_init(bars + 3 + i, 3); }  // kv_full; kv_empty: three MMA warps read K/V
    for (int i = 0; i < kStages; ++i) { mbar_init(bars + 32 + i, 1); mbar_init(bars + 40 + i, 2); }  // st_full, st_empty
    for (int i = 0; i < 2; ++i) {
      for (int q = 0; q < 2; ++q) { mbar_init(bars + 48 + 2 * i + q, 2); mbar_init(bars + 52 + 2 * i + q, kCW / (2 * kSub)); }  // sd_full, cdone
      mbar_init(bars + 14 + i, 1); mbar_init(bars + 16 + i, kCW / 2);  // b_full, b_done
      mbar_init(bars + 19 + i, 1);                                     // dq_full
      mbar_init(bars + 23 + i, kCW / 2);                               // sdone
    }
    mbar_init(bars + 18, 1);  // ds_empty
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
    prefetch_tmap(&tmNL); prefetch_tmap(&tmDL); prefetch_tmap(&tmDQ);
    if (has_bias) prefetch_tmap(&tmB);
    if (flush_dbias) prefetch_tmap(&tmDB);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp >= kCW) {
    setmaxnreg_dec<kServiceRegs>();
    if (warp <= kCW + 1) {
      // =============================== tensor-core issuers: warp 16 (S^T, dV), warp 17 (dP^T, dK) ==========
      // Issuing a tcgen05.mma costs the issuing warp fifty cycles and more, so the 32 MMAs of a step
      // are spread over three warps on three schedulers.  A thread's MMAs run in issue order, MMAs of
      // different threads in no particular order, so the split follows the data: warp 16 owns the
      // S^T columns of both buffers (S^T = K_j Q_i^T in, dV_j += P^T dO_i out), warp 17 the dP^T columns
      // (dP^T = V_j dO_i^T in, dK_j += dS^T Q_i out): the MMA that overwrites a buffer is always issued
      // by the thread that issued the MMAs reading it.  Warp 18 issues dQ_i = dS K_j, which depends on
      // neither.  One lane of each warp runs the whole issue loop (measured: a tcgen05.mma issued from a
      // single-thread branch costs the warp a quarter less than the same instruction predicated on a
      // leader lane in a converged warp).
      const bool isA = (warp == kCW);
      if (lane == 0) {
      constexpr uint32_t kIdescSD = make_idesc(kBf16, false, false, BT, HT / kSub);   // S^T, dP^T: K-major operands, N = 64 or 32
      constexpr uint32_t kIdescOut = make_idesc(kBf16, false, true, BT, DP);   // dV, dK: A from TMEM, B MN-major
      constexpr uint32_t kHiOp = static_cast<uint32_t>(make_sdesc_const(16, 8 * RB, SWZ) >> 32);
      constexpr uint32_t kLoLbo = static_cast<uint32_t>(make_sdesc_const(16, 0, 0) & 0xffffffffu);
      constexpr uint32_t kRowBlk = (16 * RB) >> 4;  // 16 tile rows, in descriptor address units
      // warp 16 reads K (A operand) and Q (B), then dO (B of dV); warp 17 reads V and dO, then Q (B of dK)
      const uint32_t kv_lo = (smem_u32(sKV) >> 4) + (isA ? 0 : (L::kTile >> 4));
      const uint32_t in_lo = (smem_u32(sStage) >> 4) + (isA ? 0 : (L::kTile >> 4));
      const uint32_t out_lo = (smem_u32(sStage) >> 4) + (isA ? (L::kTile >> 4) : 0);
      const uint32_t col_in0 = isA ? colS0 : colDP0, col_in1 = isA ? colS1 : colDP1;
      const uint32_t col_acc = isA ? colDV : colDK;

      // Position of a step inside this CTA's list, advanced without divisions: row g of the group,
      // query tile it, ring stage and the parities of the stage ring and of the item.
      struct Pos { int g, it; uint32_t stg, ring_par, item_par; };
      auto after = [&](Pos p) {
        if (++p.g == G) { p.g = 0; if (++p.it == NT) { p.it = 0; p.item_par ^= 1u; } }
        if (++p.stg == (uint32_t)kStages) { p.stg = 0; p.ring_par ^= 1u; }
        return p;
      };
      constexpr int QB = HT / kSub;  // queries per S^T / dP^T buffer
      // Everything an MMA group needs is computed before the wait it follows: this thread shares its
      // scheduler with four arithmetic warps, so every instruction between the wake-up and the MMA is
      // paid several times over, and it sits on the critical path of the half that waits for it.
      auto issue_in = [&](const Pos& p, uint32_t ka, uint32_t qb, int h, int sub) {
        // (the second commit: the item's last read of this warp's K or V tile of row g)
        const uint32_t bar2 = (h == 1 && sub == kSub - 1 && p.it == NT - 1) ? (kv_empty + p.g).a : 0u;
        const uint32_t tD = tmem + (h ? col_in1 : col_in0) + sub * QB, qa = qb + (h * HT + sub * QB) * (RB >> 4);
        if constexpr (DP == 32) {  // two K slices of 16
          mma_ss_x2_commit(tD, ka, qa, kHiOp, 2, kIdescSD, (sd_full + (2 * h + sub)).a, bar2);
        } else {                   // four
          mma_ss_x4_commit(tD, ka, qa, kHiOp, 2, kIdescSD, (sd_full + (2 * h + sub)).a, bar2);
        }
      };
      Pos cur{0, 0, 0u, 0u, 0u};
      if (total_steps > 0) {
        mbar_wait(st_full + 0, 0, abort_s, a.status, DEV_TIMEOUT_TMA);
        mbar_wait(kv_full + 0, 0, abort_s, a.status, DEV_TIMEOUT_TMA);
        tc_fence_after();
        const uint32_t ka = (kv_lo + 0) | kLoLbo, qb = in_lo | kLoLbo;
#pragma unroll
        for (int sub = 0; sub < kSub; ++sub) { issue_in(cur, ka, qb, 0, sub); issue_in(cur, ka, qb, 1, sub); }
      }
      for (int n = 0; n < total_steps; ++n) {
        const Pos nxt = after(cur);
        const bool more = n + 1 < total_steps;
        // this step: dV_j[g] += P^T dO_i (warp 16) or dK_j[g] += dS^T Q_i (warp 17);
        // A = 16 queries of P^T / dS^T (8 packed TMEM columns), B = their dO / Q rows
        const uint32_t acc = tmem + col_acc + cur.g * DP;
        const uint32_t ob = (out_lo + cur.stg * (L::kStage >> 4)) | kLoLbo;
        const uint32_t first0 = (cur.it == 0) ? 0u : 1u;  // the item's first MMA of row g overwrites
        const uint32_t st_empty_bar = (st_empty + (int)cur.stg).a;
        // next step: S^T = K_j Q_i^T (warp 16) or dP^T = V_j dO_i^T (warp 17) into the buffer just read
        const uint32_t ka = (kv_lo + (2 * nxt.g) * (L::kTile >> 4)) | kLoLbo;
        const uint32_t qb = (in_lo + nxt.stg * (L::kStage >> 4)) | kLoLbo;
        const uint32_t st_full_bar = (st_full + (int)nxt.stg).a, kv_full_bar = (kv_full + nxt.g).a;
#pragma unroll
        for (int sub = 0; sub < kSub; ++sub) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            mbar_wait(cdone + (2 * h + sub), n & 1, abort_s, a.status, DEV_TIMEOUT_SYNC);
            // (an item's first MMA of row g overwrites an accumulator that all warps of half 0 drain first)
            if (kSub == 2 && h == 0 && sub == 0 && cur.it == 0) mbar_wait(cdone + 1, n & 1, abort_s, a.status, DEV_TIMEOUT_SYNC);
            tc_fence_after();
            const uint32_t tA = tmem + (h ? col_in1 : col_in0) + sub * QB;
            const uint32_t ba = ob + (4 * h + (4 / kSub) * sub) * kRowBlk;
            const uint32_t first = (h == 0 && sub == 0) ? first0 : 1u;
            if constexpr (kSub == 1) mma_ts_x4(acc, tA, ba, kHiOp, kRowBlk, kIdescOut, first);
            else mma_ts_x2(acc, tA, ba, kHiOp, kRowBlk, kIdescOut, first);
            if (h == 1 && sub == kSub - 1) mma_commit_if_s(1u, st_empty_bar);
            if (more) {
              if (h == 0 && sub == 0) {
                mbar_wait_s(st_full_bar, nxt.ring_par, abort_s, a.status, DEV_TIMEOUT_TMA);
                if (nxt.it == 0) mbar_wait_s(kv_full_bar, nxt.item_par, abort_s, a.status, DEV_TIMEOUT_TMA);
                tc_fence_after();
              }
              issue_in(nxt, ka, qb, h, sub);
            }
          }
        }
        cur = nxt;
      }
      }  // lane 0
    } else if (warp == kCW + 2) {
      // =============================== tensor-core issuer of dQ; pair-bias loads ===============================
      if (lane == 0) {
      constexpr uint32_t kIdescDQ = make_idesc(kBf16, true, true, BT, DP);     // A = dS^T read MN-major, B = K MN-major
      constexpr uint32_t kHiOp = static_cast<uint32_t>(make_sdesc_const(16, 8 * RB, SWZ) >> 32);
      constexpr uint32_t kHiDS = static_cast<uint32_t>(make_sdesc_const(16, 1024, SWZ_128B) >> 32);
      constexpr uint32_t kLoLbo = static_cast<uint32_t>(make_sdesc_const(16, 0, 0) & 0xffffffffu);
      constexpr uint32_t kLoLboDS = static_cast<uint32_t>(make_sdesc_const(BT * 128, 0, 0) & 0xffffffffu);
      constexpr uint32_t kRowBlk = (16 * RB) >> 4;
      const uint32_t kv_lo = smem_u32(sKV) >> 4, ds_lo = smem_u32(sDS) >> 4;
      const uint32_t sBias_s = smem_u32(sBias);
      // The bias tile (i, j) is the same for the G rows of a group; each half (64 queries) is loaded
      // for the group's first step and replaced as soon as the warps of that half have read it for
      // the last time.
      auto load_bias = [&](const StepT& d, int h) {
        mbar_expect_tx(b_full + h, HT * kBRow);
        tma_load_4d_s(sBias_s + h * (HT * kBRow), &tmB, (b_full + h).a, d.j0, d.it * BT + h * HT, d.h, d.b);
      };
      const int tiles = my_items * NT;
      if (has_bias && tiles > 0) { const StepT d0 = decode(0); load_bias(d0, 0); load_bias(d0, 1); }
      int g = 0, it = 0, t = 0;  // row of the group, query tile, running (item, query tile) index
      for (int n = 0; n < total_steps; ++n) {
        const bool turn = has_bias && g == G - 1 && t + 1 < tiles;  // the group's last step: the halves come back
        StepT nb = StepT{0, 0, 0, 0, 0, 0};
        if (turn) nb = decode((t + 1) * G);  // (divisions: before the waits, not between them)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mbar_wait(sdone + h, n & 1, abort_s, a.status, DEV_TIMEOUT_SYNC);
          if (turn) {
            mbar_wait(b_done + h, t & 1, abort_s, a.status, DEV_TIMEOUT_SYNC);
            load_bias(nb, h);
          }
        }
        tc_fence_after();
        const uint32_t ka = (kv_lo + (2 * g) * (L::kTile >> 4)) | kLoLbo;
        // dQ_i partial = dS K_j : A = dS^T tile [key][query] read MN-major (M = query), K runs over the keys
        mma_ss_x8(tmem + colDQ + (n & 1) * DP, ds_lo | kLoLboDS, kHiDS, 128, ka, kHiOp, kRowBlk, kIdescDQ);
        mma_commit_if(1u, dq_full + (n & 1));
        mma_commit_if(1u, ds_empty);
        if (it == NT - 1) mma_commit_if(1u, kv_empty + g);
        if (++g == G) { g = 0; ++t; if (++it == NT) it = 0; }
      }
      }  // lane 0
    } else {
      // =============================== tile loader ===============================
      // K/V of row g stay for the whole item and are replaced when the item's last MMAs that read them
      // have completed; Q, dO and the two statistics vectors of a step ride a two-deep ring.
      const uint32_t sKV_s = smem_u32(sKV), sStage_s = smem_u32(sStage);
      StepT d = decode(0);
      for (int n = 0; n < total_steps; ++n) {
        const int stg = n % kStages;
        if (d.it == 0) {
          const int k = n / SPI;
          mbar_wait(kv_empty + d.g, (k & 1) ^ 1, abort_s, a.status, DEV_TIMEOUT_MMA);
          if (lane == 0) {
            const uint32_t dst = sKV_s + (2 * d.g) * L::kTile;
            mbar_expect_tx(kv_full + d.g, 2 * L::kTile);
            tma_load_5d_s(dst, &tmK, (kv_full + d.g).a, 0, d.j0, d.s, d.h, d.b);
            tma_load_5d_s(dst + L::kTile, &tmV, (kv_full + d.g).a, 0, d.j0, d.s, d.h, d.b);
          }
          __syncwarp();
        }
        mbar_wait(st_empty + stg, ((n / kStages) & 1) ^ 1, abort_s, a.status, DEV_TIMEOUT_MMA);
        if (lane == 0) {
          const uint32_t dst = sStage_s + stg * L::kStage;
          const uint32_t bar = (st_full + stg).a;
          mbar_expect_tx(st_full + stg, L::kStage);
          tma_load_5d_s(dst, &tmQ, bar, 0, d.it * BT, d.s, d.h, d.b);
          tma_load_5d_s(dst + L::kTile, &tmDO, bar, 0, d.it * BT, d.s, d.h, d.b);
          tma_load_3d_s(dst + 2 * L::kTile, &tmNL, bar, d.it * BT, d.s, d.b * a.H + d.h);
          tma_load_3d_s(dst + 2 * L::kTile + L::kVec, &tmDL, bar, d.it * BT, d.s, d.b * a.H + d.h);
        }
        __syncwarp();
        d = advance(d, n + 1);
      }
    }
  } else {
    // =============================== compute warps ===============================
    // Warps 0-7 work on half 0 (queries 0..63 of the tile) of every step, warps 8-15 on half 1: two
    // groups that run half a step apart, so that while one waits (for its S^T/dP^T, for tensor
    // memory, for its MMAs) the other has arithmetic to issue.  Warp w: keys 32*(w%4).. (its TMEM
    // lanes), queries 32*((w/4)%2).. of its half, in two chunks of 16.
    setmaxnreg_inc<kComputeRegs>();
    const int q4 = warp & 3, cb2 = (warp >> 2) & 1, H = warp >> 3;
    const int jrow = q4 * 32 + lane;
    const uint32_t t_lane = tmem + (static_cast<uint32_t>(q4 * 32) << 16);
    const uint32_t cS = t_lane + (H ? colS1 : colS0) + QT * cb2, cP = t_lane + (H ? colDP1 : colDP0) + QT * cb2;
    const float scale = a.scale;
    const float inv_r = 1.f / (float)a.R;
    const float kInf = __int_as_float(0x7f800000);
    const float c1 = scale * kLog2e;
    // 32-bit shared-window addresses: every access below stays a shared-memory instruction
    const uint32_t sStage_s = smem_u32(sStage), sDS_s = smem_u32(sDS);
    const uint32_t out_s = smem_u32(sOut) + warp * L::kOutWarp;  // this warp's private staging area
    const uint32_t brow0 = smem_u32(sBias) + (H * HT + QT * cb2) * kBRow + jrow * (kBias16 ? 2 : 4);
    const uint32_t drow = sDS_s + H * (L::kDS / 2) + jrow * 128;

    // The residue mask of (b, s, key) in two halves, so that the load can be issued a step before
    // its value is needed: the raw element ...
    auto mask_fetch = [&](int b, int s, int j, bool wanted) -> uint32_t {
      const bool ok = wanted && s < a.S && j < a.R && a.mask_kind != EVOATTN_MASK_NONE;
      const long long mi = (long long)b * a.smask.a + (long long)s * a.smask.b + (long long)j * a.smask.c;
      if (a.mask_kind == EVOATTN_MASK_BOOL) return ldg_u8_if(reinterpret_cast<const unsigned char*>(a.mask) + mi, ok);
      if (a.mask_kind == EVOATTN_MASK_ADD_F32) return ldg_u32_if(reinterpret_cast<const uint32_t*>(a.mask) + mi, ok);
      return ldg_u16_if(reinterpret_cast<const uint16_t*>(a.mask) + mi, ok);
    };
    // ... and the float that is added to a score in the log2 domain: 0 keeps it, -inf drops it (a
    // dropped score gives P = 0 exactly, as exp(-FLT_MAX - lse) does in evoformer.py:69,600)
    auto mask_decode = [&](uint32_t raw, int s, int j) -> float {
      if (s >= a.S || j >= a.R) return -kInf;
      if (a.mask_kind == EVOATTN_MASK_NONE) return 0.f;
      if (a.mask_kind == EVOATTN_MASK_BOOL) return raw ? 0.f : -kInf;
      if (a.mask_kind == EVOATTN_MASK_ADD_F32) return __uint_as_float(raw) * kLog2e;
      const uint16_t h16 = (uint16_t)raw;
      return to_float<T>(*reinterpret_cast<const T*>(&h16)) * kLog2e;
    };
    // This warp's staging area is free again once its previous bulk reduction has read it.
    auto staging_free = [&]() {
      if (lane == 0) tma_wait_group_read0();
      __syncwarp();
    };

    // dK, dV of row-group slot g (MSA row s of (b,h), keys j0..): TMEM -> registers -> global.
    // Done by the warps of half 0 (half of the DP columns each, 16 at a time): they are the ones
    // whose arrival lets the next item's first MMAs overwrite the slot.
    auto drain_dkdv = [&](int b, int h, int s, int j0, int g) {
      const int j = j0 + jrow;
#pragma unroll
      for (int part = 0; part < DP / 32; ++part) {
        const int c0 = cb2 * (DP / 2) + part * 16;
        uint32_t kr[16], vr[16];
        tmem_ld16(t_lane + colDK + g * DP + c0, kr);
        tmem_ld16(t_lane + colDV + g * DP + c0, vr);
        tmem_wait_ld();
        if (j < a.R && s < a.S) {
          T* kd = reinterpret_cast<T*>(a.dk) + off4(a.sdk, b, h, s, j) + c0;
          T* vd = reinterpret_cast<T*>(a.dv) + off4(a.sdv, b, h, s, j) + c0;
#pragma unroll
          for (int d8 = 0; d8 < 2; ++d8) {
            if (c0 + d8 * 8 < a.D) {
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
    };
    // The dQ partial of step m at position d (TMEM lanes = queries): this warp's DP/4 columns of its 32
    // query rows go through its staging area ([32 rows][DP/4 floats]) into the fp32 accumulator in global
    // memory, as one small bulk tensor reduction that the warp issues itself.  It happens after the
    // warp's arrival, underneath the tensor core's turnaround for its half.
    constexpr int QC = DP / 4;       // dQ columns per warp (8 or 16)
    const int colblk = 2 * H + cb2;  // which of the four column blocks this warp drains
    auto send_dq = [&](int m, const StepT& d) {
      mbar_wait(dq_full + (m & 1), (m >> 1) & 1, abort_s, a.status, DEV_TIMEOUT_MMA);
      tc_fence_after();
      uint32_t qr[QC];
      tmem_ld<QC>(t_lane + colDQ + (m & 1) * DP + colblk * QC, qr);
      staging_free();
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < QC / 4; ++c)
        sts_v4(out_s + lane * (QC * 4) + 16 * c, qr[4 * c], qr[4 * c + 1], qr[4 * c + 2], qr[4 * c + 3]);
      fence_async_shared();
      __syncwarp();
      if (lane == 0 && d.s < a.S && colblk * QC < a.D) {
        tma_reduce_add_3d_s(&tmDQ, out_s, colblk * QC, d.it * BT + q4 * 32, (d.b * a.H + d.h) * a.S + d.s);
        tma_commit_group();
      }
    };

    StepT cur = decode(0), prv = cur;
    uint32_t mraw = mask_fetch(cur.b, cur.s, cur.j0 + jrow, total_steps > 0);
    int pb = 0, ph = 0, ps0 = 0, pj0 = 0;  // the item whose dK/dV still sit in TMEM
    float bacc[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) bacc[e] = 0.f;

    for (int n = 0; n < total_steps; ++n) {
      const StepT nxt = advance(cur, n + 1);
      const bool more = n + 1 < total_steps;
      const int g = cur.g;
      const float mj = mask_decode(mraw, cur.s, cur.j0 + jrow);
      mraw = mask_fetch(nxt.b, nxt.s, nxt.j0 + jrow, more);  // in flight during this step
      const int stg = n % kStages;
      const uint32_t vec_s = sStage_s + stg * L::kStage + 2 * L::kTile;
      const bool last_of_group = (g == G - 1);
      // the statistics vectors of this step are read with ordinary loads: observe their arrival here
      mbar_wait(st_full + stg, (n / kStages) & 1, abort_s, a.status, DEV_TIMEOUT_TMA);
      if (has_bias && g == 0) mbar_wait(b_full + H, (n / G) & 1, abort_s, a.status, DEV_TIMEOUT_TMA);
      // a row whose keys are all dropped has nl = +inf for every query (the mask row is shared by
      // all queries of the MSA row): the whole step is uniform, P = 1/N_res, dS = 0
      const bool deadstep = (lds_f32(vec_s) == kInf);
      uint32_t dk[16];
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        // this warp's queries of the half: 32*cb2 + 16*sub .. +16
        if (sub == 0) {
          mbar_wait(sd_full + (2 * H + (kSub == 2 ? cb2 : 0)), n & 1, abort_s, a.status, DEV_TIMEOUT_MMA);
          tc_fence_after();
        }
        uint32_t sr[16], dr[16];
        tmem_ld16(cS + 16 * sub, sr);
        tmem_ld16(cP + 16 * sub, dr);
        const uint32_t vnl = vec_s + (H * HT + QT * cb2 + 16 * sub) * 4, vdl = vnl + BT * 4;
        const uint32_t brow = brow0 + (16 * sub) * kBRow;
        tmem_wait_ld();
        uint32_t pk[8];
        if (!deadstep) {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const float4 nl = lds_v4f(vnl + 16 * c4);
            const float4 dl = lds_v4f(vdl + 16 * c4);
            float t[4] = {nl.x, nl.y, nl.z, nl.w};
            const float de[4] = {dl.x, dl.y, dl.z, dl.w};
            if (has_bias) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                float bv;
                if constexpr (kBias16) {
                  const uint16_t raw = lds_u16(brow + (4 * c4 + u) * kBRow);
                  bv = to_float<T>(*reinterpret_cast<const T*>(&raw));
                } else {
                  bv = lds_f32(brow + (4 * c4 + u) * kBRow);
                }
                t[u] = fmaf(bv, kLog2e, t[u]);
              }
            }
            float p[4], ds[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              // x = S*(scale*log2e) + (bias*log2e - lse*log2e) + mask
              const float x = fmaf(__uint_as_float(sr[4 * c4 + u]), c1, t[u]) + mj;
              p[u] = ex2(x);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              // dS = P (dP - delta); d_bias_acc += dS
              ds[u] = p[u] * (__uint_as_float(dr[4 * c4 + u]) - de[u]);
              bacc[sub * 16 + 4 * c4 + u] += ds[u];
            }
            pk[2 * c4] = Pack2<T>::pack(p[0], p[1]);
            pk[2 * c4 + 1] = Pack2<T>::pack(p[2], p[3]);
            dk[sub * 8 + 2 * c4] = Pack2<T>::pack(ds[0], ds[1]);
            dk[sub * 8 + 2 * c4 + 1] = Pack2<T>::pack(ds[2], ds[3]);
          }
        } else {
          const float pu = (cur.j0 + jrow < a.R) ? inv_r : 0.f;
          const uint32_t w = Pack2<T>::pack(pu, pu);
#pragma unroll
          for (int e = 0; e < 8; ++e) { pk[e] = w; dk[sub * 8 + e] = 0u; }  // replaced scores are constants: dS = 0
        }
        // P^T and dS^T, two 16-bit values per column, over the columns this thread has just read:
        // the A operands of the dV and dK MMAs (16 queries = 8 packed columns each)
        tmem_st8(cS + 16 * sub, pk);
        tmem_st8(cP + 16 * sub, *reinterpret_cast<uint32_t(*)[8]>(&dk[sub * 8]));
        // P^T and dS^T of this warp's score buffer are in tensor memory: its dV / dK MMAs may go
        if (sub == 1 && H == 0 && cur.it == 0 && n >= SPI) drain_dkdv(pb, ph, ps0 + g, pj0, g);  // before those MMAs overwrite it
        if (sub == 1) {
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(cdone + (2 * H + (kSub == 2 ? cb2 : 0)));
        }
        if (flush_dbias && last_of_group) {
          // The group's last row: this thread's 16 d_bias values of the chunk (one key, 16 queries) go
          // through the warp's staging area ([16 queries][32 keys]) and are added to d_bias in global
          // memory by a bulk tensor reduction that the warp issues itself.
          staging_free();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            sts_f32(out_s + c * 128 + lane * 4, bacc[sub * 16 + c]);
            bacc[sub * 16 + c] = 0.f;
          }
          fence_async_shared();
          __syncwarp();
          if (lane == 0) {
            tma_reduce_add_4d_s(&tmDB, out_s, cur.j0 + q4 * 32, cur.it * BT + H * HT + QT * cb2 + 16 * sub, cur.h, cur.b);
            tma_commit_group();
          }
        }
      }
      // dS^T -> shared memory, [key][query] rows of 128 bytes per half, 128-byte swizzle; the tile is
      // free once the dQ MMAs of the previous step have read it
      mbar_wait(ds_empty, (n & 1) ^ 1, abort_s, a.status, DEV_TIMEOUT_MMA);
#pragma unroll
      for (int c = 0; c < 4; ++c)  // dk[4 * c ..]: queries 32 * cb2 + 8 * c .. of this half
        sts_v4(drow + (((4 * cb2 + c) ^ (jrow & 7)) << 4), dk[4 * c], dk[4 * c + 1], dk[4 * c + 2], dk[4 * c + 3]);
      fence_async_shared();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(sdone + H);
        if (has_bias && last_of_group) mbar_arrive(b_done + H);
      }
      if (n > 0) send_dq(n - 1, prv);  // its MMAs ran underneath this step
      if (cur.it == NT - 1 && last_of_group) { pb = cur.b; ph = cur.h; ps0 = cur.s - g; pj0 = cur.j0; }
      prv = cur;
      cur = nxt;
    }

    if (total_steps > 0) {
      send_dq(total_steps - 1, prv);
      if (H == 0) {
        // every dV / dK MMA of this CTA has completed once the last step's tile stage has been released
        const int last = total_steps - 1;
        mbar_wait(st_empty + (last % kStages), (last / kStages) & 1, abort_s, a.status, DEV_TIMEOUT_MMA);
        tc_fence_after();
        for (int g = 0; g < G; ++g) drain_dkdv(pb, ph, ps0 + g, pj0, g);
      }
    }
    if (lane == 0) tma_wait_group0();  // this warp's reductions have completed before the CTA may exit
  }

  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kTmemCols);
}

size_t align_up(size_t x, size_t al) { return (x + al - 1) / al * al; }

template <class T, int DP>
int launch_t(const Args& a0, void* ws, size_t ws_bytes, cudaStream_t st, int* launches) {
  constexpr int G = RowsPerItem<DP>::G;
  using L = SmemT<DP>;
  Args a = a0;
  const size_t rows = (size_t)a.B * a.H * a.S * a.R;
  const size_t vec_bytes = align_up(rows * sizeof(float), 256);
  const size_t dq_bytes = rows * a.D * sizeof(float);
  if (ws_bytes < 2 * vec_bytes + dq_bytes) return EVOATTN_ERR_WORKSPACE;
  a.delta = reinterpret_cast<float*>(ws);
  float* nl = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + vec_bytes);
  float* dq_acc = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + 2 * vec_bytes);

  CUtensorMap tq, tk, tv, tdo, tb, tdb, tdq, tnl, tdl;
  if (!make_qkv_map(&tq, a.q, a.sq, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tk, a.k, a.sk, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tv, a.v, a.sv, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_qkv_map(&tdo, a.d_o, a.sdo, a.B, a.H, a.S, a.R, a.D, DP, BT)) return EVOATTN_ERR_CUDA;
  if (!make_rows_f32_plain_map(&tdq, dq_acc, a.D, a.R, (long long)a.B * a.H * a.S, DP / 4, 32)) return EVOATTN_ERR_CUDA;
  if (!make_stats_map(&tnl, nl, a.B * a.H, a.S, a.R, BT)) return EVOATTN_ERR_CUDA;
  if (!make_stats_map(&tdl, a.delta, a.B * a.H, a.S, a.R, BT)) return EVOATTN_ERR_CUDA;
  tb = tq;
  tdb = tq;
  if (a.bias) {
    const bool ok = a.bias16 ? make_bias16_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, HT, BT, /*swizzle=*/false)
                             : make_bias_plain_map(&tb, a.bias, a.sbias, a.B, a.H, a.R, HT, BT);
    if (!ok) return EVOATTN_ERR_CUDA;
    const Str3 dense{(long long)a.H * a.R * a.R, (long long)a.R * a.R, (long long)a.R};
    if (a.dbias && !make_bias_plain_map(&tdb, a.dbias, dense, a.B, a.H, a.R, 16, 32)) return EVOATTN_ERR_CUDA;
  }
  if (a.dbias && cudaMemsetAsync(a.dbias, 0, (size_t)a.B * a.H * a.R * a.R * sizeof(float), st) != cudaSuccess)
    return EVOATTN_ERR_CUDA;
  prep_kernel<T><<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(a, nl, dq_acc);

  const int NT = (a.R + BT - 1) / BT;
  const long long items = (long long)a.B * a.H * NT * ((a.S + G - 1) / G);
  if (items > 0x7fffffffLL / (G * NT)) return EVOATTN_ERR_SHAPE;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return EVOATTN_ERR_CUDA;
  const long long ctas = items < sms ? items : sms;
  auto kern = !a.bias ? evo_bwd_sm100_kernel<T, DP, false, false>
                      : (a.bias16 ? evo_bwd_sm100_kernel<T, DP, true, true> : evo_bwd_sm100_kernel<T, DP, true, false>);
  // setmaxnreg.inc waits until the scheduler's register pool (five warps at the launch-time count)
  // has what it asks for: never launch a build whose pool cannot hold the warps' requests.
  int num_regs = 0;
  if (!kernel_ready(reinterpret_cast<const void*>(kern), (int)L::bytes, &num_regs)) return EVOATTN_ERR_CUDA;
  if ((kThreadsT / 128) * num_regs < 4 * kComputeRegs + kServiceRegs) return EVOATTN_ERR_UNSUPPORTED;
  kern<<<(unsigned)ctas, kThreadsT, L::bytes, st>>>(a, (int)items, tq, tk, tv, tdo, tb, tdb, tdq, tnl, tdl);
  // d(pair_bias) is complete: its sum over the GPUs of the node, if the caller asked for one, runs on
  // a stream of its own next to the dQ store below; the caller's stream waits for it at the end
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  if (a.exchange) {
    if (!exchange_lane(&side, &fork, &join)) return EVOATTN_ERR_CUDA;
    if (cudaEventRecord(fork, st) != cudaSuccess || cudaStreamWaitEvent(side, fork, 0) != cudaSuccess) return EVOATTN_ERR_CUDA;
    const int rc = launch_peer_allreduce(reinterpret_cast<const evoattn_peer_allreduce_params*>(a.exchange), side);
    if (cudaEventRecord(join, side) != cudaSuccess) return EVOATTN_ERR_CUDA;  // (join even after a failed launch)
    if (rc) { cudaStreamWaitEvent(st, join, 0); return rc; }
    *launches += 1;
  }
  const long long n8 = (long long)rows * (a.D / 8);
  dq_store_kernel<T><<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(a, dq_acc);
  if (a.exchange && cudaStreamWaitEvent(st, join, 0) != cudaSuccess) return EVOATTN_ERR_CUDA;
  *launches += 3;
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

}  // namespace


bool sm100_bwd_supported(int dtype, const Args& a) {
  if (!sm100_fwd_supported(dtype, a)) return false;
  const long long NT = (a.R + BT - 1) / BT;
  if ((long long)a.B * a.H * NT * a.S > 2147483647LL) return false;
  return true;
}

size_t sm100_bwd_workspace_bytes(int, const Args& a) {
  const size_t rows = (size_t)a.B * a.H * a.S * a.R;
  return 2 * align_up(rows * sizeof(float), 256) + rows * a.D * sizeof(float);
}

int launch_sm100_bwd(int dtype, const Args& a, void* workspace, size_t workspace_bytes, cudaStream_t st,
                     int* launches) {
  if (a.D <= 32) {
    if (dtype == EVOATTN_BF16) return launch_t<__nv_bfloat16, 32>(a, workspace, workspace_bytes, st, launches);
    return launch_t<__half, 32>(a, workspace, workspace_bytes, st, launches);
  }
  if (dtype == EVOATTN_BF16) return launch_t<__nv_bfloat16, 64>(a, workspace, workspace_bytes, st, launches);
  return launch_t<__half, 64>(a, workspace, workspace_bytes, st, launches);
}

}  // namespace evo
