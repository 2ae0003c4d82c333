// Sum of one fp32 buffer over the GPUs of a node through peer memory (NVLink / NVSwitch), in
// place: the d(pair_bias) exchange of the N_seq-sharded op.
//
// The reference is a single-GPU program (its d_pair_bias is complete after the local atomics of
// dsevoformer-triton/evoformer.py:458 and the cast at :860); sharding the MSA rows over GPUs adds
// one sum over ranks, and for the few megabytes involved a library all-reduce costs more in launch
// and protocol latency than in bytes.  Here every rank maps every other rank's buffer (CUDA IPC)
// and one kernel per rank does a two-shot all-reduce in which all traffic between GPUs is stores
// (posted writes; a load from a peer costs a round trip of microseconds):
//   rank r stores slice q of its local sums into rank q's staging area, for every q != r
//   barrier  - all contributions to my slice have landed
//   rank r adds up slice r over the ranks in rank order and stores the result into slice r of
//   every rank's buffer
//   barrier  - all slices have landed everywhere
// The staging area follows the data in the same allocation (evoattn_peer_data_bytes).  Barriers
// are per thread block (block b of every rank meets block b of the others) through flag
// words in each rank's own memory that peers write with system-scope release stores; flags carry
// an epoch that grows with every call, so they are never reset.  Every wait is bounded: when it
// runs out the kernel records a code in the status word and goes on without waiting (the result
// is then invalid, the GPU stays usable).  No multicast loads, no multimem.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "launch.h"

namespace evo {
namespace {

constexpr int kMaxPeers = 8;
constexpr int kBlocks = 128;  // one per SM or fewer: blocks of different ranks wait for one another, all must be resident
constexpr int kThreads = 512;
constexpr long long kPeerWaitCycles = 4000000000LL;  // about two seconds

struct PeerArgs {
  float* buf[kMaxPeers];
  uint32_t* flag[kMaxPeers];  // each rank's pad: [2 barriers][kBlocks][kMaxPeers] words
  int world, rank;
  unsigned long long count;
  uint32_t epoch;
  int* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Where the staging area starts inside a rank's allocation that holds `count` floats of data.
__host__ __device__ inline unsigned long long stage_offset(unsigned long long count) { return (count * 4 + 255) / 256 * 256; }

// Staged contributions were written by peers and published by the barrier's acquire.
__device__ __forceinline__ float4 ld_staged_v4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kThreads) peer_allreduce_kernel(const PeerArgs p) {
  const int b = blockIdx.x, tid = threadIdx.x;
  float tail_value = 0.f;
  // The epoch of this call: the caller's, or (epoch 0) one more than this block's own counter, which
  // lives behind the flags in this rank's flag buffer.  Every rank makes the same calls, so block b
  // of every rank counts alike; a launch replayed from a CUDA graph, whose arguments are frozen,
  // still gets a new epoch each time.
  uint32_t* const my_count = p.flag[p.rank] + 2 * kBlocks * kMaxPeers + b;
  const uint32_t epoch = p.epoch ? p.epoch : *reinterpret_cast<volatile uint32_t*>(my_count) + 1u;
  // meet block b of every other rank: tell them, then wait for them (thread q handles rank q)
  auto barrier = [&](int which, int code) {
    __syncthreads();
    if (tid < p.world) {
      __threadfence_system();
      st_release_sys(p.flag[tid] + (which * kBlocks + b) * kMaxPeers + p.rank, epoch);
      const uint32_t* mine = p.flag[p.rank] + (which * kBlocks + b) * kMaxPeers + tid;
      const long long t0 = clock64();
      // epochs only grow: a value at or beyond this call's epoch means that rank has arrived
      while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
        if (clock64() - t0 > kPeerWaitCycles) {
          if (p.status) atomicCAS(p.status, 0, code);
          break;
        }
      }
    }
    __syncthreads();
  };

  const unsigned long long n4 = p.count / 4;
  const unsigned long long seg = (n4 + p.world - 1) / p.world;  // float4 per staging segment (one per contributing rank)
  const unsigned long long stride = (unsigned long long)kBlocks * kThreads;
  const unsigned long long t0 = (unsigned long long)b * kThreads + tid;
  const float4* mine = reinterpret_cast<const float4*>(p.buf[p.rank]);
  auto stage_of = [&](int q) { return reinterpret_cast<float4*>(reinterpret_cast<char*>(p.buf[q]) + stage_offset(p.count)); };

  // my contribution to every other rank's slice goes into that rank's staging area, segment `rank`
  for (int d = 1; d < p.world; ++d) {
    const int q = (p.rank + d) % p.world;  // start with a different peer on every rank
    const unsigned long long lo = n4 * q / p.world, hi = n4 * (q + 1) / p.world;
    float4* dst = stage_of(q) + (unsigned long long)p.rank * seg;
    for (unsigned long long i = lo + t0; i < hi; i += stride) dst[i - lo] = mine[i];
  }

  barrier(0, DEV_TIMEOUT_SYNC);

  {
    const unsigned long long lo = n4 * p.rank / p.world, hi = n4 * (p.rank + 1) / p.world;
    const float4* stage = stage_of(p.rank);
    for (unsigned long long i = lo + t0; i < hi; i += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)  // rank order: the same bits whatever the timing
        if (q < p.world) {
          const float4 v = (q == p.rank) ? mine[i] : ld_staged_v4(stage + (unsigned long long)q * seg + (i - lo));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)
        if (q < p.world) reinterpret_cast<float4*>(p.buf[q])[i] = acc;
    }
  }
  if (p.count & 3) {  // the last count % 4 elements: every rank sums them itself, from the peers' buffers
    // (they lie outside every slice, so nothing overwrites them before the second barrier)
    if (b == 0 && tid < (int)(p.count & 3)) {
      const unsigned long long i = n4 * 4 + tid;
      float acc = 0.f;
      for (int q = 0; q < p.world; ++q) acc += ld_peer_f32(p.buf[q] + i);
      tail_value = acc;
    }
  }

  barrier(1, DEV_TIMEOUT_SYNC);
  if (p.epoch == 0 && tid == 0) *my_count = epoch;
  // (all ranks have read the tail elements of all buffers: now each may overwrite its own)
  if ((p.count & 3) && b == 0 && tid < (int)(p.count & 3)) p.buf[p.rank][n4 * 4 + tid] = tail_value;
}

}  // namespace

int launch_peer_allreduce(const evoattn_peer_allreduce_params* p, cudaStream_t st) {
  if (!p || !p->bufs || !p->flags) return EVOATTN_ERR_NULL;
  if (p->world < 1 || p->world > kMaxPeers || p->rank < 0 || p->rank >= p->world) return EVOATTN_ERR_SHAPE;
  if (p->count == 0) return EVOATTN_OK;
  PeerArgs a;
  memset(&a, 0, sizeof(a));
  for (int q = 0; q < p->world; ++q) {
    if (!p->bufs[q] || !p->flags[q]) return EVOATTN_ERR_NULL;
    if (((uintptr_t)p->bufs[q]) & 255) return EVOATTN_ERR_ALIGN;
    a.buf[q] = p->bufs[q];
    a.flag[q] = p->flags[q];
  }
  a.world = p->world; a.rank = p->rank; a.count = p->count; a.epoch = p->epoch; a.status = p->status;
  peer_allreduce_kernel<<<kBlocks, kThreads, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

// The stream and the two events with which a backward call runs its exchange next to its last
// kernel: one set per device, made at the first call that asks for it (which therefore must not be
// inside a stream capture) and kept until the process ends.
bool exchange_lane(cudaStream_t* side, cudaEvent_t* fork, cudaEvent_t* join) {
  struct Lane { cudaStream_t s; cudaEvent_t f, j; bool ok; };
  static Lane lanes[64] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  Lane& l = lanes[dev];
  if (!l.ok) {
    if (cudaStreamCreateWithFlags(&l.s, cudaStreamNonBlocking) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&l.f, cudaEventDisableTiming) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&l.j, cudaEventDisableTiming) != cudaSuccess) return false;
    l.ok = true;
  }
  *side = l.s; *fork = l.f; *join = l.j;
  return true;
}

}  // namespace evo

extern "C" {

size_t evoattn_peer_data_bytes(uint64_t count, int world) {
  if (world < 1) world = 1;
  const unsigned long long n4 = count / 4, seg = (n4 + world - 1) / world;
  return (size_t)(evo::stage_offset(count) + (unsigned long long)world * seg * 16);
}

size_t evoattn_peer_flag_bytes(void) {
  return ((size_t)2 * evo::kBlocks * evo::kMaxPeers + evo::kBlocks) * sizeof(uint32_t);  // flags, then the blocks' call counters
}

int evoattn_peer_buffer_create(size_t bytes, void** dev_ptr, unsigned char handle_out[64]) {
  if (!dev_ptr || !handle_out || bytes == 0) return EVOATTN_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* ptr = nullptr;
  if (cudaMalloc(&ptr, bytes) != cudaSuccess) return EVOATTN_ERR_CUDA;
  if (cudaMemset(ptr, 0, bytes) != cudaSuccess) { cudaFree(ptr); return EVOATTN_ERR_CUDA; }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) { cudaFree(ptr); return EVOATTN_ERR_CUDA; }
  memcpy(handle_out, &h, 64);
  *dev_ptr = ptr;
  return EVOATTN_OK;
}

int evoattn_peer_buffer_open(const unsigned char handle[64], void** dev_ptr) {
  if (!handle || !dev_ptr) return EVOATTN_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* ptr = nullptr;
  if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return EVOATTN_ERR_CUDA;
  }
  *dev_ptr = ptr;
  return EVOATTN_OK;
}

int evoattn_peer_buffer_close(void* dev_ptr) {
  return cudaIpcCloseMemHandle(dev_ptr) == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

int evoattn_peer_buffer_destroy(void* dev_ptr) { return cudaFree(dev_ptr) == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA; }

int evoattn_peer_allreduce_f32(const evoattn_peer_allreduce_params* p, void* cuda_stream) {
  return evo::launch_peer_allreduce(p, reinterpret_cast<cudaStream_t>(cuda_stream));
}

}  // extern "C"
