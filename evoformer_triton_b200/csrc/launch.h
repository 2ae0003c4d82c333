// Host-side launch entry points of the kernel families (internal to the library).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>

#include <mutex>
#include <unordered_map>
#include <utility>

#include "common.cuh"

namespace evo {

// Per (device, kernel) facts that cost a driver call each: the dynamic shared memory limit that has
// been set for the kernel and its launch-time register count.  Looked up on every launch, asked of
// the driver once (the limit again only when a launch needs more than any before it).
struct KernelFacts {
  int smem_limit = 0;
  int num_regs = 0;
};
inline bool kernel_ready(const void* kern, int smem_bytes, int* num_regs) {
  static std::mutex mu;
  static std::unordered_map<const void*, KernelFacts> facts[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  KernelFacts& f = facts[dev][kern];
  if (f.num_regs == 0) {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) return false;
    f.num_regs = fa.numRegs;
  }
  if (smem_bytes > f.smem_limit) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return false;
    f.smem_limit = smem_bytes;
  }
  if (num_regs) *num_regs = f.num_regs;
  return true;
}

// CUDA-core kernels (generic_kernels.cu).  Backward needs a.delta = [B,H,S,R] fp32 scratch.
cudaError_t launch_generic_fwd(int dtype, const Args& a, cudaStream_t st, int* launches);
cudaError_t launch_generic_bwd(int dtype, const Args& a, cudaStream_t st, int* launches);

// tcgen05 / TMEM / TMA kernels (fwd_sm100.cu, bwd_sm100.cu).  The *_supported
// predicates say whether a request is covered; the launchers return an EVOATTN_* status.
bool sm100_fwd_supported(int dtype, const Args& a);
int launch_sm100_fwd(int dtype, const Args& a, cudaStream_t st, int* launches);
bool sm100_bwd_supported(int dtype, const Args& a);
size_t sm100_bwd_workspace_bytes(int dtype, const Args& a);
int launch_sm100_bwd(int dtype, const Args& a, void* workspace, size_t workspace_bytes, cudaStream_t st,
                     int* launches);

// The exchange of d(pair_bias) between the GPUs of a node (peer_reduce.cu), and the side stream
// with its fork / join events on which a backward call runs it next to its last kernel.
int launch_peer_allreduce(const evoattn_peer_allreduce_params* p, cudaStream_t st);
bool exchange_lane(cudaStream_t* side, cudaEvent_t* fork, cudaEvent_t* join);

// Backward half of the gated output (extras.cu): writes delta, the effective dO (into `scratch`) and
// dgate, and redirects `a` to the effective dO.
size_t gate_backward_scratch_bytes(int dtype, const Args& a);
int launch_gate_backward(int dtype, Args* a, void* scratch, void* dgate, const Str4& sdgate, cudaStream_t st, int* launches);

}  // namespace evo
