// extern "C" surface of libevoattn.so: argument validation, dispatch, launches.
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "launch.h"

namespace {

thread_local int g_last_path = EVOATTN_PATH_NONE;
thread_local int g_last_launches = 0;
thread_local int g_ctx_bound_device = -1;

// Tensor maps are encoded through the driver API, which needs the device's primary context
// to be current on the calling thread.  A thread that has made no runtime call yet (PyTorch's
// autograd worker on its first backward) gets it bound here, once per thread and device.
void bind_context_once() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  if (g_ctx_bound_device != dev) {
    cudaFree(nullptr);  // the customary no-op that initialises / binds the primary context
    g_ctx_bound_device = dev;
  }
}

bool stride_ok16(const int64_t* s, int esize) {
  for (int i = 0; i < 4; ++i)
    if ((s[i] * esize) % 16 != 0) return false;
  return true;
}

evo::Str4 str4(const int64_t* s) { return evo::Str4{s[0], s[1], s[2], s[3]}; }

int esize_of(int dtype) { return dtype == EVOATTN_FP32 ? 4 : 2; }

int validate_fwd(const evoattn_fwd_params* p) {
  if (!p) return EVOATTN_ERR_NULL;
  if (!p->q || !p->k || !p->v || !p->o || !p->lse) return EVOATTN_ERR_NULL;
  if (p->dtype != EVOATTN_BF16 && p->dtype != EVOATTN_FP16 && p->dtype != EVOATTN_FP32) return EVOATTN_ERR_DTYPE;
  if (p->B <= 0 || p->H <= 0 || p->S <= 0 || p->R <= 0 || p->D <= 0) return EVOATTN_ERR_SHAPE;
  if ((long long)p->B * p->H * p->S > 2147483647LL) return EVOATTN_ERR_SHAPE;
  if (p->R > 65535 * 8) return EVOATTN_ERR_SHAPE;
  if (p->D > 128) return EVOATTN_ERR_UNSUPPORTED;
  if (p->mask_kind < EVOATTN_MASK_NONE || p->mask_kind > EVOATTN_MASK_ADD_SAME) return EVOATTN_ERR_DTYPE;
  if (p->mask_kind != EVOATTN_MASK_NONE && !p->mask) return EVOATTN_ERR_NULL;
  if (p->bias_dtype != EVOATTN_BIAS_F32 && p->bias_dtype != EVOATTN_BIAS_SAME) return EVOATTN_ERR_DTYPE;
  if (!(p->scale == p->scale)) return EVOATTN_ERR_SHAPE;  // NaN scale
  return EVOATTN_OK;
}

void fill_args(const evoattn_fwd_params* p, evo::Args* a) {
  memset(a, 0, sizeof(*a));
  a->B = p->B; a->H = p->H; a->S = p->S; a->R = p->R; a->D = p->D;
  a->scale = p->scale;
  a->q = p->q; a->k = p->k; a->v = p->v; a->o = p->o; a->lse = p->lse;
  a->sq = str4(p->q_stride); a->sk = str4(p->k_stride); a->sv = str4(p->v_stride); a->so = str4(p->o_stride);
  a->mask = p->mask_kind == EVOATTN_MASK_NONE ? nullptr : p->mask;
  a->mask_kind = p->mask_kind;
  a->smask = evo::Str3{p->mask_stride[0], p->mask_stride[1], p->mask_stride[2]};
  a->bias = reinterpret_cast<const float*>(p->bias);
  a->sbias = evo::Str3{p->bias_stride[0], p->bias_stride[1], p->bias_stride[2]};
  a->bias16 = (p->bias && p->bias_dtype == EVOATTN_BIAS_SAME && p->dtype != EVOATTN_FP32) ? 1 : 0;
  a->status = p->status;
  a->gate = p->gate;
  a->sgate = str4(p->gate_stride);
}

int validate_bwd(const evoattn_bwd_params* p) {
  if (!p) return EVOATTN_ERR_NULL;
  int rc = validate_fwd(&p->fwd);
  if (rc) return rc;
  if (!p->d_o || !p->dq || !p->dk || !p->dv) return EVOATTN_ERR_NULL;
  if (p->fwd.gate && !p->dgate) return EVOATTN_ERR_NULL;
  if (p->exchange) {  // the in-call sum of d(pair_bias) over the node's GPUs works on the caller's exchange buffer
    const evoattn_peer_allreduce_params* x = p->exchange;
    if (!p->fwd.bias || !p->dbias || !x->bufs) return EVOATTN_ERR_NULL;
    if (x->world < 1 || x->world > 8 || x->rank < 0 || x->rank >= x->world) return EVOATTN_ERR_SHAPE;
    if (x->bufs[x->rank] != p->dbias) return EVOATTN_ERR_SHAPE;
    if (x->count != (uint64_t)p->fwd.B * p->fwd.H * p->fwd.R * p->fwd.R) return EVOATTN_ERR_SHAPE;
  }
  return EVOATTN_OK;
}

void fill_bwd_args(const evoattn_bwd_params* p, evo::Args* a) {
  fill_args(&p->fwd, a);
  a->d_o = p->d_o; a->dq = p->dq; a->dk = p->dk; a->dv = p->dv;
  a->dbias = p->fwd.bias ? p->dbias : nullptr;
  a->sdo = str4(p->do_stride); a->sdq = str4(p->dq_stride); a->sdk = str4(p->dk_stride); a->sdv = str4(p->dv_stride);
  a->dmask = p->dmask;
  a->exchange = p->exchange;
}

size_t generic_bwd_workspace(const evo::Args& a) {
  return (size_t)a.B * a.H * a.S * a.R * sizeof(float);  // delta
}

bool use_sm100_fwd(const evoattn_fwd_params* p, const evo::Args& a) {
  if (p->flags & EVOATTN_FLAG_FORCE_GENERIC) return false;
  if (p->dtype == EVOATTN_FP32) return false;
  if (((uintptr_t)p->q | (uintptr_t)p->k | (uintptr_t)p->v | (uintptr_t)p->o) & 15) return false;
  const int es = esize_of(p->dtype);
  if (p->gate && ((((uintptr_t)p->gate) & 15) || !stride_ok16(p->gate_stride, es))) return false;
  if (!stride_ok16(p->q_stride, es) || !stride_ok16(p->k_stride, es) || !stride_ok16(p->v_stride, es) ||
      !stride_ok16(p->o_stride, es))
    return false;
  return evo::sm100_fwd_supported(p->dtype, a);
}

bool use_sm100_bwd(const evoattn_bwd_params* p, const evo::Args& a) {
  if (!use_sm100_fwd(&p->fwd, a)) return false;
  if (p->dmask) return false;  // the gradient of an additive mask is produced by the CUDA-core kernels
  if (((uintptr_t)p->d_o | (uintptr_t)p->dq | (uintptr_t)p->dk | (uintptr_t)p->dv) & 15) return false;
  const int es = esize_of(p->fwd.dtype);
  if (!stride_ok16(p->do_stride, es) || !stride_ok16(p->dq_stride, es) || !stride_ok16(p->dk_stride, es) ||
      !stride_ok16(p->dv_stride, es))
    return false;
  // d(pair_bias) leaves through a tensor map over its dense [B,H,R,R] layout: 16-byte base and rows
  if (p->fwd.bias && p->dbias && ((((uintptr_t)p->dbias) & 15) != 0 || (p->fwd.R % 4) != 0)) return false;
  return evo::sm100_bwd_supported(p->fwd.dtype, a);
}

// Scratch of evoattn_bwd_static_scratch(): part of the library image, so every GPU that loads
// the library holds it until the process exits.  In host code this name is only a stand-in
// for the symbol, never a device address: the address is looked up per device below.
static __device__ __align__(256) unsigned char g_static_scratch[EVOATTN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of the static scratch on the current device.  The lookup is repeated on every
// call: it is cheap, it allocates nothing, and it is also what makes the device's primary
// context current on a host thread that has made no CUDA call yet (a fresh worker thread, the
// autograd engine's thread), which the tensor-map encoder needs.  The per-device table is only a
// cross-check that the address never changes.
int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return EVOATTN_ERR_CUDA;
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return EVOATTN_ERR_CUDA;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_addr[dev]) g_static_scratch_addr[dev] = ptr;
    else if (g_static_scratch_addr[dev] != ptr) return EVOATTN_ERR_CUDA;
  }
  *out = ptr;
  return EVOATTN_OK;
}

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Scratch of a backward call: what the kernel family needs, then (gated output) the effective dO.
size_t path_scratch_need(const evoattn_bwd_params* p, const evo::Args& a, bool fast) {
  return align256(fast ? evo::sm100_bwd_workspace_bytes(p->fwd.dtype, a) : generic_bwd_workspace(a));
}
size_t bwd_scratch_need(const evoattn_bwd_params* p, const evo::Args& a, bool fast) {
  return path_scratch_need(p, a, fast) + (p->fwd.gate ? evo::gate_backward_scratch_bytes(p->fwd.dtype, a) : 0);
}

// The backward with its scratch at `scratch` (caller-provided or the static array).
int run_bwd(const evoattn_bwd_params* p, evo::Args& a, bool fast, void* scratch, cudaStream_t st) {
  const size_t path_bytes = path_scratch_need(p, a, fast);
  a.delta = reinterpret_cast<float*>(scratch);  // every kernel family keeps delta at the start of its scratch
  if (p->fwd.gate) {
    const int rc = evo::launch_gate_backward(p->fwd.dtype, &a, reinterpret_cast<unsigned char*>(scratch) + path_bytes, p->dgate,
                                             str4(p->dgate_stride), st, &g_last_launches);
    if (rc) return rc;
  }
  if (a.dmask &&
      cudaMemsetAsync(a.dmask, 0, (size_t)a.B * a.S * a.R * sizeof(float), st) != cudaSuccess)
    return EVOATTN_ERR_CUDA;
  if (fast) {
    g_last_path = EVOATTN_PATH_TCGEN05;
    return evo::launch_sm100_bwd(p->fwd.dtype, a, scratch, path_bytes, st, &g_last_launches);
  }
  g_last_path = EVOATTN_PATH_GENERIC;
  if (evo::launch_generic_bwd(p->fwd.dtype, a, st, &g_last_launches) != cudaSuccess) return EVOATTN_ERR_CUDA;
  if (p->exchange) {  // (the CUDA-core kernels have nothing to run the exchange next to)
    const int rc = evo::launch_peer_allreduce(p->exchange, st);
    if (rc) return rc;
    g_last_launches += 1;
  }
  return EVOATTN_OK;
}

}  // namespace

extern "C" {

int evoattn_abi_version(void) { return EVOATTN_ABI_VERSION; }

const char* evoattn_strerror(int status) {
  switch (status) {
    case EVOATTN_OK: return "ok";
    case EVOATTN_ERR_NULL: return "a required pointer is null";
    case EVOATTN_ERR_SHAPE: return "a dimension or scale is out of range";
    case EVOATTN_ERR_DTYPE: return "unknown dtype or mask kind";
    case EVOATTN_ERR_ALIGN: return "base address or stride is not 16-byte aligned";
    case EVOATTN_ERR_UNSUPPORTED: return "no kernel covers this request (head dimension above 128?)";
    case EVOATTN_ERR_CUDA: return "a CUDA call failed (launch or tensor-map creation)";
    case EVOATTN_ERR_WORKSPACE: return "workspace is null or smaller than evoattn_bwd_workspace_bytes()";
    case EVOATTN_ERR_DEVICE: return "a kernel gave up a bounded wait and set the device status word";
    default: return "unknown status";
  }
}

int evoattn_fwd(const evoattn_fwd_params* p, void* cuda_stream) {
  g_last_path = EVOATTN_PATH_NONE;
  g_last_launches = 0;
  int rc = validate_fwd(p);
  if (rc) return rc;
  evo::Args a;
  fill_args(p, &a);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  bind_context_once();
  if (use_sm100_fwd(p, a)) {
    g_last_path = EVOATTN_PATH_TCGEN05;
    return evo::launch_sm100_fwd(p->dtype, a, st, &g_last_launches);
  }
  g_last_path = EVOATTN_PATH_GENERIC;
  return evo::launch_generic_fwd(p->dtype, a, st, &g_last_launches) == cudaSuccess ? EVOATTN_OK : EVOATTN_ERR_CUDA;
}

size_t evoattn_bwd_workspace_bytes(const evoattn_bwd_params* p) {
  if (validate_bwd(p)) return 0;
  evo::Args a;
  fill_bwd_args(p, &a);
  return bwd_scratch_need(p, a, use_sm100_bwd(p, a));
}

int evoattn_bwd(const evoattn_bwd_params* p, void* cuda_stream) {
  g_last_path = EVOATTN_PATH_NONE;
  g_last_launches = 0;
  int rc = validate_bwd(p);
  if (rc) return rc;
  evo::Args a;
  fill_bwd_args(p, &a);
  bind_context_once();
  const bool fast = use_sm100_bwd(p, a);
  const size_t need = bwd_scratch_need(p, a, fast);
  if (need && (!p->workspace || p->workspace_bytes < need)) return EVOATTN_ERR_WORKSPACE;
  if (need && ((uintptr_t)p->workspace & 255)) return EVOATTN_ERR_ALIGN;
  return run_bwd(p, a, fast, p->workspace, reinterpret_cast<cudaStream_t>(cuda_stream));
}

int evoattn_bwd_static_scratch(const evoattn_bwd_params* p, void* cuda_stream) {
  g_last_path = EVOATTN_PATH_NONE;
  g_last_launches = 0;
  int rc = validate_bwd(p);
  if (rc) return rc;
  evo::Args a;
  fill_bwd_args(p, &a);
  const bool fast = use_sm100_bwd(p, a);
  if (bwd_scratch_need(p, a, fast) > EVOATTN_STATIC_SCRATCH_BYTES) return EVOATTN_ERR_WORKSPACE;
  // Looking the symbol up (done on every call) also makes the device's primary context current
  // on this thread, which the tensor-map encoder needs; nothing here allocates.
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc) return rc;
  return run_bwd(p, a, fast, scratch, reinterpret_cast<cudaStream_t>(cuda_stream));
}

int evoattn_last_path(void) { return g_last_path; }
int evoattn_last_launch_count(void) { return g_last_launches; }

}  // extern "C"
