/*
 * evoattn.h - C ABI of libevoattn.so: Evoformer attention (pair-bias + residue-mask
 * flash attention, forward and backward) for NVIDIA B200 (sm_100a).
 *
 * Plain C, plain pointers and sizes.  The library owns no memory: every input,
 * output and scratch buffer is device memory allocated by the caller (the one exception
 * is the fixed scratch array of evoattn_bwd_static_scratch, see there).  All work is
 * enqueued on the CUDA stream handed in (a cudaStream_t passed as void*); nothing
 * synchronises, nothing is freed, no pointer is kept after a call returns.
 *
 * Tensors are described in the *attention view* [B, H, S, R, D]:
 *   B batch, H heads, S = N_seq (MSA rows), R = N_res, D = head dimension.
 * The reference obtains this view by reinterpreting its [B, N_seq, N_res, H, D]
 * tensors (dsevoformer-triton/evoformer.py:648-650); a caller that wants true head
 * semantics passes the strides of a permuted view instead.  Strides are in elements,
 * for the axes (b, h, s, r); the D axis is contiguous.
 */
#ifndef EVOATTN_H_
#define EVOATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EVOATTN_ABI_VERSION 3

/* status codes (0 = success). */
enum {
  EVOATTN_OK = 0,
  EVOATTN_ERR_NULL = 1,        /* a required pointer is null */
  EVOATTN_ERR_SHAPE = 2,       /* a dimension is out of range */
  EVOATTN_ERR_DTYPE = 3,       /* unknown dtype / mask kind */
  EVOATTN_ERR_ALIGN = 4,       /* base address or stride breaks the 16-byte rule */
  EVOATTN_ERR_UNSUPPORTED = 5, /* valid request that no kernel covers */
  EVOATTN_ERR_CUDA = 6,        /* a CUDA call (launch, tensor map) failed */
  EVOATTN_ERR_WORKSPACE = 7,   /* workspace missing or too small */
  EVOATTN_ERR_DEVICE = 8       /* the device status word was set by a kernel */
};

enum { EVOATTN_BF16 = 0, EVOATTN_FP16 = 1, EVOATTN_FP32 = 2 };

/* res_mask forms.  BOOL: one byte per key, non-zero = keep; dropped keys have their
 * score *replaced* by -FLT_MAX (evoformer.py:69, test.py:54).  The additive forms add
 * the value to the score (the DS4Sci "mask bias" convention). */
enum {
  EVOATTN_MASK_NONE = 0,
  EVOATTN_MASK_BOOL = 1,
  EVOATTN_MASK_ADD_F32 = 2,
  EVOATTN_MASK_ADD_SAME = 3 /* additive, stored in the q/k/v dtype */
};

/* Storage type of the pair bias.  The reference's callers pass it in fp32 (test.py:36-42) or in
 * the 16-bit type of q/k/v (memory_benchmark.py:20, speed_benchmark.py:83); the kernels read
 * either as it is and widen in registers. */
enum {
  EVOATTN_BIAS_F32 = 0,
  EVOATTN_BIAS_SAME = 1 /* stored in the q/k/v dtype (bf16 or fp16) */
};

/* flags */
enum {
  EVOATTN_FLAG_FORCE_GENERIC = 1 /* use the CUDA-core kernels even where a tcgen05 kernel exists */
};

/* Which kernel family served the last call on this thread (for tests and logs). */
enum { EVOATTN_PATH_NONE = 0, EVOATTN_PATH_GENERIC = 1, EVOATTN_PATH_TCGEN05 = 2 };

typedef struct evoattn_fwd_params {
  int32_t dtype;          /* EVOATTN_BF16 / FP16 / FP32: type of q, k, v, o */
  int32_t B, H, S, R, D;
  float scale;            /* softmax scale, D^-1/2 in the reference (evoformer.py:646) */
  uint32_t flags;
  const void* q;          /* [B,H,S,R,D] attention view */
  const void* k;
  const void* v;
  void* o;                /* out, same dtype */
  float* lse;             /* out, contiguous [B,H,S,R] fp32: log-sum-exp of each score row
                             (the tensor M of evoformer.py:669-671) */
  int64_t q_stride[4];    /* element strides of (b,h,s,r) */
  int64_t k_stride[4];
  int64_t v_stride[4];
  int64_t o_stride[4];
  const void* mask;       /* [B,S,R] or null */
  int32_t mask_kind;
  int32_t bias_dtype;     /* EVOATTN_BIAS_F32 or EVOATTN_BIAS_SAME */
  int64_t mask_stride[3]; /* element strides of (b,s,r) */
  const void* bias;       /* pair bias [B,H,R,R] (type: bias_dtype) or null; last axis contiguous */
  int64_t bias_stride[3]; /* element strides of (b,h,i) */
  int32_t* status;        /* optional device word; a kernel that gives up a bounded wait
                             writes a non-zero code here instead of hanging or trapping */
  const void* gate;       /* optional gating logits, attention view, q/k/v dtype: the output becomes
                             sigmoid(gate) * O, applied in the kernel's epilogue (the step that follows
                             the attention in a gated-attention block; the reference has no such input).
                             Null: plain attention, as the reference computes it */
  int64_t gate_stride[4]; /* element strides of (b,h,s,r) */
} evoattn_fwd_params;

struct evoattn_peer_allreduce_params;  /* below: the exchange between the GPUs of a node */

typedef struct evoattn_bwd_params {
  evoattn_fwd_params fwd; /* same q,k,v,o,lse,mask,bias as the forward call (o and lse are inputs) */
  const void* d_o;        /* dO, attention view */
  void* dq;               /* out */
  void* dk;               /* out */
  void* dv;               /* out */
  float* dbias;           /* out, fp32 [B,H,R,R] contiguous: the sum over the S rows of dS
                             (evoformer.py:458), written in full (no need to zero it first).
                             Null when bias is null, or when the caller wants no gradient for
                             the bias (the kernels then skip its reductions altogether) */
  int64_t do_stride[4];
  int64_t dq_stride[4];
  int64_t dk_stride[4];
  int64_t dv_stride[4];
  void* workspace;        /* device scratch of at least evoattn_bwd_workspace_bytes() */
  size_t workspace_bytes;
  void* dgate;            /* out, gradient of fwd.gate (same dtype), required when fwd.gate is set;
                             d_o is then the gradient of the GATED output and fwd.o the gated output */
  int64_t dgate_stride[4];
  float* dmask;           /* optional out, fp32 [B,S,R] contiguous: gradient of an additive mask
                             (sum of dS over heads and queries; DS4Sci returns a gradient for both
                             biases, the reference returns None, evoformer.py:862).  Requests with
                             dmask set are served by the CUDA-core kernels */
  const struct evoattn_peer_allreduce_params* exchange;
                          /* optional (null: none): sum d(pair_bias) over the GPUs that share the MSA
                             rows as part of this call.  dbias must then be this rank's exchange buffer
                             (exchange->bufs[exchange->rank]) and exchange->count = B*H*R*R.  The sum is
                             launched as soon as d(pair_bias) is complete, on a stream of the library's
                             own, next to the call's remaining kernel; the call's stream then waits
                             for it, so everything the call returns is ordered on `cuda_stream` as usual */
} evoattn_bwd_params;

/* ABI version of the loaded library; compare with EVOATTN_ABI_VERSION. */
int evoattn_abi_version(void);

/* Human-readable text of a status code.  Never null. */
const char* evoattn_strerror(int status);

/* Forward pass.  Replaces the device side of EvoformerAttention.forward
 * (dsevoformer-triton/evoformer.py:635-737: the _attn_fwd launch at :676-724,
 * kernel at :103-297). */
int evoattn_fwd(const evoattn_fwd_params* p, void* cuda_stream);

/* Bytes of device scratch evoattn_bwd needs for these shapes (may be 0).
 * The reference allocates its scratch (delta, fp32 d_pair_bias) inside backward
 * (evoformer.py:749-758); here the caller does. */
size_t evoattn_bwd_workspace_bytes(const evoattn_bwd_params* p);

/* Backward pass.  Replaces the device side of EvoformerAttention.backward
 * (evoformer.py:741-862: _attn_bwd_preprocess :299-326, _attn_bwd_dk_dv :479-630,
 * _attn_bwd_dq :329-476). */
int evoattn_bwd(const evoattn_bwd_params* p, void* cuda_stream);

/* Backward pass for callers that cannot hand the library a scratch buffer.  It has no
 * counterpart in the reference.
 *
 * Some hosts of this library may not allocate device memory at the moment they need a
 * backward pass: a runtime whose memory pool is fixed when the process starts, a plugin that
 * runs inside someone else's allocator-free region, a serving loop with a frozen memory plan.
 * For them this entry point is evoattn_bwd() with the scratch taken from a fixed array that
 * is part of the library image (EVOATTN_STATIC_SCRATCH_BYTES of device memory on every GPU
 * that loads the library, held until the process exits).  `workspace` and `workspace_bytes`
 * in the parameters are ignored; inputs and outputs are still the caller's.
 *
 *  - A request that needs more than EVOATTN_STATIC_SCRATCH_BYTES of scratch (see
 *    evoattn_bwd_workspace_bytes) returns EVOATTN_ERR_WORKSPACE and launches nothing.
 *  - The function calls no cudaMalloc, cudaFree or any other allocating routine.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call before you start capturing a stream.
 *  - All calls share the one array.  Whatever has to start from zero is cleared on the stream
 *    by every call, but two calls that overlap on the GPU (different streams, no ordering)
 *    race on it: keep calls on one device ordered. */
#define EVOATTN_STATIC_SCRATCH_BYTES (64u << 20)
int evoattn_bwd_static_scratch(const evoattn_bwd_params* p, void* cuda_stream);

/* ---- Sum over the GPUs of one node through peer memory (for the N_seq-sharded op).
 *
 * These have no counterpart in the reference, which runs on one GPU: there d_pair_bias is
 * complete after the local atomics (evoformer.py:458) and the cast (:860).  When the MSA rows
 * are sharded over GPUs, every rank holds a partial fp32 d(pair_bias) and the sum over ranks is
 * the one exchange step of the path.  evoattn_peer_allreduce_f32 does it in place with one kernel
 * per rank over NVLink (plain stores into the peers' memory, flag barriers with bounded waits; no
 * multicast): all ranks call it with the same count and epoch, and afterwards every rank's
 * buffer holds the same bits.
 *
 * Set-up (once, outside the hot path; these are the only functions of the library that allocate):
 * each rank creates a data buffer of evoattn_peer_data_bytes(count, world) bytes (the first
 * count floats are the data, the rest is a staging area that peers write into) and a flag buffer
 * of evoattn_peer_flag_bytes(), sends the 64-byte handles to the other ranks (any transport), and
 * opens theirs. */
typedef struct evoattn_peer_allreduce_params {
  int32_t world;            /* GPUs taking part, 1..8 */
  int32_t rank;             /* this GPU's index */
  float* const* bufs;       /* host array [world]: every rank's data buffer as seen from this rank
                               (bufs[rank] is this rank's own); 256-byte aligned, each of at least
                               evoattn_peer_data_bytes(count, world) bytes */
  uint32_t* const* flags;   /* host array [world]: every rank's flag buffer, zero when created */
  uint64_t count;           /* floats to sum */
  uint32_t epoch;           /* 0: the library counts the calls on these buffers itself (in the flag
                               buffer; the form to use when the launch is replayed from a CUDA graph);
                               otherwise 1, 2, 3, ... : one more with every call.  Use one form only
                               on a given set of buffers */
  int32_t* status;          /* optional device word, set when a bounded wait runs out */
} evoattn_peer_allreduce_params;

/* Bytes of a data buffer that can take part in sums of up to `count` floats over `world` ranks. */
size_t evoattn_peer_data_bytes(uint64_t count, int world);
size_t evoattn_peer_flag_bytes(void);
/* cudaMalloc + clear + IPC handle of a buffer other ranks may open. */
int evoattn_peer_buffer_create(size_t bytes, void** dev_ptr, unsigned char handle_out[64]);
/* Map another rank's buffer (same node, NVLink / PCIe peer access). */
int evoattn_peer_buffer_open(const unsigned char handle[64], void** dev_ptr);
int evoattn_peer_buffer_close(void* dev_ptr);
int evoattn_peer_buffer_destroy(void* dev_ptr);
int evoattn_peer_allreduce_f32(const evoattn_peer_allreduce_params* p, void* cuda_stream);

/* ---- Pair bias in the layout a linear layer emits it, [B, R, R, H] (heads last).
 *
 * The reference takes the bias as [B, 1, H, R, R] (evoformer.py:638,652), which makes its caller
 * permute and copy an R*R*H tensor on every call, and the same for the gradient.  These two
 * kernels do that conversion on the device in one pass each; the second also casts the fp32
 * gradient to the bias type on the way.  `dtype` is the element type of the 16/32-bit side. */
int evoattn_bias_to_heads_first(const void* src_brrh, void* dst_bhrr, int dtype, int B, int H, int R, void* cuda_stream);
int evoattn_dbias_to_heads_last(const float* src_bhrr, void* dst_brrh, int dtype, int B, int H, int R, void* cuda_stream);

/* EVOATTN_PATH_* of the most recent forward / backward call made by this thread. */
int evoattn_last_path(void);

/* Number of kernels the most recent forward / backward call of this thread launched. */
int evoattn_last_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* EVOATTN_H_ */
