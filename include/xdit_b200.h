/*
 * xdit_b200 -- C ABI of the B200 (sm_100a) kernels behind xDiT's Unified-Sequence-Parallel
 * (USP) attention path.
 *
 * The reference is pure Python and has no FFI of its own; each entry point below replaces a
 * run of torch calls in the reference (cited as file:line inside the xDiT source tree) and
 * is what a Python/ctypes binding of that path binds.
 *
 * Conventions
 *   - every function returns 0 on success, a negative XDIT_E_* code for a rejected argument
 *     and a positive value (a cudaError_t) when the CUDA runtime reported an error;
 *     xdit_last_error_string() gives a human-readable reason for the calling thread;
 *   - no function allocates or frees device memory, and none synchronises the device: work is
 *     enqueued on `stream` (a cudaStream_t passed as void*; NULL is the legacy default stream);
 *   - pointers are device pointers unless stated otherwise; the caller keeps ownership;
 *   - strides are in ELEMENTS of the tensor's dtype; the innermost (head_dim) axis is
 *     contiguous everywhere;
 *   - kernels are built for sm_100a only; on any other device calls fail with
 *     XDIT_E_UNSUPPORTED_DEVICE.
 */
#ifndef XDIT_B200_H_
#define XDIT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XDIT_ABI_VERSION 3

#if defined(__GNUC__)
#define XDIT_API __attribute__((visibility("default")))
#else
#define XDIT_API
#endif

enum xdit_dtype { XDIT_BF16 = 0, XDIT_F16 = 1, XDIT_F32 = 2 };

enum xdit_status {
  XDIT_OK = 0,
  XDIT_E_NULL = -1,               /* a required pointer is NULL */
  XDIT_E_SHAPE = -2,              /* a size is zero, negative or out of the supported range */
  XDIT_E_ALIGN = -3,              /* a pointer or stride breaks an alignment rule */
  XDIT_E_DTYPE = -4,              /* unknown or unsupported dtype for this entry point */
  XDIT_E_UNSUPPORTED_DEVICE = -5, /* current device is not sm_100 */
  XDIT_E_KERNEL_TIMEOUT = -6,     /* a bounded wait inside a kernel gave up (xdit_attn_params.status / status_host) */
  XDIT_E_DRIVER = -7              /* a CUDA driver entry point could not be resolved */
};

struct xdit_caps {
  int abi_version;
  int device;
  int sm_major, sm_minor;
  int sm_count;
  int max_smem_per_block;
  int supported; /* 1 when the device is sm_100 and the tcgen05 path can run */
};

/* Diagnostics (proposed in place of Python exceptions raised by the reference). */
XDIT_API int xdit_query_caps(struct xdit_caps* out);
XDIT_API const char* xdit_last_error_string(void);

/* A sequence as the attention kernel sees it: `nseg` equally long segments of `seg_len`
 * rows.  After a Ulysses all-to-all every source rank's rows form one segment of the receive
 * buffer; a plain tensor is one segment.  Row r of segment g of head h of batch b starts at
 * ptr + b*stride_b + h*stride_h + g*stride_seg + r*stride_row  (elements). */
struct xdit_seq {
  const void* ptr;
  int64_t stride_b, stride_h, stride_seg, stride_row;
  int32_t nseg, seg_len;
};

/* Dense softmax attention forward, with the joint (replicated text) K/V as a second key/value
 * source and the ring-step merge fused into the epilogue.
 *
 * Replaces: the back-end call (q,k,v)->(out,lse) xfuser/core/distributed/attention_backend.py:492-566,
 * :887-918; torch.cat of joint K/V xfuser/model_executor/layers/usp.py:218-245 and
 * xfuser/core/long_ctx_attention/ring/ring_flash_attn.py:89-102; the post-all-to-all re-layout
 * copies usp.py:107,132; the partial-result merge (torch _SDPAMerger._merge_one; yunchang
 * update_out_and_lse called at ring_flash_attn.py:138).
 *
 * out has the segmentation of q.  lse/lse_acc are [B,H,Sq] fp32 contiguous and o_acc is
 * [B,H,Sq,D] fp32 contiguous, with Sq = q.nseg*q.seg_len rows in segment-major order.
 *   acc_in  != 0 : merge this call's (out,lse) into (o_acc,lse_acc) read from memory;
 *   acc_out != 0 : write the (merged) result to (o_acc,lse_acc) in fp32, leave `out` untouched;
 *   acc_out == 0 : write the (merged) result to `out` in `dtype` (and to `lse` when not NULL).
 * causal != 0 masks key j > query i (top-left aligned, the torch SDPA convention; flash-attn
 * aligns bottom-right, which differs when Sq != Sk), one segment only.
 * B and H are grid dimensions and must not exceed 65535. */
struct xdit_attn_params {
  int32_t dtype; /* xdit_dtype of q,k,v,out */
  int32_t B, H, D;
  struct xdit_seq q;   /* queries */
  struct xdit_seq k, v; /* main keys / values: same nseg and seg_len */
  struct xdit_seq k2, v2; /* joint keys / values (ptr NULL when absent): nseg must be 1 */
  void* out;
  int64_t out_stride_b, out_stride_h, out_stride_seg, out_stride_row;
  float* lse;     /* optional */
  float* o_acc;   /* required when acc_in or acc_out */
  float* lse_acc; /* required when acc_in or acc_out */
  int32_t acc_in, acc_out;
  int32_t causal;
  float softmax_scale; /* <= 0 selects D^-1/2 */
  int32_t force_generic; /* != 0: use the CUDA-core kernel even where the tcgen05 kernel applies */
  int32_t* status;       /* optional device int32: set non-zero when a bounded wait gave up */
  /* Failure reporting without polling.  Every wait inside the tcgen05 kernel is bounded in time
   * (wait_limit_ns; 0 selects 0.2 s).  When one runs out the launch drains, frees its TMEM, sets
   * *status (device) and, when status_host is given, the same code in *status_host: a 4-byte word
   * in pinned, device-mapped host memory (cudaHostAlloc) that the kernel only ever writes.  While
   * *status is non-zero later launches do no work, so that one failure does not cost a time limit
   * per CTA.  xdit_attn_fwd reads *status_host on entry (a plain host load, no synchronisation):
   * when it is non-zero the call launches nothing and returns XDIT_E_KERNEL_TIMEOUT, until the
   * caller has cleared both words (cudaMemsetAsync of *status, a store to *status_host).  A caller
   * that passes only `status` has to read it back itself after a synchronise. */
  int32_t* status_host;
  uint32_t wait_limit_ns;
  /* Test aid for the failure path: != 0 makes the tcgen05 kernel's loader leave the first K/V
   * stage un-armed, so that the consumer's bounded wait runs out after wait_limit_ns.  The launch
   * ends normally with the status words set and writes nothing to out. */
  int32_t selftest_stall;
  /* Output of a Ulysses exchange written where it is needed: when not NULL, a host array of q.nseg
   * device pointers; rows of query segment g go to out_segments[g] + b*out_stride_b + h*out_stride_h +
   * row*out_stride_row (elements) and `out` / out_stride_seg are ignored.  A pointer may be a peer GPU's
   * memory mapped into this process (xdit_peer_open): query segment g holds the rows of source rank g,
   * so the kernel's epilogue can store every rank's result rows straight into that rank's [B, s, H, D]
   * buffer with plain stores over NVLink -- the return all-to-all and the re-layout after it
   * (xfuser/model_executor/layers/usp.py:138-150) disappear into the epilogue.  The caller orders the
   * consumers on the other ranks after this launch (a collective or an event).  At most
   * XDIT_MAX_OUT_SEGMENTS segments; served by the tcgen05 kernel only (XDIT_E_DTYPE otherwise). */
  void* const* out_segments;
  /* Optional scratch that lets the tcgen05 kernel split the keys of a call over several CTAs per pair of
   * query tiles when the launch would otherwise fill at most half of the GPU's SMs (a Flux layer at Ulysses
   * degree 8 is 54 CTAs): every split writes a normalised fp32 partial result and its log-sum-exp here and a
   * second, small kernel merges them into the output (same formula as the ring merge).  Device memory,
   * 16-byte aligned, of split_scratch_bytes bytes; NULL / 0: never split.  Not used together with acc_in /
   * acc_out.  xdit_attn_split_scratch_bytes() gives the size that allows every split the library would
   * choose for a parameter block (0 when it would not split). */
  void* split_scratch;
  int64_t split_scratch_bytes;
};
#define XDIT_MAX_OUT_SEGMENTS 16
XDIT_API int xdit_attn_fwd(const struct xdit_attn_params* p, void* stream);
XDIT_API int64_t xdit_attn_split_scratch_bytes(const struct xdit_attn_params* p);
/* Which kernel xdit_attn_fwd would run for these parameters: 1 = tcgen05/TMEM/TMA kernel,
 * 0 = CUDA-core kernel, negative = the error the call would return. */
XDIT_API int xdit_attn_which(const struct xdit_attn_params* p);

/* Ring-step attention for callers that cannot allocate device memory.
 *
 * No counterpart in the reference (which allocates its merge buffers through torch).  Some
 * hosts of this library have no allocator to offer at the point of the call: a C or C++ serving
 * loop that was handed fixed input/output buffers, a plugin running under a framework whose
 * allocator it must not touch, or code that runs while allocation is forbidden.  For them this
 * variant of xdit_attn_fwd keeps the fp32 running accumulators of a ring sequence (what
 * xdit_attn_fwd takes as o_acc / lse_acc) in an array that is part of the library image
 * (XDIT_STATIC_ACC_FLOATS floats = 32 MiB, held by every GPU that loads the library until the
 * process exits).  The caller still passes q, k, v, the joint k2/v2, out and lse.
 *
 *   - p->o_acc and p->lse_acc must be NULL; at least one of acc_in / acc_out must be set
 *     (first step: acc_in=0, acc_out=1; middle steps: 1,1; last step: acc_in=1, acc_out=0);
 *   - B*H*Sq*D (rounded up to 64) + B*H*Sq floats must fit in XDIT_STATIC_ACC_FLOATS, otherwise
 *     the call returns XDIT_E_SHAPE and launches nothing;
 *   - the function calls no cudaMalloc/cudaFree and no allocating library routine.  The first
 *     call on each device looks the array's device address up (cudaGetSymbolAddress with that
 *     device current) and caches it; make that first call before starting a stream capture;
 *   - every call on a device shares the one array and the array keeps what the last call left.
 *     Nothing needs clearing as long as each sequence starts with acc_in=0, which overwrites the
 *     rows it uses.  Two sequences whose kernels overlap on the GPU (different streams, or
 *     interleaved steps) race on the array: keep one sequence at a time per device;
 *   - the cached address belongs to the device's primary context: after cudaDeviceReset() it is
 *     stale and the library does not notice, so a process that resets a device must not call this
 *     entry point on that device again. */
#define XDIT_STATIC_ACC_FLOATS (8 * 1024 * 1024)
XDIT_API int xdit_attn_fwd_static_acc(const struct xdit_attn_params* p, void* stream);

/* Ulysses input pack: [B,H,s,D] (any strides) plus optional joint rows -> the all-to-all send
 * buffer, peer-major.  For peer p the block at dst + p*dst_peer_stride holds
 * [H/U][B][s + s_joint][D] contiguous, i.e. heads [p*H/U,(p+1)*H/U) of the source; joint rows
 * are placed after (joint_front == 0) or before (joint_front != 0) the s source rows.
 * Up to XDIT_MAX_PACK_JOBS tensors (q, k, v) are packed by one launch.
 *
 * Replaces: x.permute(1,0,2,3).contiguous() usp.py:105, the stack/permute/contiguous of
 * usp.py:122-126 and the query concat usp.py:294 (hybrid/attn_layer.py:136-158, :185). */
#define XDIT_MAX_PACK_JOBS 4
struct xdit_pack_job {
  const void* src;
  int64_t src_stride_b, src_stride_h, src_stride_row;
  const void* joint; /* optional [B,H,s_joint,D] */
  int64_t joint_stride_b, joint_stride_h, joint_stride_row;
  void* dst;
  int64_t dst_peer_stride; /* elements between consecutive peers' blocks */
  int32_t s, s_joint, joint_front;
  /* Packing a group of heads only (the exchange of one head group can then run while another group is
   * being attended to): `H` of the call counts the group's heads over all peers, src / joint point at
   * the group's first head of peer 0, and these give the distance in elements between the first heads
   * of consecutive peers' blocks in src / joint.  0 selects (H/U) * stride_h, i.e. all heads. */
  int64_t src_stride_peer, joint_stride_peer;
};
XDIT_API int xdit_ulysses_pack(const struct xdit_pack_job* jobs, int32_t njobs, int32_t dtype, int32_t B,
                      int32_t H, int32_t D, int32_t U, void* stream);

/* The same pack, but peer p's block is written at peer_base[p] + dst_offset[j] (elements) for job j
 * instead of into one local send buffer: peer_base[p] is rank p's receive buffer mapped into this
 * process (xdit_peer_open; the own rank's entry is a local pointer).  The send buffer, the NCCL
 * all-to-all and its receive copy (usp.py:87-108) collapse into one pass of plain peer stores over NVLink.
 * jobs[j].dst and dst_peer_stride are ignored; U is at most XDIT_MAX_PACK_PEERS.  The caller orders the
 * readers on the other ranks after this launch. */
#define XDIT_MAX_PACK_PEERS 16
XDIT_API int xdit_ulysses_pack_peers(const struct xdit_pack_job* jobs, int32_t njobs, int32_t dtype, int32_t B,
                                     int32_t H, int32_t D, int32_t U, void* const* peer_base,
                                     const int64_t* dst_offset, void* stream);

/* Buffers that peer GPUs of the same node can store into (set-up, not hot path: these are the only entry
 * points that allocate).  xdit_peer_alloc: a device buffer from cudaMalloc on the current device plus a
 * 64-byte handle for other processes; xdit_peer_open: map a peer's buffer from its handle (enables peer
 * access); xdit_peer_close / xdit_peer_free release them.  No counterpart in the reference, which moves
 * everything through NCCL collectives. */
#define XDIT_PEER_HANDLE_BYTES 64
XDIT_API int xdit_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle /*[XDIT_PEER_HANDLE_BYTES]*/);
XDIT_API int xdit_peer_open(const unsigned char* handle, void** ptr);
XDIT_API int xdit_peer_close(void* ptr);
XDIT_API int xdit_peer_free(void* ptr);

/* Barrier between the U ranks whose buffers are mapped into each other: rank `rank` stores its barrier
 * count into word `rank` of every rank's flag array (peer_flags[r]: rank r's array of U uint32 words,
 * mapped into this process; the own entry is local_flags) and waits until every word of local_flags has
 * reached the same count.  `epoch` is a uint32 in this rank's device memory, zero at set-up, advanced by
 * the kernel (so a captured launch replays).  The wait is bounded by wait_limit_ns (0: 2 s); when it runs
 * out, *status / *status_host are set like xdit_attn_params.status / status_host (code 400 + the rank that
 * did not arrive) and the kernel returns; while *status is non-zero barriers do not wait.  Every rank must
 * call it the same number of times.  No counterpart in the reference. */
XDIT_API int xdit_peer_barrier(void* const* peer_flags, void* local_flags, void* epoch, int32_t U, int32_t rank,
                               uint32_t wait_limit_ns, int32_t* status, int32_t* status_host, void* stream);

/* One asynchronous copy of `bytes` bytes from this GPU's memory into a buffer that may be a peer's
 * (xdit_peer_open), issued on `stream` as a single cudaMemcpyAsync: the copy engines move it over NVLink
 * and no SM is used.  The ring K/V rotation uses it in place of an NCCL send/recv pair
 * (usp.py:46-74 via torch's ring rotater; ring_flash_attn.py:84-87,140-143), whose kernels would hold SMs
 * that the attention kernel, with one CTA per SM, then has to do without.  The caller orders the readers
 * with xdit_peer_barrier after the copy. */
XDIT_API int xdit_peer_copy(void* dst, const void* src, int64_t bytes, void* stream);

/* Ulysses output pack in the reference's own wire layout: [B,Hl,S,D] (any strides) ->
 * send buffer [S][B][Hl][D] contiguous (peer p's block = rows [p*S/U,(p+1)*S/U)), and the
 * inverse on the receive side: [U][s][B][Hl][D] -> [B][U*Hl][s][D] contiguous.
 * Replaces: usp.py:147 (permute(2,0,1,3).contiguous()) and usp.py:149. */
XDIT_API int xdit_ulysses_pack_out(const void* src, int64_t stride_b, int64_t stride_h, int64_t stride_row,
                          void* dst, int32_t dtype, int32_t B, int32_t Hl, int32_t S, int32_t D,
                          void* stream);
XDIT_API int xdit_ulysses_unpack_out(const void* recv, void* dst, int32_t dtype, int32_t B, int32_t Hl,
                            int32_t s, int32_t D, int32_t U, void* stream);

/* Ulysses input unpack in the reference's wire layout: recv [U][Hl][B][s][D] -> [B][Hl][U*s][D]
 * contiguous.  Replaces usp.py:107 for callers that need the materialised tensor. */
XDIT_API int xdit_ulysses_unpack_in(const void* recv, void* dst, int32_t dtype, int32_t B, int32_t Hl,
                           int32_t s, int32_t D, int32_t U, void* stream);

/* Sequence sharding at the model boundary.
 *
 * xdit_seq_shard_pad: the rows of src [B,S,C] (element strides stride_b, stride_row; C contiguous)
 * that sequence-parallel rank `rank` of W owns after S has been zero-padded up to a multiple of W:
 * dst [B, s, C] contiguous with s = ceil(S/W), rows at or past S written as zeros.  One pass over the
 * local rows only.  Replaces: torch.cat([x, zeros]) + torch.chunk(...)[rank]
 * (xfuser/model_executor/models/transformers/transformer_wan.py:219-234 _chunk_and_pad_sequence;
 * transformer_flux.py:279-284, 307-309).
 *
 * xdit_seq_gather_unpad: recv [W][B][s][C] (what all_gather_into_tensor leaves) -> dst [B][keep][C],
 * keep = W*s - padding rows, i.e. the gathered sequence with the padding dropped, in one pass.
 * Replaces: reshape([W,...]).movedim(0, dim).reshape(...) of GroupCoordinator.all_gather
 * (xfuser/core/distributed/group_coordinator.py:243-262) and the narrow / slice that drops the
 * padding (transformer_wan.py:236-239 _gather_and_unpad; transformer_flux.py:333-336). */
XDIT_API int xdit_seq_shard_pad(const void* src, int64_t stride_b, int64_t stride_row, void* dst,
                                int32_t dtype, int32_t B, int32_t S, int32_t C, int32_t W, int32_t rank,
                                void* stream);
XDIT_API int xdit_seq_gather_unpad(const void* recv, void* dst, int32_t dtype, int32_t W, int32_t B,
                                   int32_t s, int32_t C, int32_t keep, void* stream);

/* PipeFusion stale-KV patch update: overwrite rows [row_start, row_start + nseg*n) of the
 * persistent K and V caches (attention layout, strides given) with fresh rows.  The fresh rows
 * come as `nseg` segments of `n` rows (one segment per Ulysses source rank; nseg = 1 without
 * sequence parallelism); segment g lands at cache rows row_start + g*n.
 *
 * Replaces: torch.cat(new_kv,-1) cache_manager.py:76, the slice-assign of
 * cache_manager.py:127-133 / :172-192 -> _update_kv_in_dim :196-219, torch.chunk :99 and the
 * two .contiguous() copies of usp.py:201-202 / ring_flash_attn.py:80-81. */
struct xdit_kv_patch_params {
  int32_t dtype, B, H, D;
  void* k_cache; void* v_cache;
  int64_t cache_stride_b, cache_stride_h, cache_stride_row; /* same for both caches */
  int32_t cache_rows;
  struct xdit_seq k_new, v_new; /* nseg segments of seg_len = n rows */
  int32_t row_start;
};
XDIT_API int xdit_kv_patch_update(const struct xdit_kv_patch_params* p, void* stream);

/* Stand-alone online-softmax merge of a partial result into fp32 accumulators:
 *   o_acc <- o_acc - sigmoid(lse_b - lse_acc) * (o_acc - out_b);
 *   lse_acc <- lse_acc - logsigmoid(lse_acc - lse_b)
 * over `rows` rows of D elements; first != 0 initialises the accumulators from the block.
 * out_final (optional, dtype) receives the merged rows cast to `dtype`.
 * Replaces: torch _SDPAMerger.step / yunchang update_out_and_lse (ring_flash_attn.py:138). */
XDIT_API int xdit_merge_out_lse(float* o_acc, float* lse_acc, const void* out_b, const float* lse_b,
                       void* out_final, int32_t dtype, int64_t rows, int32_t D, int32_t first,
                       void* stream);

/* Attention prologue of the DiT processors fused with the Ulysses pack, for the projections of one
 * layer: q and k are RMS-normalised (over all H*D elements of a token when norm_per_head == 0, over
 * each head's D elements otherwise; a NULL weight skips the norm of that tensor), rotated
 * (interleaved pairs (2i, 2i+1): out[2i] = x1*cos[2i] - x2*sin[2i+1], out[2i+1] = x1*sin[2i+1] +
 * x2*cos[2i]; NULL cos skips it), split into heads and written, together with v, in the all-to-all
 * send layout [U][H/U][B][s][D] (peer blocks dst_*_peer_stride elements apart; U = 1 gives
 * [H][B][s][D]).  q, k, v: [B, s, H*D] with element strides, innermost contiguous; weights [H*D]
 * (or [D] with norm_per_head) in `dtype`; cos, sin: fp32 [s, D] rows cos_sin_stride_row apart.
 * dtype bf16 or fp16; D % 8 == 0; H*D <= 8192; with norm_per_head D/8 must be a power of two <= 32.
 * Replaces: norm_q / norm_k, the inline apply_rotary_emb, unflatten + transpose
 * (xfuser/model_executor/models/transformers/transformer_wan.py:97-122, 143-147; the same steps at
 * transformer_flux.py:113-147, 170-172) and the re-layout copies of _ft_c_input_all_to_all
 * (xfuser/model_executor/layers/usp.py:96-108). */
struct xdit_prologue_params {
  int32_t dtype;
  int32_t B, H, D, s, U;
  int32_t norm_per_head;
  float eps;
  const void *q, *k, *v;
  int64_t q_stride_b, q_stride_row, k_stride_b, k_stride_row, v_stride_b, v_stride_row;
  const void *norm_q_weight, *norm_k_weight;
  const float *cos, *sin;
  int64_t cos_sin_stride_row;
  void *dst_q, *dst_k, *dst_v;
  int64_t dst_q_peer_stride, dst_k_peer_stride, dst_v_peer_stride;
  /* Placement inside a peer's block, per tensor (q, k, v): elements between consecutive heads and between
   * consecutive batches of the destination; rows are always D elements apart.  0 selects the packed send
   * layout [H/U][B][s][D] (head stride B*s*D, batch stride s*D).  Other values let a tensor land somewhere
   * else in one pass, e.g. the fresh K and V rows of a PipeFusion patch straight in the layer's persistent
   * [B,H,S,D] stale-KV buffers (dst = buffer + row_start*D, head stride S*D, batch stride H*S*D), which
   * replaces the separate patch update of xdit_kv_patch_update for callers that own the projections. */
  int64_t dst_stride_h[3], dst_stride_b[3];
};
XDIT_API int xdit_qk_norm_rope_pack(const struct xdit_prologue_params* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XDIT_B200_H_ */
