// extern "C" entry points of libxdit_b200: argument checking and translation of the
// domain-level parameters (Ulysses peers, joint rows, KV patches) into kernel launches.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace xdit {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_device(int* sm_count) {
  // Cached per device: the attributes do not change while the process lives.
  static std::mutex mu;
  static int cached_dev[16], cached_major[16], cached_sms[16], ncached = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  int major = -1, sms = 0;
  {
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < ncached; ++i)
      if (cached_dev[i] == dev) { major = cached_major[i]; sms = cached_sms[i]; }
    if (major < 0) {
      e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
      if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
      if (ncached < 16) {
        cached_dev[ncached] = dev; cached_major[ncached] = major; cached_sms[ncached] = sms;
        ++ncached;
      }
    }
  }
  if (major != 10) {
    set_error("device %d is sm_%d?: this library is built for sm_100a only", dev, major);
    return XDIT_E_UNSUPPORTED_DEVICE;
  }
  if (sm_count) *sm_count = sms;
  return XDIT_OK;
}

}  // namespace xdit

using namespace xdit;

extern "C" {

const char* xdit_last_error_string(void) { return g_err; }

int xdit_query_caps(struct xdit_caps* out) {
  if (!out) { set_error("xdit_query_caps: NULL out"); return XDIT_E_NULL; }
  out->abi_version = XDIT_ABI_VERSION;
  out->supported = 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  out->device = dev;
  cudaDeviceGetAttribute(&out->sm_major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&out->sm_minor, cudaDevAttrComputeCapabilityMinor, dev);
  cudaDeviceGetAttribute(&out->sm_count, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&out->max_smem_per_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  out->supported = (out->sm_major == 10) ? 1 : 0;
  return XDIT_OK;
}

}  // extern "C"

namespace xdit {
// Shared body of xdit_ulysses_pack (one local send buffer, peers a fixed stride apart) and
// xdit_ulysses_pack_peers (one base pointer per peer).
static int pack_impl(const char* who, const struct xdit_pack_job* jobs, int32_t njobs, int32_t dtype, int32_t B,
                     int32_t H, int32_t D, int32_t U, void* const* peer_base, const int64_t* dst_offset,
                     void* stream) {
  const int es = dtype_size(dtype);
  if (!es) { set_error("%s: bad dtype %d", who, dtype); return XDIT_E_DTYPE; }
  if (!jobs) { set_error("%s: NULL jobs", who); return XDIT_E_NULL; }
  if (njobs < 1 || njobs > XDIT_MAX_PACK_JOBS) {
    set_error("%s: njobs=%d (1..%d)", who, njobs, XDIT_MAX_PACK_JOBS);
    return XDIT_E_SHAPE;
  }
  if (B < 1 || H < 1 || D < 1 || U < 1 || H % U != 0) {
    set_error("%s: B=%d H=%d D=%d U=%d (H must be divisible by U)", who, B, H, D, U);
    return XDIT_E_SHAPE;
  }
  const int Hl = H / U;
  if (peer_base && U > kMaxRowCopyPeers) {
    set_error("%s: U=%d peers (at most %d)", who, U, kMaxRowCopyPeers);
    return XDIT_E_SHAPE;
  }
  RowCopyJob rc[kMaxRowCopyJobs];
  int n = 0;
  for (int j = 0; j < njobs; ++j) {
    const xdit_pack_job& pj = jobs[j];
    if (pj.s < 0 || pj.s_joint < 0 || pj.s + pj.s_joint == 0) {
      set_error("%s: job %d has s=%d s_joint=%d", who, j, pj.s, pj.s_joint);
      return XDIT_E_SHAPE;
    }
    if ((!peer_base && !pj.dst) || (pj.s && !pj.src) || (pj.s_joint && !pj.joint)) {
      set_error("%s: NULL pointer in job %d", who, j);
      return XDIT_E_NULL;
    }
    const int64_t rows = (int64_t)pj.s + pj.s_joint;
    // destination dims: (peer, head-in-peer, batch, row); with per-peer bases the peer index picks
    // the base and the job's destination is the offset inside every peer's buffer
    const int64_t d_row = (int64_t)D * es;
    const int64_t d_b = rows * d_row;
    const int64_t d_h = B * d_b;
    const int64_t d_p = peer_base ? 0 : pj.dst_peer_stride * es;
    const int main_off = pj.joint_front ? pj.s_joint : 0;
    const int joint_off = pj.joint_front ? 0 : pj.s;
    const int64_t sp_main = (pj.src_stride_peer ? pj.src_stride_peer : (int64_t)Hl * pj.src_stride_h) * es;
    const int64_t sp_joint = (pj.joint_stride_peer ? pj.joint_stride_peer : (int64_t)Hl * pj.joint_stride_h) * es;
    char* dbase = peer_base ? reinterpret_cast<char*>(static_cast<intptr_t>(dst_offset[j] * es)) : (char*)pj.dst;
    if (pj.s) {
      RowCopyJob& r = rc[n++];
      r.src = (const char*)pj.src;
      r.dst = dbase + main_off * d_row;
      r.n[0] = U; r.n[1] = Hl; r.n[2] = B; r.n[3] = pj.s;
      r.s_stride[0] = sp_main; r.s_stride[1] = pj.src_stride_h * es;
      r.s_stride[2] = pj.src_stride_b * es; r.s_stride[3] = pj.src_stride_row * es;
      r.d_stride[0] = d_p; r.d_stride[1] = d_h; r.d_stride[2] = d_b; r.d_stride[3] = d_row;
      r.row_bytes = D * es;
    }
    if (pj.s_joint) {
      RowCopyJob& r = rc[n++];
      r.src = (const char*)pj.joint;
      r.dst = dbase + joint_off * d_row;
      r.n[0] = U; r.n[1] = Hl; r.n[2] = B; r.n[3] = pj.s_joint;
      r.s_stride[0] = sp_joint; r.s_stride[1] = pj.joint_stride_h * es;
      r.s_stride[2] = pj.joint_stride_b * es; r.s_stride[3] = pj.joint_stride_row * es;
      r.d_stride[0] = d_p; r.d_stride[1] = d_h; r.d_stride[2] = d_b; r.d_stride[3] = d_row;
      r.row_bytes = D * es;
    }
  }
  return launch_row_copy(rc, n, (cudaStream_t)stream, peer_base, peer_base ? U : 0);
}
}  // namespace xdit

extern "C" {

int xdit_ulysses_pack(const struct xdit_pack_job* jobs, int32_t njobs, int32_t dtype, int32_t B,
                      int32_t H, int32_t D, int32_t U, void* stream) {
  return pack_impl("xdit_ulysses_pack", jobs, njobs, dtype, B, H, D, U, nullptr, nullptr, stream);
}

int xdit_ulysses_pack_peers(const struct xdit_pack_job* jobs, int32_t njobs, int32_t dtype, int32_t B, int32_t H,
                            int32_t D, int32_t U, void* const* peer_base, const int64_t* dst_offset, void* stream) {
  if (!peer_base || !dst_offset) { set_error("xdit_ulysses_pack_peers: NULL peer_base / dst_offset"); return XDIT_E_NULL; }
  return pack_impl("xdit_ulysses_pack_peers", jobs, njobs, dtype, B, H, D, U, peer_base, dst_offset, stream);
}

// ---- buffers that peer GPUs can store into (set-up path) ----------------------------------------
int xdit_peer_alloc(int64_t bytes, void** ptr, unsigned char* handle) {
  if (!ptr || !handle) { set_error("xdit_peer_alloc: NULL argument"); return XDIT_E_NULL; }
  if (bytes < 1) { set_error("xdit_peer_alloc: bytes=%lld", (long long)bytes); return XDIT_E_SHAPE; }
  static_assert(sizeof(cudaIpcMemHandle_t) == XDIT_PEER_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return cuda_fail(e, "xdit_peer_alloc: cudaMalloc");
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "xdit_peer_alloc: cudaIpcGetMemHandle"); }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return XDIT_OK;
}

int xdit_peer_open(const unsigned char* handle, void** ptr) {
  if (!ptr || !handle) { set_error("xdit_peer_open: NULL argument"); return XDIT_E_NULL; }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e, "xdit_peer_open: cudaIpcOpenMemHandle");
  *ptr = p;
  return XDIT_OK;
}

int xdit_peer_close(void* ptr) {
  if (!ptr) return XDIT_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return cuda_fail(e, "xdit_peer_close: cudaIpcCloseMemHandle");
  return XDIT_OK;
}

int xdit_peer_free(void* ptr) {
  if (!ptr) return XDIT_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return cuda_fail(e, "xdit_peer_free: cudaFree");
  return XDIT_OK;
}

int xdit_peer_copy(void* dst, const void* src, int64_t bytes, void* stream) {
  if (!dst || !src) { set_error("xdit_peer_copy: NULL pointer"); return XDIT_E_NULL; }
  if (bytes < 0) { set_error("xdit_peer_copy: bytes=%lld", (long long)bytes); return XDIT_E_SHAPE; }
  if (bytes == 0) return XDIT_OK;
  cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "xdit_peer_copy: cudaMemcpyAsync");
  return XDIT_OK;
}

int xdit_qk_norm_rope_pack(const struct xdit_prologue_params* p, void* stream) {
  if (!p) { set_error("xdit_qk_norm_rope_pack: NULL params"); return XDIT_E_NULL; }
  if (p->dtype != XDIT_BF16 && p->dtype != XDIT_F16) {
    set_error("xdit_qk_norm_rope_pack: dtype %d (bf16 or fp16)", p->dtype);
    return XDIT_E_DTYPE;
  }
  if (p->B < 1 || p->H < 1 || p->D < 8 || p->s < 1 || p->U < 1 || p->H % p->U || p->D % 8 ||
      (int64_t)p->H * p->D > 8192) {
    set_error("xdit_qk_norm_rope_pack: B=%d H=%d D=%d s=%d U=%d (D %% 8 == 0, H %% U == 0, H*D <= 8192)", p->B, p->H,
              p->D, p->s, p->U);
    return XDIT_E_SHAPE;
  }
  const int vpd = p->D / 8;
  if (p->norm_per_head && (p->norm_q_weight || p->norm_k_weight) && (vpd > 32 || (vpd & (vpd - 1)))) {
    set_error("xdit_qk_norm_rope_pack: per-head norm needs D/8 to be a power of two up to 32 (D=%d)", p->D);
    return XDIT_E_SHAPE;
  }
  if (!p->q || !p->k || !p->v || !p->dst_q || !p->dst_k || !p->dst_v || ((p->cos == nullptr) != (p->sin == nullptr))) {
    set_error("xdit_qk_norm_rope_pack: NULL pointer (cos and sin go together)");
    return XDIT_E_NULL;
  }
  const uintptr_t ptrs = (uintptr_t)p->q | (uintptr_t)p->k | (uintptr_t)p->v | (uintptr_t)p->dst_q |
                         (uintptr_t)p->dst_k | (uintptr_t)p->dst_v | (uintptr_t)p->norm_q_weight |
                         (uintptr_t)p->norm_k_weight | (uintptr_t)p->cos | (uintptr_t)p->sin;
  int64_t strides = p->q_stride_b | p->q_stride_row | p->k_stride_b | p->k_stride_row | p->v_stride_b |
                    p->v_stride_row | p->dst_q_peer_stride | p->dst_k_peer_stride | p->dst_v_peer_stride;
  for (int i = 0; i < 3; ++i) {
    if (p->dst_stride_h[i] < 0 || p->dst_stride_b[i] < 0) {
      set_error("xdit_qk_norm_rope_pack: negative destination stride");
      return XDIT_E_SHAPE;
    }
    strides |= p->dst_stride_h[i] | p->dst_stride_b[i];
  }
  if ((ptrs & 15) || (strides & 7) || (p->cos && (p->cos_sin_stride_row & 3))) {
    set_error("xdit_qk_norm_rope_pack: pointers must be 16-byte aligned and strides multiples of 8 elements");
    return XDIT_E_ALIGN;
  }
  return launch_prologue(*p, (cudaStream_t)stream);
}

int xdit_ulysses_pack_out(const void* src, int64_t stride_b, int64_t stride_h, int64_t stride_row,
                          void* dst, int32_t dtype, int32_t B, int32_t Hl, int32_t S, int32_t D,
                          void* stream) {
  const int es = dtype_size(dtype);
  if (!es) { set_error("xdit_ulysses_pack_out: bad dtype %d", dtype); return XDIT_E_DTYPE; }
  if (!src || !dst) { set_error("xdit_ulysses_pack_out: NULL pointer"); return XDIT_E_NULL; }
  if (B < 1 || Hl < 1 || S < 1 || D < 1) { set_error("xdit_ulysses_pack_out: bad shape"); return XDIT_E_SHAPE; }
  // dst [S][B][Hl][D]; iterate (1, b, h, row) so that the long axis is innermost
  RowCopyJob r;
  r.src = (const char*)src; r.dst = (char*)dst;
  r.n[0] = 1; r.n[1] = B; r.n[2] = Hl; r.n[3] = S;
  r.s_stride[0] = 0; r.s_stride[1] = stride_b * es; r.s_stride[2] = stride_h * es; r.s_stride[3] = stride_row * es;
  const int64_t row = (int64_t)D * es;
  r.d_stride[0] = 0; r.d_stride[1] = Hl * row; r.d_stride[2] = row; r.d_stride[3] = (int64_t)B * Hl * row;
  r.row_bytes = D * es;
  return launch_row_copy(&r, 1, (cudaStream_t)stream);
}

int xdit_ulysses_unpack_out(const void* recv, void* dst, int32_t dtype, int32_t B, int32_t Hl,
                            int32_t s, int32_t D, int32_t U, void* stream) {
  const int es = dtype_size(dtype);
  if (!es) { set_error("xdit_ulysses_unpack_out: bad dtype %d", dtype); return XDIT_E_DTYPE; }
  if (!recv || !dst) { set_error("xdit_ulysses_unpack_out: NULL pointer"); return XDIT_E_NULL; }
  if (B < 1 || Hl < 1 || s < 1 || D < 1 || U < 1) { set_error("xdit_ulysses_unpack_out: bad shape"); return XDIT_E_SHAPE; }
  // recv [U][s][B][Hl][D] -> dst [B][U][Hl][s][D]; dims (u, b, h, row)
  const int64_t row = (int64_t)D * es;
  RowCopyJob r;
  r.src = (const char*)recv; r.dst = (char*)dst;
  r.n[0] = U; r.n[1] = B; r.n[2] = Hl; r.n[3] = s;
  r.s_stride[0] = (int64_t)s * B * Hl * row; r.s_stride[1] = Hl * row; r.s_stride[2] = row;
  r.s_stride[3] = (int64_t)B * Hl * row;
  r.d_stride[0] = (int64_t)Hl * s * row; r.d_stride[1] = (int64_t)U * Hl * s * row;
  r.d_stride[2] = (int64_t)s * row; r.d_stride[3] = row;
  r.row_bytes = D * es;
  return launch_row_copy(&r, 1, (cudaStream_t)stream);
}

int xdit_ulysses_unpack_in(const void* recv, void* dst, int32_t dtype, int32_t B, int32_t Hl,
                           int32_t s, int32_t D, int32_t U, void* stream) {
  const int es = dtype_size(dtype);
  if (!es) { set_error("xdit_ulysses_unpack_in: bad dtype %d", dtype); return XDIT_E_DTYPE; }
  if (!recv || !dst) { set_error("xdit_ulysses_unpack_in: NULL pointer"); return XDIT_E_NULL; }
  if (B < 1 || Hl < 1 || s < 1 || D < 1 || U < 1) { set_error("xdit_ulysses_unpack_in: bad shape"); return XDIT_E_SHAPE; }
  // recv [U][Hl][B][s][D] -> dst [B][Hl][U][s][D]; dims (u, h, b, row)
  const int64_t row = (int64_t)D * es;
  RowCopyJob r;
  r.src = (const char*)recv; r.dst = (char*)dst;
  r.n[0] = U; r.n[1] = Hl; r.n[2] = B; r.n[3] = s;
  r.s_stride[0] = (int64_t)Hl * B * s * row; r.s_stride[1] = (int64_t)B * s * row;
  r.s_stride[2] = (int64_t)s * row; r.s_stride[3] = row;
  r.d_stride[0] = (int64_t)s * row; r.d_stride[1] = (int64_t)U * s * row;
  r.d_stride[2] = (int64_t)Hl * U * s * row; r.d_stride[3] = row;
  r.row_bytes = D * es;
  return launch_row_copy(&r, 1, (cudaStream_t)stream);
}

int xdit_seq_shard_pad(const void* src, int64_t stride_b, int64_t stride_row, void* dst, int32_t dtype,
                       int32_t B, int32_t S, int32_t C, int32_t W, int32_t rank, void* stream) {
  const int es = dtype_size(dtype);
  if (!es) { set_error("xdit_seq_shard_pad: bad dtype %d", dtype); return XDIT_E_DTYPE; }
  if (!src || !dst) { set_error("xdit_seq_shard_pad: NULL pointer"); return XDIT_E_NULL; }
  if (B < 1 || S < 1 || C < 1 || W < 1 || rank < 0 || rank >= W) {
    set_error("xdit_seq_shard_pad: B=%d S=%d C=%d W=%d rank=%d", B, S, C, W, rank);
    return XDIT_E_SHAPE;
  }
  const int s = (S + W - 1) / W;            // rows per rank after padding S up to a multiple of W
  const int first = rank * s;
  const int valid = first >= S ? 0 : (S - first < s ? S - first : s);
  const int64_t row = (int64_t)C * es;
  RowCopyJob rc[2];
  int n = 0;
  if (valid > 0) {
    RowCopyJob& r = rc[n++];
    r.src = (const char*)src + (int64_t)first * stride_row * es;
    r.dst = (char*)dst;
    r.n[0] = 1; r.n[1] = 1; r.n[2] = B; r.n[3] = valid;
    r.s_stride[0] = 0; r.s_stride[1] = 0; r.s_stride[2] = stride_b * es; r.s_stride[3] = stride_row * es;
    r.d_stride[0] = 0; r.d_stride[1] = 0; r.d_stride[2] = (int64_t)s * row; r.d_stride[3] = row;
    r.row_bytes = (int32_t)row;
  }
  if (valid < s) {  // zero rows past the end of the sequence
    RowCopyJob& r = rc[n++];
    r.src = nullptr;
    r.dst = (char*)dst + (int64_t)valid * row;
    r.n[0] = 1; r.n[1] = 1; r.n[2] = B; r.n[3] = s - valid;
    r.s_stride[0] = r.s_stride[1] = r.s_stride[2] = r.s_stride[3] = 0;
    r.d_stride[0] = 0; r.d_stride[1] = 0; r.d_stride[2] = (int64_t)s * row; r.d_stride[3] = row;
    r.row_bytes = (int32_t)row;
  }
  return launch_row_copy(rc, n, (cudaStream_t)stream);
}

int xdit_seq_gather_unpad(const void* recv, void* dst, int32_t dtype, int32_t W, int32_t B, int32_t s,
                          int32_t C, int32_t keep, void* stream) {
  const int es = dtype_size(dtype);
  if (!es) { set_error("xdit_seq_gather_unpad: bad dtype %d", dtype); return XDIT_E_DTYPE; }
  if (!recv || !dst) { set_error("xdit_seq_gather_unpad: NULL pointer"); return XDIT_E_NULL; }
  if (W < 1 || B < 1 || s < 1 || C < 1 || keep < 1 || keep > (int64_t)W * s) {
    set_error("xdit_seq_gather_unpad: W=%d B=%d s=%d C=%d keep=%d", W, B, s, C, keep);
    return XDIT_E_SHAPE;
  }
  // recv [W][B][s][C] -> dst [B][keep][C]; source rank w contributes rows [w*s, min((w+1)*s, keep))
  const int64_t row = (int64_t)C * es;
  const int full = keep / s;          // ranks whose rows are all kept
  const int tail = keep - full * s;   // kept rows of the next rank
  RowCopyJob rc[2];
  int n = 0;
  if (full > 0) {
    RowCopyJob& r = rc[n++];
    r.src = (const char*)recv; r.dst = (char*)dst;
    r.n[0] = 1; r.n[1] = full; r.n[2] = B; r.n[3] = s;
    r.s_stride[0] = 0; r.s_stride[1] = (int64_t)B * s * row; r.s_stride[2] = (int64_t)s * row; r.s_stride[3] = row;
    r.d_stride[0] = 0; r.d_stride[1] = (int64_t)s * row; r.d_stride[2] = (int64_t)keep * row; r.d_stride[3] = row;
    r.row_bytes = (int32_t)row;
  }
  if (tail > 0) {
    RowCopyJob& r = rc[n++];
    r.src = (const char*)recv + (int64_t)full * B * s * row; r.dst = (char*)dst + (int64_t)full * s * row;
    r.n[0] = 1; r.n[1] = 1; r.n[2] = B; r.n[3] = tail;
    r.s_stride[0] = 0; r.s_stride[1] = 0; r.s_stride[2] = (int64_t)s * row; r.s_stride[3] = row;
    r.d_stride[0] = 0; r.d_stride[1] = 0; r.d_stride[2] = (int64_t)keep * row; r.d_stride[3] = row;
    r.row_bytes = (int32_t)row;
  }
  return launch_row_copy(rc, n, (cudaStream_t)stream);
}

int xdit_kv_patch_update(const struct xdit_kv_patch_params* p, void* stream) {
  if (!p) { set_error("xdit_kv_patch_update: NULL params"); return XDIT_E_NULL; }
  const int es = dtype_size(p->dtype);
  if (!es) { set_error("xdit_kv_patch_update: bad dtype %d", p->dtype); return XDIT_E_DTYPE; }
  if (!p->k_cache || !p->v_cache || !p->k_new.ptr || !p->v_new.ptr) {
    set_error("xdit_kv_patch_update: NULL pointer");
    return XDIT_E_NULL;
  }
  if (p->B < 1 || p->H < 1 || p->D < 1 || p->k_new.nseg < 1 || p->k_new.seg_len < 1 ||
      p->v_new.nseg != p->k_new.nseg || p->v_new.seg_len != p->k_new.seg_len) {
    set_error("xdit_kv_patch_update: bad shape");
    return XDIT_E_SHAPE;
  }
  const int64_t nrows = (int64_t)p->k_new.nseg * p->k_new.seg_len;
  if (p->row_start < 0 || p->row_start + nrows > p->cache_rows) {
    set_error("xdit_kv_patch_update: rows [%d,%lld) outside the cache of %d rows", p->row_start,
              (long long)(p->row_start + nrows), p->cache_rows);
    return XDIT_E_SHAPE;
  }
  RowCopyJob rc[2];
  const xdit_seq* srcs[2] = {&p->k_new, &p->v_new};
  void* dsts[2] = {p->k_cache, p->v_cache};
  for (int i = 0; i < 2; ++i) {
    RowCopyJob& r = rc[i];
    const xdit_seq& s = *srcs[i];
    r.src = (const char*)s.ptr;
    r.dst = (char*)dsts[i] + (int64_t)p->row_start * p->cache_stride_row * es;
    r.n[0] = p->B; r.n[1] = p->H; r.n[2] = s.nseg; r.n[3] = s.seg_len;
    r.s_stride[0] = s.stride_b * es; r.s_stride[1] = s.stride_h * es;
    r.s_stride[2] = s.stride_seg * es; r.s_stride[3] = s.stride_row * es;
    r.d_stride[0] = p->cache_stride_b * es; r.d_stride[1] = p->cache_stride_h * es;
    r.d_stride[2] = (int64_t)s.seg_len * p->cache_stride_row * es;
    r.d_stride[3] = p->cache_stride_row * es;
    r.row_bytes = p->D * es;
  }
  return launch_row_copy(rc, 2, (cudaStream_t)stream);
}

}  // extern "C"
namespace xdit {
int attn_check(const struct xdit_attn_params* p) {
  if (!p) { set_error("xdit_attn_fwd: NULL params"); return XDIT_E_NULL; }
  if (!dtype_size(p->dtype)) { set_error("xdit_attn_fwd: bad dtype %d", p->dtype); return XDIT_E_DTYPE; }
  if (p->B < 1 || p->H < 1 || p->D < 1 || p->D > 256 || p->B > 65535 || p->H > 65535) {
    set_error("xdit_attn_fwd: B=%d H=%d D=%d (D must be 1..256, B and H at most 65535)", p->B, p->H, p->D);
    return XDIT_E_SHAPE;
  }
  if (!p->q.ptr || !p->k.ptr || !p->v.ptr) { set_error("xdit_attn_fwd: NULL q/k/v"); return XDIT_E_NULL; }
  if (p->q.nseg < 1 || p->q.seg_len < 1 || p->k.nseg < 1 || p->k.seg_len < 1 ||
      p->v.nseg != p->k.nseg || p->v.seg_len != p->k.seg_len) {
    set_error("xdit_attn_fwd: bad segment shape (q %dx%d, k %dx%d, v %dx%d)", p->q.nseg,
              p->q.seg_len, p->k.nseg, p->k.seg_len, p->v.nseg, p->v.seg_len);
    return XDIT_E_SHAPE;
  }
  if ((p->k2.ptr == nullptr) != (p->v2.ptr == nullptr)) {
    set_error("xdit_attn_fwd: k2 and v2 must be given together");
    return XDIT_E_NULL;
  }
  if (p->k2.ptr && (p->k2.nseg != 1 || p->v2.nseg != 1 || p->k2.seg_len < 1 ||
                    p->v2.seg_len != p->k2.seg_len)) {
    set_error("xdit_attn_fwd: joint K/V must be one segment of equal length");
    return XDIT_E_SHAPE;
  }
  if ((p->acc_in || p->acc_out) && (!p->o_acc || !p->lse_acc)) {
    set_error("xdit_attn_fwd: acc_in/acc_out need o_acc and lse_acc");
    return XDIT_E_NULL;
  }
  if (!p->acc_out && !p->out && !p->out_segments) { set_error("xdit_attn_fwd: NULL out"); return XDIT_E_NULL; }
  if (p->out_segments) {
    if (p->q.nseg > XDIT_MAX_OUT_SEGMENTS) {
      set_error("xdit_attn_fwd: out_segments with %d segments (at most %d)", p->q.nseg, XDIT_MAX_OUT_SEGMENTS);
      return XDIT_E_SHAPE;
    }
    for (int g = 0; g < p->q.nseg; ++g)
      if (!p->out_segments[g]) { set_error("xdit_attn_fwd: out_segments[%d] is NULL", g); return XDIT_E_NULL; }
  }
  if (p->causal && (p->q.nseg != 1 || p->k.nseg != 1)) {
    set_error("xdit_attn_fwd: causal needs single-segment q and k");
    return XDIT_E_SHAPE;
  }
  const int64_t sq = (int64_t)p->q.nseg * p->q.seg_len;
  const int64_t sk = (int64_t)p->k.nseg * p->k.seg_len + (p->k2.ptr ? p->k2.seg_len : 0);
  if (sq >= (1ll << 30) || sk >= (1ll << 30)) { set_error("xdit_attn_fwd: sequence too long"); return XDIT_E_SHAPE; }
  return XDIT_OK;
}

}  // namespace xdit
extern "C" {

int xdit_attn_which(const struct xdit_attn_params* p) {
  int rc = attn_check(p);
  if (rc) return rc;
  if (p->force_generic) return 0;
  return attn_sm100_applicable(*p);
}

int64_t xdit_attn_split_scratch_bytes(const struct xdit_attn_params* p) {
  if (!p || attn_check(p) != XDIT_OK) return 0;
  if (p->force_generic || p->acc_in || p->acc_out || attn_sm100_applicable(*p) != 1) return 0;
  return attn_sm100_split_scratch_bytes(*p);
}

int xdit_attn_fwd(const struct xdit_attn_params* p, void* stream) {
  int rc = attn_check(p);
  if (rc) return rc;
  if (p->status_host) {
    const int32_t code = *reinterpret_cast<const volatile int32_t*>(p->status_host);
    if (code != 0) {
      set_error("xdit_attn_fwd: an earlier launch gave up a bounded wait (code %d); nothing is launched until "
                "the status words are cleared", code);
      return XDIT_E_KERNEL_TIMEOUT;
    }
  }
  rc = check_device(nullptr);
  if (rc) return rc;
  if (!p->force_generic && attn_sm100_applicable(*p) == 1)
    return launch_attn_sm100(*p, (cudaStream_t)stream);
  if (p->out_segments) {
    set_error("xdit_attn_fwd: out_segments is served by the tcgen05 kernel only (bf16/fp16, head_dim %% 8 == 0)");
    return XDIT_E_DTYPE;
  }
  return launch_attn_generic(*p, (cudaStream_t)stream);
}

}  // extern "C"
