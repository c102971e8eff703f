// Shared host-side helpers of the xdit_b200 C-ABI library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/xdit_b200.h"

namespace xdit {

// Thread-local reason of the last failure, read by xdit_last_error_string().
void set_error(const char* fmt, ...);

inline int dtype_size(int dtype) {
  switch (dtype) {
    case XDIT_BF16: return 2;
    case XDIT_F16: return 2;
    case XDIT_F32: return 4;
    default: return 0;
  }
}

// Returns 0 when the current device is sm_100, else XDIT_E_UNSUPPORTED_DEVICE or a cudaError_t.
int check_device(int* sm_count);

inline int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

// ---- strided row copy (rowcopy.cu) -------------------------------------------------------
// dst[i0,i1,i2,i3,:] = src[i0,i1,i2,i3,:] with per-dimension byte strides on both sides and
// rows of row_bytes contiguous bytes.
struct RowCopyJob {
  const char* src;  // NULL: the destination rows are filled with zeros
  char* dst;
  int64_t s_stride[4];  // bytes
  int64_t d_stride[4];  // bytes
  int32_t n[4];
  int32_t row_bytes;
};
constexpr int kMaxRowCopyJobs = 36;
constexpr int kMaxRowCopyPeers = XDIT_MAX_PACK_PEERS;
// peer_base (npeers entries): index i0 of every job selects a base pointer, job.dst holds the byte
// offset from that base and d_stride[0] is ignored; the destinations may then be peer GPUs' memory
// and every thread ends with a system-scope fence.
int launch_row_copy(const RowCopyJob* jobs, int njobs, cudaStream_t stream, void* const* peer_base = nullptr,
                    int npeers = 0);

// ---- attention kernels ------------------------------------------------------------------------
// Argument check shared by the attention entry points (bounds B, H, D and the sequence lengths).
int attn_check(const struct xdit_attn_params* p);
int launch_attn_generic(const xdit_attn_params& p, cudaStream_t stream);
// Returns 1 when the tcgen05 kernel accepts p, 0 when it does not (reason in set_error).
int attn_sm100_applicable(const xdit_attn_params& p);
int launch_attn_sm100(const xdit_attn_params& p, cudaStream_t stream);
// Scratch bytes with which launch_attn_sm100 may split the keys of p over several CTAs (0: it would not).
int64_t attn_sm100_split_scratch_bytes(const xdit_attn_params& p);

// ---- attention prologue (prologue.cu) ------------------------------------------------------------
int launch_prologue(const xdit_prologue_params& p, cudaStream_t stream);

}  // namespace xdit
