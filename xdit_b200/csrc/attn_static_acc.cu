// xdit_attn_fwd_static_acc: the ring-step attention call for callers that cannot allocate
// device memory.  The fp32 running accumulators that xdit_attn_fwd takes from the caller
// (o_acc, lse_acc) live here in a fixed array inside the library image instead.
#include <mutex>

#include "common.cuh"

namespace xdit {
namespace {

// Scratch for the running (o_acc, lse_acc) pair of one ring sequence.  It is part of the loaded
// module: every GPU that loads the library holds these 32 MiB until the process exits.
static __device__ __align__(256) float g_static_acc[XDIT_STATIC_ACC_FLOATS];

// In host code `g_static_acc` is only a handle for the symbol, not a device address; the address
// a kernel can use comes from cudaGetSymbolAddress, per device, with that device current.
std::mutex g_mu;
float* g_addr[64] = {};

int static_acc_address(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) { set_error("xdit_attn_fwd_static_acc: device index %d out of range", dev); return XDIT_E_SHAPE; }
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_acc);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_static_acc)");
    g_addr[dev] = static_cast<float*>(p);
  }
  *out = g_addr[dev];
  return XDIT_OK;
}

}  // namespace
}  // namespace xdit

extern "C" XDIT_API int xdit_attn_fwd_static_acc(const struct xdit_attn_params* p, void* stream) {
  using namespace xdit;
  if (!p) { set_error("xdit_attn_fwd_static_acc: NULL params"); return XDIT_E_NULL; }
  if (p->o_acc || p->lse_acc) {
    set_error("xdit_attn_fwd_static_acc: o_acc/lse_acc must be NULL (the library's own array is used)");
    return XDIT_E_SHAPE;
  }
  if (!p->acc_in && !p->acc_out) {
    set_error("xdit_attn_fwd_static_acc: neither acc_in nor acc_out is set; call xdit_attn_fwd for a single step");
    return XDIT_E_SHAPE;
  }
  {
    // the shared argument check bounds B, H, D and the sequence length before any size is computed;
    // it wants accumulator pointers for acc_in/acc_out, so it sees a copy that has placeholders
    xdit_attn_params chk = *p;
    chk.o_acc = reinterpret_cast<float*>(uintptr_t(256));
    chk.lse_acc = reinterpret_cast<float*>(uintptr_t(256));
    const int rc = attn_check(&chk);
    if (rc) return rc;
  }
  const int64_t rows = (int64_t)p->B * p->H * p->q.nseg * p->q.seg_len;
  // layout inside the array: [rows][D] output accumulator, padded to 64 floats, then [rows] lse
  const int64_t o_floats = ((rows * p->D + 63) / 64) * 64;
  const int64_t need = o_floats + rows;
  if (need > (int64_t)XDIT_STATIC_ACC_FLOATS) {
    set_error("xdit_attn_fwd_static_acc: B*H*Sq*(D+1) = %lld floats exceeds the built-in scratch of %lld floats; "
              "use xdit_attn_fwd with caller-provided accumulators",
              (long long)need, (long long)XDIT_STATIC_ACC_FLOATS);
    return XDIT_E_SHAPE;
  }
  float* base = nullptr;
  int rc = static_acc_address(&base);
  if (rc) return rc;
  xdit_attn_params q = *p;
  q.o_acc = base;
  q.lse_acc = base + o_floats;
  return xdit_attn_fwd(&q, stream);
}
