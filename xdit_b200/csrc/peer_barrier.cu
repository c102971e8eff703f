// Barrier between the ranks of a node whose buffers are mapped into each other (xdit_peer_open): every
// rank stores its epoch number into every peer's flag array with plain stores over NVLink, then waits
// until all peers' stores for this epoch have arrived in its own array.  One warp, a few microseconds --
// an order of magnitude below a collective launched for the same purpose -- which is what the Ulysses
// exchange by direct stores needs twice per attention call.
//
// The wait is bounded in time: when it runs out the kernel records a status code (device word and the
// host-visible word that the attention entry point checks) and returns, and while a failure is pending
// later barriers do not wait at all.  The epoch lives in device memory and is advanced by the kernel
// itself, so a captured launch replays correctly.
#include "common.cuh"

namespace xdit {
namespace {

struct BarrierArgs {
  uint32_t* peer_flags[XDIT_MAX_OUT_SEGMENTS];  // rank r's flag array (U words), mapped here
  uint32_t* local_flags;                        // this rank's own array: word r is written by rank r
  uint32_t* epoch;                              // this rank's barrier count (device memory)
  int32_t U, rank;
  uint32_t wait_limit_ns;
  int32_t* status;
  int32_t* status_host;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t timer_lo() {
  uint32_t t;
  asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(t));
  return t;
}

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ BarrierArgs a) {
  const int tid = threadIdx.x;
  uint32_t e = 0;
  if (tid == 0) {
    e = *a.epoch + 1;
    *a.epoch = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  const bool pending = a.status != nullptr && *reinterpret_cast<volatile int32_t*>(a.status) != 0;
  int code = 0;
  if (tid < a.U) {
    // everything this rank stored into its peers before this launch (earlier kernels on the stream) is
    // ordered before the flag by the release
    st_release_sys(a.peer_flags[tid] + a.rank, e);
    if (!pending) {
      const uint32_t t0 = timer_lo();
      for (uint32_t it = 0;; ++it) {
        if ((int32_t)(ld_acquire_sys(a.local_flags + tid) - e) >= 0) break;
        if ((it & 63) == 63 && timer_lo() - t0 > a.wait_limit_ns) {
          code = 400 + tid;  // peer `tid` did not arrive in time
          break;
        }
      }
    }
  }
  code = __reduce_max_sync(0xffffffffu, code);
  if (tid == 0 && code > 0) {
    if (a.status) atomicCAS(a.status, 0, code);
    if (a.status_host) {
      *reinterpret_cast<volatile int32_t*>(a.status_host) = code;
      __threadfence_system();
    }
  }
}

}  // namespace
}  // namespace xdit

extern "C" XDIT_API int xdit_peer_barrier(void* const* peer_flags, void* local_flags, void* epoch, int32_t U,
                                          int32_t rank, uint32_t wait_limit_ns, int32_t* status,
                                          int32_t* status_host, void* stream) {
  using namespace xdit;
  if (!peer_flags || !local_flags || !epoch) { set_error("xdit_peer_barrier: NULL pointer"); return XDIT_E_NULL; }
  if (U < 1 || U > XDIT_MAX_OUT_SEGMENTS || rank < 0 || rank >= U) {
    set_error("xdit_peer_barrier: U=%d rank=%d (1..%d ranks)", U, rank, XDIT_MAX_OUT_SEGMENTS);
    return XDIT_E_SHAPE;
  }
  BarrierArgs a;
  for (int r = 0; r < XDIT_MAX_OUT_SEGMENTS; ++r) a.peer_flags[r] = nullptr;
  for (int r = 0; r < U; ++r) {
    if (!peer_flags[r] || (((uintptr_t)peer_flags[r]) & 3)) {
      set_error("xdit_peer_barrier: flag array of rank %d is NULL or misaligned", r);
      return XDIT_E_NULL;
    }
    a.peer_flags[r] = static_cast<uint32_t*>(peer_flags[r]);
  }
  a.local_flags = static_cast<uint32_t*>(local_flags);
  a.epoch = static_cast<uint32_t*>(epoch);
  a.U = U;
  a.rank = rank;
  a.wait_limit_ns = wait_limit_ns ? wait_limit_ns : 2000000000u;  // 2 s
  a.status = status;
  a.status_host = status_host;
  int rc = check_device(nullptr);
  if (rc) return rc;
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "peer_barrier_kernel launch");
  return XDIT_OK;
}
