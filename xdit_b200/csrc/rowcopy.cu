// Strided row copy: the one HBM-bound kernel behind the Ulysses pack/unpack entry points and the
// PipeFusion stale-KV patch update.  A "row" is head_dim contiguous elements; the four outer
// indices have independent byte strides on the source and on the destination side.
//
// Work decomposition: a unit is (job, i0, a block of i1, i2, a run of kRowsPerUnit consecutive i3
// rows).  The unit index is decomposed once per CTA iteration with scalar arithmetic; inside a
// unit the threads move 16-byte vectors with four independent loads in flight per thread.  When
// consecutive i1 (heads) are adjacent in memory on one side -- the [B,S,H,D] views the DiT
// processors pass -- a unit takes several of them, so that the scattered side still moves in runs
// of a few KB instead of single 256-byte rows.  The grid is a multiple of the SM count and
// grid-strides over units.
#include "common.cuh"

namespace xdit {
namespace {

constexpr int kRowsPerUnit = 64;
constexpr int kThreads = 256;

constexpr int kMaxBlock1 = 8;
#ifndef XDIT_ROWCOPY_UNROLL
#define XDIT_ROWCOPY_UNROLL 4
#endif
constexpr int kInFlight = XDIT_ROWCOPY_UNROLL;  // independent 16-byte loads per thread before the first store

struct RowCopyArgs {
  RowCopyJob job[kMaxRowCopyJobs];
  int64_t unit_end[kMaxRowCopyJobs];  // exclusive prefix end of each job's units
  int32_t blk1[kMaxRowCopyJobs];      // how many consecutive i1 a unit covers
  int32_t njobs;
  int32_t npeers;  // > 0: index i0 selects peer[i0] and job.dst is a byte offset from that base
  char* peer[kMaxRowCopyPeers];
};

template <int VEC>
struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<8> { using type = uint2; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<2> { using type = uint16_t; };

template <int VEC>
__global__ void __launch_bounds__(kThreads) row_copy_kernel(const __grid_constant__ RowCopyArgs args) {
  using V = typename VecT<VEC>::type;
  const int64_t total_units = args.unit_end[args.njobs - 1];
  for (int64_t unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
    int j = 0;
    while (unit >= args.unit_end[j]) ++j;
    const RowCopyJob& jb = args.job[j];
    int64_t u = unit - (j ? args.unit_end[j - 1] : 0);
    const int chunks = (jb.n[3] + kRowsPerUnit - 1) / kRowsPerUnit;
    const int hb = args.blk1[j];
    const int n1b = (jb.n[1] + hb - 1) / hb;
    const int c3 = (int)(u % chunks); u /= chunks;
    const int i2 = (int)(u % jb.n[2]); u /= jb.n[2];
    const int i1 = (int)(u % n1b) * hb; u /= n1b;
    const int i0 = (int)u;
    const int r0 = c3 * kRowsPerUnit;
    const int nrows = min(kRowsPerUnit, jb.n[3] - r0);
    const uint32_t nhb = min(hb, jb.n[1] - i1);
    const bool zero = jb.src == nullptr;  // fill job (padding rows): nothing is read
    const char* s = jb.src + i0 * jb.s_stride[0] + i1 * jb.s_stride[1] + i2 * jb.s_stride[2] +
                    (int64_t)r0 * jb.s_stride[3];
    char* d = (args.npeers ? args.peer[i0] + reinterpret_cast<intptr_t>(jb.dst) : jb.dst + i0 * jb.d_stride[0]) +
              i1 * jb.d_stride[1] + i2 * jb.d_stride[2] + (int64_t)r0 * jb.d_stride[3];
    const uint32_t vpr = jb.row_bytes / VEC;
    const uint32_t vpg = vpr * nhb;  // vectors per row group: nhb rows of adjacent i1
    const uint32_t nvec = nrows * vpg;
    const int64_t ss = jb.s_stride[3], ds = jb.d_stride[3];
    const int64_t ss1 = jb.s_stride[1], ds1 = jb.d_stride[1];
    auto locate = [&](uint32_t e, int64_t& so, int64_t& dof) {
      const uint32_t r = e / vpg, rem = e - r * vpg;
      const uint32_t h = rem / vpr, c = rem - h * vpr;
      so = r * ss + h * ss1 + (int64_t)c * VEC;
      dof = r * ds + h * ds1 + (int64_t)c * VEC;
    };
    uint32_t idx = threadIdx.x;
    for (; idx + (kInFlight - 1) * kThreads < nvec; idx += kInFlight * kThreads) {
      V val[kInFlight];
      int64_t so[kInFlight], dof[kInFlight];
#pragma unroll
      for (int k = 0; k < kInFlight; ++k) {
        locate(idx + k * kThreads, so[k], dof[k]);
        val[k] = zero ? V{} : __ldg(reinterpret_cast<const V*>(s + so[k]));
      }
#pragma unroll
      for (int k = 0; k < kInFlight; ++k) *reinterpret_cast<V*>(d + dof[k]) = val[k];
    }
    for (; idx < nvec; idx += kThreads) {
      int64_t so, dof;
      locate(idx, so, dof);
      *reinterpret_cast<V*>(d + dof) = zero ? V{} : __ldg(reinterpret_cast<const V*>(s + so));
    }
  }
  if (args.npeers) {  // destinations in peer GPUs' memory: one system-scope fence per CTA
    __syncthreads();
    if (threadIdx.x == 0) __threadfence_system();
  }
}

int pick_vec(const RowCopyJob* jobs, int njobs, uint64_t base_bits) {
  int vec = 16;
  for (int j = 0; j < njobs; ++j) {
    uint64_t bits = (uint64_t)(uintptr_t)jobs[j].src | (uint64_t)(uintptr_t)jobs[j].dst |
                    (uint64_t)jobs[j].row_bytes | base_bits;
    for (int k = 0; k < 4; ++k) {
      if (jobs[j].n[k] > 1) bits |= (uint64_t)jobs[j].s_stride[k] | (uint64_t)jobs[j].d_stride[k];
    }
    while (vec > 2 && (bits & (vec - 1))) vec >>= 1;
  }
  return vec;
}

}  // namespace

int launch_row_copy(const RowCopyJob* jobs, int njobs, cudaStream_t stream, void* const* peer_base, int npeers) {
  if (njobs <= 0 || njobs > kMaxRowCopyJobs) {
    set_error("row copy: %d jobs (1..%d supported)", njobs, kMaxRowCopyJobs);
    return XDIT_E_SHAPE;
  }
  RowCopyArgs args;
  int64_t total = 0;
  int live = 0;
  for (int j = 0; j < njobs; ++j) {
    const RowCopyJob& jb = jobs[j];
    // block consecutive i1 when they are adjacent in memory on either side
    int hb = 1;
    if (jb.n[1] > 1 && (jb.s_stride[1] == jb.row_bytes || jb.d_stride[1] == jb.row_bytes)) {
      hb = jb.n[1] < kMaxBlock1 ? jb.n[1] : kMaxBlock1;
      while (hb > 1 && (int64_t)hb * jb.row_bytes > 4096) hb >>= 1;  // keep runs around 2-4 KB
    }
    int64_t units = (int64_t)jb.n[0] * ((jb.n[1] + hb - 1) / hb) * jb.n[2];
    units *= (jb.n[3] + kRowsPerUnit - 1) / kRowsPerUnit;
    if (units <= 0 || jb.row_bytes <= 0) continue;  // empty job: nothing to move
    if (!jb.dst && !peer_base) {
      set_error("row copy: NULL pointer in job %d", j);
      return XDIT_E_NULL;
    }
    total += units;
    args.job[live] = jb;
    args.blk1[live] = hb;
    args.unit_end[live] = total;
    ++live;
  }
  if (live == 0) return XDIT_OK;
  args.njobs = live;
  args.npeers = 0;
  if (peer_base) {
    if (npeers < 1 || npeers > kMaxRowCopyPeers) {
      set_error("row copy: %d peer bases (1..%d supported)", npeers, kMaxRowCopyPeers);
      return XDIT_E_SHAPE;
    }
    for (int q = 0; q < npeers; ++q) {
      if (!peer_base[q]) { set_error("row copy: NULL base pointer for peer %d", q); return XDIT_E_NULL; }
      args.peer[q] = (char*)peer_base[q];
    }
    args.npeers = npeers;
  }
  int sms = 0;
  int rc = check_device(&sms);
  if (rc) return rc;
  uint64_t base_bits = 0;
  for (int q = 0; q < args.npeers; ++q) base_bits |= (uint64_t)(uintptr_t)args.peer[q];
  const int vec = pick_vec(args.job, live, base_bits);
  int grid = (int)((total < (int64_t)sms * 8) ? total : (int64_t)sms * 8);
  if (grid < 1) grid = 1;
  switch (vec) {
    case 16: row_copy_kernel<16><<<grid, kThreads, 0, stream>>>(args); break;
    case 8: row_copy_kernel<8><<<grid, kThreads, 0, stream>>>(args); break;
    case 4: row_copy_kernel<4><<<grid, kThreads, 0, stream>>>(args); break;
    default: row_copy_kernel<2><<<grid, kThreads, 0, stream>>>(args); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "row_copy_kernel launch");
  return XDIT_OK;
}

}  // namespace xdit
