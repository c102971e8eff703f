// Strided row copy: the one HBM-bound kernel behind the Ulysses pack/unpack entry points and the
// PipeFusion stale-KV patch update.  A "row" is head_dim contiguous elements; the four outer
// indices have independent byte strides on the source and on the destination side.
//
// Work decomposition: a unit is (job, i0, i1, i2, a run of kRowsPerUnit consecutive i3 rows).
// The unit index is decomposed once per CTA iteration with scalar arithmetic; inside a unit the
// threads move 16-byte vectors with four independent loads in flight per thread.  The grid is a
// multiple of the SM count and grid-strides over units.
#include "common.cuh"

namespace xdit {
namespace {

constexpr int kRowsPerUnit = 64;
constexpr int kThreads = 256;

struct RowCopyArgs {
  RowCopyJob job[kMaxRowCopyJobs];
  int64_t unit_end[kMaxRowCopyJobs];  // exclusive prefix end of each job's units
  int32_t njobs;
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
    const int c3 = (int)(u % chunks); u /= chunks;
    const int i2 = (int)(u % jb.n[2]); u /= jb.n[2];
    const int i1 = (int)(u % jb.n[1]); u /= jb.n[1];
    const int i0 = (int)u;
    const int r0 = c3 * kRowsPerUnit;
    const int nrows = min(kRowsPerUnit, jb.n[3] - r0);
    const char* s = jb.src + i0 * jb.s_stride[0] + i1 * jb.s_stride[1] + i2 * jb.s_stride[2] +
                    (int64_t)r0 * jb.s_stride[3];
    char* d = jb.dst + i0 * jb.d_stride[0] + i1 * jb.d_stride[1] + i2 * jb.d_stride[2] +
              (int64_t)r0 * jb.d_stride[3];
    const uint32_t vpr = jb.row_bytes / VEC;
    const uint32_t nvec = nrows * vpr;
    const int64_t ss = jb.s_stride[3], ds = jb.d_stride[3];
    uint32_t idx = threadIdx.x;
    for (; idx + 3 * kThreads < nvec; idx += 4 * kThreads) {
      V val[4];
      uint32_t r[4], c[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t e = idx + k * kThreads;
        r[k] = e / vpr;
        c[k] = e - r[k] * vpr;
        val[k] = __ldg(reinterpret_cast<const V*>(s + r[k] * ss + (int64_t)c[k] * VEC));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)
        *reinterpret_cast<V*>(d + r[k] * ds + (int64_t)c[k] * VEC) = val[k];
    }
    for (; idx < nvec; idx += kThreads) {
      const uint32_t r = idx / vpr, c = idx - r * vpr;
      *reinterpret_cast<V*>(d + r * ds + (int64_t)c * VEC) =
          __ldg(reinterpret_cast<const V*>(s + r * ss + (int64_t)c * VEC));
    }
  }
}

int pick_vec(const RowCopyJob* jobs, int njobs) {
  int vec = 16;
  for (int j = 0; j < njobs; ++j) {
    uint64_t bits = (uint64_t)(uintptr_t)jobs[j].src | (uint64_t)(uintptr_t)jobs[j].dst |
                    (uint64_t)jobs[j].row_bytes;
    for (int k = 0; k < 4; ++k) {
      if (jobs[j].n[k] > 1) bits |= (uint64_t)jobs[j].s_stride[k] | (uint64_t)jobs[j].d_stride[k];
    }
    while (vec > 2 && (bits & (vec - 1))) vec >>= 1;
  }
  return vec;
}

}  // namespace

int launch_row_copy(const RowCopyJob* jobs, int njobs, cudaStream_t stream) {
  if (njobs <= 0 || njobs > kMaxRowCopyJobs) {
    set_error("row copy: %d jobs (1..%d supported)", njobs, kMaxRowCopyJobs);
    return XDIT_E_SHAPE;
  }
  RowCopyArgs args;
  int64_t total = 0;
  int live = 0;
  for (int j = 0; j < njobs; ++j) {
    const RowCopyJob& jb = jobs[j];
    int64_t units = 1;
    for (int k = 0; k < 3; ++k) units *= jb.n[k];
    units *= (jb.n[3] + kRowsPerUnit - 1) / kRowsPerUnit;
    if (units <= 0 || jb.row_bytes <= 0) continue;  // empty job: nothing to move
    if (!jb.src || !jb.dst) {
      set_error("row copy: NULL pointer in job %d", j);
      return XDIT_E_NULL;
    }
    total += units;
    args.job[live] = jb;
    args.unit_end[live] = total;
    ++live;
  }
  if (live == 0) return XDIT_OK;
  args.njobs = live;
  int sms = 0;
  int rc = check_device(&sms);
  if (rc) return rc;
  const int vec = pick_vec(args.job, live);
  if ((args.job[0].row_bytes & 1) != 0) {
    set_error("row copy: odd row size");
    return XDIT_E_ALIGN;
  }
  int64_t want = (total + 0) ;
  int grid = (int)((want < (int64_t)sms * 8) ? want : (int64_t)sms * 8);
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
