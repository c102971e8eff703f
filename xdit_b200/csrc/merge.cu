// Stand-alone online-softmax merge of a partial attention result into fp32 accumulators
// (HBM-bound, elementwise).  The attention kernels fuse the same arithmetic into their epilogue;
// this entry point serves callers that hold partial (out, lse) pairs of their own.
#include "common.cuh"

namespace xdit {
namespace {

template <typename T> __device__ inline float to_f(T x);
template <> __device__ inline float to_f<float>(float x) { return x; }
template <> __device__ inline float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ inline float to_f<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ inline T from_f(float x);
template <> __device__ inline float from_f<float>(float x) { return x; }
template <> __device__ inline __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ inline __half from_f<__half>(float x) { return __float2half_rn(x); }

// sigmoid(x) and log(sigmoid(x)) evaluated without overflow on either side
__device__ inline float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ inline float logsigmoidf_(float x) {
  return fminf(x, 0.f) - log1pf(__expf(-fabsf(x)));
}

// Vector access helpers: VEC elements of the block's dtype / of fp32 in one load or store.
template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[VEC]) {
  if constexpr (VEC == 1) {
    out[0] = to_f<T>(p[0]);
  } else {
    using P = Pack<T, VEC>;
    const P x = *reinterpret_cast<const P*>(p);  // 8 bytes (16-bit types) or 16 bytes (fp32), aligned: D % 4 == 0
#pragma unroll
    for (int k = 0; k < VEC; ++k) out[k] = to_f<T>(x.v[k]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T* p, const float (&in)[VEC]) {
  if constexpr (VEC == 1) {
    p[0] = from_f<T>(in[0]);
  } else {
    Pack<T, VEC> x;
#pragma unroll
    for (int k = 0; k < VEC; ++k) x.v[k] = from_f<T>(in[k]);
    *reinterpret_cast<Pack<T, VEC>*>(p) = x;
  }
}

// One group of LPR lanes (a power of two, at most a warp) owns a row's vectors.  A row never spans warps,
// so no other warp touches lse_acc[r].  A warp takes kRowsInFlight row groups per iteration and issues all
// their loads before the arithmetic, which is what keeps enough bytes in flight for an HBM-bound kernel;
// the per-row exponentials and logarithms are done once per row, by one lane, not by every lane of the row.
constexpr int kRowsInFlight = 4;

template <typename T, int VEC>
__global__ void __launch_bounds__(256) merge_kernel(float* __restrict__ o_acc, float* lse_acc,
                                                   const T* __restrict__ out_b,
                                                   const float* __restrict__ lse_b,
                                                   T* __restrict__ out_final, int64_t rows, int D,
                                                   int first, int lpr) {
  const int vpr = D / VEC;
  const int lane = threadIdx.x & 31;
  const int sub = lane & (lpr - 1);        // lane inside its row group
  const int rows_per_warp = 32 / lpr;
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t n_groups = (rows + rows_per_warp - 1) / rows_per_warp;
  // every lane has at most one vector of its row (D <= 128 with VEC 4) and an iteration's rows fit the lanes
  const bool one_vec = vpr <= lpr && kRowsInFlight * rows_per_warp <= 32;
  for (int64_t g0 = warp_id * kRowsInFlight; g0 < n_groups; g0 += n_warps * kRowsInFlight) {
    if (one_vec) {
      // The rows of one iteration are consecutive: row (g0 * rows_per_warp + L) belongs to lane L for the
      // per-row arithmetic (lse, weight), one row per lane, and the weights are handed to the lanes that
      // hold the row's vectors by shuffles.  No lane reads another row's lse from memory.
      const int64_t row0 = g0 * rows_per_warp;
      const bool has_row = lane < kRowsInFlight * rows_per_warp && row0 + lane < rows;
      float la_l = 0.f, lb_l = 0.f;
      if (has_row) {
        lb_l = lse_b[row0 + lane];
        if (!first) la_l = lse_acc[row0 + lane];
      }
      int64_t r[kRowsInFlight];
      bool mine[kRowsInFlight];
      float ob[kRowsInFlight][VEC], oa[kRowsInFlight][VEC];
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u) {
        r[u] = row0 + u * rows_per_warp + lane / lpr;
        mine[u] = r[u] < rows && sub < vpr;
#pragma unroll
        for (int k = 0; k < VEC; ++k) ob[u][k] = oa[u][k] = 0.f;
        if (mine[u]) {
          const int64_t off = r[u] * D + (int64_t)sub * VEC;
          load_vec<T, VEC>(out_b + off, ob[u]);
          if (!first) load_vec<float, VEC>(o_acc + off, oa[u]);
        }
      }
      float w_l = 0.f, lnew_l = lb_l;
      if (!first && has_row) {
        // both -inf (no keys seen on either side): keep the accumulator
        if (la_l == -INFINITY && lb_l == -INFINITY) { w_l = 0.f; lnew_l = la_l; }
        else { w_l = sigmoidf_(lb_l - la_l); lnew_l = la_l - logsigmoidf_(la_l - lb_l); }
      }
      if (has_row) lse_acc[row0 + lane] = lnew_l;
#pragma unroll
      for (int u = 0; u < kRowsInFlight; ++u) {
        const float w = __shfl_sync(0xffffffffu, w_l, u * rows_per_warp + lane / lpr);
        if (mine[u]) {
          const int64_t off = r[u] * D + (int64_t)sub * VEC;
          float res[VEC];
#pragma unroll
          for (int k = 0; k < VEC; ++k) res[k] = first ? ob[u][k] : oa[u][k] - w * (oa[u][k] - ob[u][k]);
          store_vec<float, VEC>(o_acc + off, res);
          if (out_final) store_vec<T, VEC>(out_final + off, res);
        }
      }
    } else {
      // long rows (more vectors than lanes): one row group at a time, lanes stride over the row
      for (int u = 0; u < kRowsInFlight; ++u) {
        const int64_t g = g0 + u;
        if (g >= n_groups) break;
        const int64_t rr = g * rows_per_warp + lane / lpr;
        const bool lv = rr < rows;
        float w = 0.f, lnew = 0.f;
        if (lv) {
          const float lbv = lse_b[rr];
          lnew = lbv;
          if (!first) {
            const float lav = lse_acc[rr];
            if (lav == -INFINITY && lbv == -INFINITY) { w = 0.f; lnew = lav; }
            else { w = sigmoidf_(lbv - lav); lnew = lav - logsigmoidf_(lav - lbv); }
          }
          for (int v = sub; v < vpr; v += lpr) {
            const int64_t off = rr * D + (int64_t)v * VEC;
            float obv[VEC], oav[VEC], res[VEC];
            load_vec<T, VEC>(out_b + off, obv);
            if (!first) load_vec<float, VEC>(o_acc + off, oav);
#pragma unroll
            for (int k = 0; k < VEC; ++k) res[k] = first ? obv[k] : oav[k] - w * (oav[k] - obv[k]);
            store_vec<float, VEC>(o_acc + off, res);
            if (out_final) store_vec<T, VEC>(out_final + off, res);
          }
        }
        __syncwarp();
        if (lv && sub == 0) lse_acc[rr] = lnew;
      }
    }
  }
}

template <typename T>
int launch(float* o_acc, float* lse_acc, const void* out_b, const float* lse_b, void* out_final,
           int64_t rows, int D, int first, cudaStream_t stream, int sms) {
  // vectors of 4 need 16-byte aligned fp32 rows and 8-byte (or 16-byte) aligned rows of the block
  const bool aligned = D % 4 == 0 && (((uintptr_t)o_acc | (uintptr_t)out_b | (uintptr_t)out_final) & 15) == 0;
  const int vec = aligned ? 4 : 1;
  const int vpr = D / vec;
  int lpr = 1;
  while (lpr < vpr && lpr < 32) lpr <<= 1;
  const int64_t groups = (rows + (32 / lpr) - 1) / (32 / lpr);
  const int64_t warps = (groups + kRowsInFlight - 1) / kRowsInFlight;
  int64_t blocks = (warps + 7) / 8;
  if (blocks > (int64_t)sms * 32) blocks = (int64_t)sms * 32;
  if (blocks < 1) blocks = 1;
  if (vec == 4)
    merge_kernel<T, 4><<<(int)blocks, 256, 0, stream>>>(o_acc, lse_acc, (const T*)out_b, lse_b,
                                                         (T*)out_final, rows, D, first, lpr);
  else
    merge_kernel<T, 1><<<(int)blocks, 256, 0, stream>>>(o_acc, lse_acc, (const T*)out_b, lse_b,
                                                         (T*)out_final, rows, D, first, lpr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "merge_kernel launch");
  return XDIT_OK;
}

}  // namespace
}  // namespace xdit

extern "C" XDIT_API int xdit_merge_out_lse(float* o_acc, float* lse_acc, const void* out_b,
                                  const float* lse_b, void* out_final, int32_t dtype, int64_t rows,
                                  int32_t D, int32_t first, void* stream) {
  using namespace xdit;
  if (!o_acc || !lse_acc || !out_b || !lse_b) { set_error("xdit_merge_out_lse: NULL pointer"); return XDIT_E_NULL; }
  if (rows < 0 || D < 1) { set_error("xdit_merge_out_lse: bad shape"); return XDIT_E_SHAPE; }
  if (rows == 0) return XDIT_OK;
  int sms = 0;
  int rc = check_device(&sms);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case XDIT_BF16: return launch<__nv_bfloat16>(o_acc, lse_acc, out_b, lse_b, out_final, rows, D, first, st, sms);
    case XDIT_F16: return launch<__half>(o_acc, lse_acc, out_b, lse_b, out_final, rows, D, first, st, sms);
    case XDIT_F32: return launch<float>(o_acc, lse_acc, out_b, lse_b, out_final, rows, D, first, st, sms);
    default: set_error("xdit_merge_out_lse: bad dtype %d", dtype); return XDIT_E_DTYPE;
  }
}
