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

// One group of LPR lanes (a power of two, at most a warp) owns a row: its lanes stride over the row's
// vectors, and the row's lse is rewritten only after every lane of the warp has read it
// (__syncwarp).  A row never spans warps, so no other thread reads lse_acc[r].
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
  for (int64_t g = warp_id; g < n_groups; g += n_warps) {
    const int64_t r = g * rows_per_warp + lane / lpr;
    const bool live = r < rows;
    float w = 0.f, lnew = 0.f;
    if (live) {
      const float lb = lse_b[r];
      lnew = lb;
      if (!first) {
        const float la = lse_acc[r];
        // both -inf (no keys seen on either side): keep the accumulator
        if (la == -INFINITY && lb == -INFINITY) { w = 0.f; lnew = la; }
        else { w = sigmoidf_(lb - la); lnew = la - logsigmoidf_(la - lb); }
      }
      for (int v = sub; v < vpr; v += lpr) {
        const int64_t off = r * D + (int64_t)v * VEC;
        float res[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const float ob = to_f<T>(out_b[off + k]);
          if (first) res[k] = ob;
          else { const float oa = o_acc[off + k]; res[k] = oa - w * (oa - ob); }
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) o_acc[off + k] = res[k];
        if (out_final) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) out_final[off + k] = from_f<T>(res[k]);
        }
      }
    }
    __syncwarp();
    if (live && sub == 0) lse_acc[r] = lnew;
  }
}

template <typename T>
int launch(float* o_acc, float* lse_acc, const void* out_b, const float* lse_b, void* out_final,
           int64_t rows, int D, int first, cudaStream_t stream, int sms) {
  const int vec = (D % 4 == 0) ? 4 : 1;
  const int vpr = D / vec;
  int lpr = 1;
  while (lpr < vpr && lpr < 32) lpr <<= 1;
  const int64_t groups = (rows + (32 / lpr) - 1) / (32 / lpr);  // one warp each
  int64_t blocks = (groups + 7) / 8;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
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
