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

template <typename T, int VEC>
__global__ void __launch_bounds__(256) merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc,
                                                   const T* __restrict__ out_b,
                                                   const float* __restrict__ lse_b,
                                                   T* __restrict__ out_final, int64_t rows, int D,
                                                   int first) {
  const int vpr = D / VEC;
  const int64_t total = rows * vpr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vpr;
    const int c = (int)(i - r * vpr) * VEC;
    const float lb = lse_b[r];
    float w = 0.f, lnew = lb;
    if (!first) {
      const float la = lse_acc[r];
      // both -inf (no keys seen on either side): keep the accumulator
      if (la == -INFINITY && lb == -INFINITY) { w = 0.f; lnew = la; }
      else { w = sigmoidf_(lb - la); lnew = la - logsigmoidf_(la - lb); }
    }
    float res[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      const float ob = to_f<T>(out_b[r * D + c + k]);
      if (first) res[k] = ob;
      else { const float oa = o_acc[r * D + c + k]; res[k] = oa - w * (oa - ob); }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) o_acc[r * D + c + k] = res[k];
    if (out_final) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) out_final[r * D + c + k] = from_f<T>(res[k]);
    }
    if (c == 0) lse_acc[r] = lnew;
  }
}

template <typename T>
int launch(float* o_acc, float* lse_acc, const void* out_b, const float* lse_b, void* out_final,
           int64_t rows, int D, int first, cudaStream_t stream, int sms) {
  const int64_t total = rows * (int64_t)(D % 4 == 0 ? D / 4 : D);
  int64_t blocks = (total + 255) / 256;
  if (blocks > (int64_t)sms * 16) blocks = (int64_t)sms * 16;
  if (blocks < 1) blocks = 1;
  if (D % 4 == 0)
    merge_kernel<T, 4><<<(int)blocks, 256, 0, stream>>>(o_acc, lse_acc, (const T*)out_b, lse_b,
                                                         (T*)out_final, rows, D, first);
  else
    merge_kernel<T, 1><<<(int)blocks, 256, 0, stream>>>(o_acc, lse_acc, (const T*)out_b, lse_b,
                                                         (T*)out_final, rows, D, first);
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
