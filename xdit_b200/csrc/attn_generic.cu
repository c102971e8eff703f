// CUDA-core flash-attention forward for the shapes the tcgen05 kernel does not take: fp32
// tensors, head_dim not a multiple of 8 or above 128, odd strides, causal masking.  Same
// contract as the tensor-core kernel (segmented q/k/v, joint K/V as a second source, merge
// epilogue); arithmetic is fp32 throughout.
//
// One CTA = 32 query rows x all keys, 128 threads.  Keys are visited in tiles of 64 rows staged
// in shared memory.  S = Q K^T is computed 4x4 per thread, the online-softmax row state lives in
// the registers of the 4 threads that also own the row's output accumulators.
#include "common.cuh"

namespace xdit {
namespace {

constexpr int BM = 32;
constexpr int BN = 64;
constexpr int NT = 128;
constexpr int MAXD4 = 64;  // D <= 256

template <typename T> __device__ inline float ld_f(const T* p);
template <> __device__ inline float ld_f<float>(const float* p) { return *p; }
template <> __device__ inline float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ inline float ld_f<__half>(const __half* p) { return __half2float(*p); }
template <typename T> __device__ inline void st_f(T* p, float x);
template <> __device__ inline void st_f<float>(float* p, float x) { *p = x; }
template <> __device__ inline void st_f<__nv_bfloat16>(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
template <> __device__ inline void st_f<__half>(__half* p, float x) { *p = __float2half_rn(x); }

struct GenericArgs {
  xdit_attn_params p;
  float scale;
  int sq_total;
};

template <typename T>
__global__ void __launch_bounds__(NT) attn_generic_kernel(const __grid_constant__ GenericArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const xdit_attn_params& p = a.p;
  const int D = p.D;
  const int Dp = D + (sizeof(T) == 2 ? 2 : 1);  // padded row, odd number of 32-bit words
  T* Qs = reinterpret_cast<T*>(smem_raw);
  T* Ks = Qs + BM * Dp;
  T* Vs = Ks + BN * Dp;
  float* Ss = reinterpret_cast<float*>(Vs + BN * Dp);  // [BM][BN+1]
  constexpr int SP = BN + 1;

  const int tid = threadIdx.x;
  const int b = blockIdx.z, h = blockIdx.y;
  const int row0 = blockIdx.x * BM;  // first virtual query row of this CTA
  const int nrows = min(BM, a.sq_total - row0);

  // ---- load Q tile ----
  const T* qbase = reinterpret_cast<const T*>(p.q.ptr) + b * p.q.stride_b + h * p.q.stride_h;
  for (int i = tid; i < BM * D; i += NT) {
    const int r = i / D, d = i - r * D;
    float v = 0.f;
    if (r < nrows) {
      const int vr = row0 + r;
      const int sg = vr / p.q.seg_len, t = vr - sg * p.q.seg_len;
      v = ld_f<T>(qbase + sg * p.q.stride_seg + t * p.q.stride_row + d);
    }
    st_f<T>(Qs + r * Dp + d, v);
  }

  // thread roles
  const int s_r4 = tid >> 4, s_tx = tid & 15;  // S: rows s_r4*4.., cols s_tx+16*j
  const int o_r = tid >> 2, o_c = tid & 3;     // O: row o_r, cols o_c+4*i
  const int nD4 = (D + 3) / 4;
  float o[MAXD4];
#pragma unroll
  for (int i = 0; i < MAXD4; ++i) o[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  const int q_idx_max = row0 + nrows - 1;  // causal: single segment, virtual row == position

  // ---- key/value sources: main segments, then the joint segment ----
  const int nsrc_seg = p.k.nseg + (p.k2.ptr ? 1 : 0);
  for (int ss = 0; ss < nsrc_seg; ++ss) {
    const bool joint = ss >= p.k.nseg;
    const xdit_seq& ks = joint ? p.k2 : p.k;
    const xdit_seq& vs = joint ? p.v2 : p.v;
    const int sg = joint ? 0 : ss;
    const int len = ks.seg_len;
    const T* kb = reinterpret_cast<const T*>(ks.ptr) + b * ks.stride_b + h * ks.stride_h + sg * ks.stride_seg;
    const T* vb = reinterpret_cast<const T*>(vs.ptr) + b * vs.stride_b + h * vs.stride_h + sg * vs.stride_seg;
    for (int k0 = 0; k0 < len; k0 += BN) {
      if (p.causal && k0 > q_idx_max) break;
      const int nk = min(BN, len - k0);
      __syncthreads();  // previous tile fully consumed (also orders the Q stores the first time)
      for (int i = tid; i < BN * D; i += NT) {
        const int r = i / D, d = i - r * D;
        float kv = 0.f, vv = 0.f;
        if (r < nk) {
          kv = ld_f<T>(kb + (int64_t)(k0 + r) * ks.stride_row + d);
          vv = ld_f<T>(vb + (int64_t)(k0 + r) * vs.stride_row + d);
        }
        st_f<T>(Ks + r * Dp + d, kv);
        st_f<T>(Vs + r * Dp + d, vv);
      }
      __syncthreads();
      // ---- S = scale * Q K^T, masked ----
      {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        for (int d = 0; d < D; ++d) {
          float qv[4], kv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) qv[i] = ld_f<T>(Qs + (s_r4 * 4 + i) * Dp + d);
#pragma unroll
          for (int j = 0; j < 4; ++j) kv[j] = ld_f<T>(Ks + (s_tx + 16 * j) * Dp + d);
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int r = s_r4 * 4 + i, c = s_tx + 16 * j;
            float s = acc[i][j] * a.scale;
            if (c >= nk) s = -INFINITY;
            if (p.causal && (k0 + c) > (row0 + r)) s = -INFINITY;
            Ss[r * SP + c] = s;
          }
      }
      __syncthreads();
      // ---- online softmax for row o_r (4 threads per row, 16 columns each) ----
      {
        float mt = -INFINITY;
#pragma unroll
        for (int j = 0; j < 16; ++j) mt = fmaxf(mt, Ss[o_r * SP + o_c + 4 * j]);
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
        const float m_new = fmaxf(m_run, mt);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_safe);
        float lt = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float pv = __expf(Ss[o_r * SP + o_c + 4 * j] - m_safe);
          Ss[o_r * SP + o_c + 4 * j] = pv;
          lt += pv;
        }
        lt += __shfl_xor_sync(0xffffffffu, lt, 1);
        lt += __shfl_xor_sync(0xffffffffu, lt, 2);
        l_run = l_run * alpha + lt;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < MAXD4; ++i)
          if (i < nD4) o[i] *= alpha;
      }
      __syncwarp();  // the 4 threads of a row sit in one warp and are the only readers of that row
      // ---- O += P V ----
      for (int k = 0; k < nk; ++k) {
        const float pv = Ss[o_r * SP + k];
#pragma unroll
        for (int i = 0; i < MAXD4; ++i) {
          if (i < nD4) {
            const int c = o_c + 4 * i;
            if (c < D) o[i] = fmaf(pv, ld_f<T>(Vs + k * Dp + c), o[i]);
          }
        }
      }
    }
  }

  // ---- epilogue: normalise, merge with the running accumulators, store ----
  if (o_r < nrows) {
    const int vr = row0 + o_r;
    const int64_t flat = ((int64_t)b * p.H + h) * a.sq_total + vr;
    const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
    float lse = (l_run > 0.f) ? m_run + __logf(l_run) : -INFINITY;
    float w = 0.f;
    bool merge = p.acc_in != 0;
    float la = 0.f;
    if (merge) {
      la = p.lse_acc[flat];
      if (la == -INFINITY && lse == -INFINITY) { w = 0.f; }
      else {
        const float x = lse - la;
        w = 1.f / (1.f + __expf(-x));
        const float y = la - lse;  // lse_new = la - logsigmoid(la - lse)
        lse = la - (fminf(y, 0.f) - log1pf(__expf(-fabsf(y))));
      }
    }
    const int sg = vr / p.q.seg_len, t = vr - sg * p.q.seg_len;
    T* orow = p.out ? reinterpret_cast<T*>(p.out) + b * p.out_stride_b + h * p.out_stride_h +
                          sg * p.out_stride_seg + t * p.out_stride_row
                    : nullptr;
    float* arow = p.o_acc ? p.o_acc + flat * D : nullptr;
#pragma unroll
    for (int i = 0; i < MAXD4; ++i) {
      if (i < nD4) {
        const int c = o_c + 4 * i;
        if (c < D) {
          float val = o[i] * inv_l;
          if (merge) { const float oa = arow[c]; val = oa - w * (oa - val); }
          if (p.acc_out) arow[c] = val;
          else st_f<T>(orow + c, val);
        }
      }
    }
    if (o_c == 0) {
      if (p.acc_out) p.lse_acc[flat] = lse;
      else if (p.lse) p.lse[flat] = lse;
    }
  }
}

template <typename T>
int launch_t(const xdit_attn_params& p, cudaStream_t stream) {
  GenericArgs a;
  a.p = p;
  a.scale = p.softmax_scale > 0.f ? p.softmax_scale : 1.0f / sqrtf((float)p.D);
  a.sq_total = p.q.nseg * p.q.seg_len;
  const int Dp = p.D + (sizeof(T) == 2 ? 2 : 1);
  const size_t smem = (size_t)(BM + 2 * BN) * Dp * sizeof(T) + (size_t)BM * (BN + 1) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(attn_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "attn_generic smem attribute");
  dim3 grid((a.sq_total + BM - 1) / BM, p.H, p.B);
  attn_generic_kernel<T><<<grid, NT, smem, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "attn_generic_kernel launch");
  return XDIT_OK;
}

}  // namespace

int launch_attn_generic(const xdit_attn_params& p, cudaStream_t stream) {
  switch (p.dtype) {
    case XDIT_BF16: return launch_t<__nv_bfloat16>(p, stream);
    case XDIT_F16: return launch_t<__half>(p, stream);
    case XDIT_F32: return launch_t<float>(p, stream);
    default: set_error("attn generic: bad dtype"); return XDIT_E_DTYPE;
  }
}

}  // namespace xdit
