// Attention prologue of the DiT processors fused with the Ulysses pack: RMSNorm of the q and k
// projections (over all heads, as Wan does, or per head, as Flux does), rotary embedding of
// interleaved pairs, head split, and the write into the all-to-all send layout -- one pass over
// q, k and v instead of a norm, a rotary, a transpose and a pack kernel per tensor.
//
// HBM-bound: per token row the kernel reads 3 x H*D elements (+ D cos and D sin values, + the two
// weight vectors, which stay in L2) and writes 3 x H*D elements.  One CTA per token row, 16-byte
// vectors of 8 elements, a row's vectors stay in registers between the sum of squares and the
// normalised write.
#include "common.cuh"

namespace xdit {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 4;  // vectors of 8 elements per thread: H*D <= 8192
constexpr int kRowRun = 8;

template <typename T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(uint32_t u, float& lo, float& hi) {
    lo = __uint_as_float(u << 16);
    hi = __uint_as_float(u & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ void unpack(uint32_t u, float& lo, float& hi) {
    const __half2 h = *reinterpret_cast<const __half2*>(&u);
    const float2 f = __half22float2(h);
    lo = f.x;
    hi = f.y;
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

struct PrologueArgs {
  const char* src[3];       // q, k, v projections
  int64_t src_stride_b[3];  // bytes
  int64_t src_stride_row[3];
  const char* weight[2];    // RMSNorm weights of q and k ([H*D] or [D]), may be null
  const float* cos;
  const float* sin;
  int64_t cs_stride_row;    // elements
  char* dst[3];
  int64_t dst_peer_stride[3];  // bytes
  int64_t dst_stride_h[3];     // bytes between heads of a peer block
  int64_t dst_stride_b[3];     // bytes between batches
  int32_t B, H, D, s, U;
  int32_t per_head;
  float eps;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 3) qk_norm_rope_pack_kernel(const __grid_constant__ PrologueArgs a) {
  __shared__ float red[kThreads / 32];
  const int HD = a.H * a.D;
  const int nvec = HD / 8;
  const int vpd = a.D / 8;  // vectors per head
  const int Hl = a.H / a.U;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)a.B * a.s;
  const bool same_col = kThreads % vpd == 0;
  // Which head, column and destination slot a thread's k-th vector belongs to does not depend on the
  // token row: the integer divisions are done once here, not per vector and row.
  int d0_k[kMaxVec], peer_k[kMaxVec], hip_k[kMaxVec];  // column, peer and head-in-peer of a thread's k-th vector
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int idx = threadIdx.x + k * kThreads;
    const int head = idx / vpd;
    d0_k[k] = (idx - head * vpd) * 8;
    peer_k[k] = head / Hl;
    hip_k[k] = head - peer_k[k] * Hl;
  }
  // a CTA takes runs of kRowRun consecutive token rows: its 256-byte writes to one head then fall
  // next to each other and leave L2 as longer runs
  const int64_t nruns = (rows + kRowRun - 1) / kRowRun;
  for (int64_t run = blockIdx.x; run < nruns; run += gridDim.x)
  for (int64_t r = run * kRowRun; r < min(rows, (run + 1) * kRowRun); ++r) {
    const int b = (int)(r / a.s), row = (int)(r - (int64_t)b * a.s);
    const int64_t row_bytes = (int64_t)row * a.D * 2;  // bytes from a (batch, head)'s first row to this one
    // With D/8 dividing the block size every vector of a thread starts at the same column of its head,
    // so the thread needs one set of eight cos and sin values per token row for q and k alike.
    float cs_row[8], sn_row[8];
    if (same_col && a.cos != nullptr) {
      const int d0 = (threadIdx.x % vpd) * 8;
      const float* cr = a.cos + (int64_t)row * a.cs_stride_row + d0;
      const float* sr = a.sin + (int64_t)row * a.cs_stride_row + d0;
      const float4 c0 = __ldg(reinterpret_cast<const float4*>(cr)), c1 = __ldg(reinterpret_cast<const float4*>(cr) + 1);
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(sr)), s1 = __ldg(reinterpret_cast<const float4*>(sr) + 1);
      cs_row[0] = c0.x; cs_row[1] = c0.y; cs_row[2] = c0.z; cs_row[3] = c0.w;
      cs_row[4] = c1.x; cs_row[5] = c1.y; cs_row[6] = c1.z; cs_row[7] = c1.w;
      sn_row[0] = s0.x; sn_row[1] = s0.y; sn_row[2] = s0.z; sn_row[3] = s0.w;
      sn_row[4] = s1.x; sn_row[5] = s1.y; sn_row[6] = s1.z; sn_row[7] = s1.w;
    }
#pragma unroll 1
    for (int tns = 0; tns < 3; ++tns) {
      const char* src = a.src[tns] + b * a.src_stride_b[tns] + row * a.src_stride_row[tns];
      uint4 v[kMaxVec];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < kMaxVec; ++k) {
        const int idx = threadIdx.x + k * kThreads;
        if (idx < nvec) {
          v[k] = __ldg(reinterpret_cast<const uint4*>(src) + idx);
          const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float lo, hi;
            Cvt<T>::unpack(w[e], lo, hi);
            ss = fmaf(lo, lo, ss);
            ss = fmaf(hi, hi, ss);
          }
        }
      }
      const bool norm = tns < 2 && a.weight[tns] != nullptr;
      const bool rope = tns < 2 && a.cos != nullptr;
      float rstd[kMaxVec];
      if (norm) {
        if (a.per_head) {
          // a head's D/8 vectors sit in D/8 consecutive lanes (a power of two): butterfly over them,
          // separately for each of this thread's vectors
#pragma unroll
          for (int k = 0; k < kMaxVec; ++k) rstd[k] = 0.f;
          // redo the per-vector sums (ss mixed all of this thread's vectors)
#pragma unroll
          for (int k = 0; k < kMaxVec; ++k) {
            const int idx = threadIdx.x + k * kThreads;
            float sk = 0.f;
            if (idx < nvec) {
              const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float lo, hi;
                Cvt<T>::unpack(w[e], lo, hi);
                sk = fmaf(lo, lo, sk);
                sk = fmaf(hi, hi, sk);
              }
            }
            for (int m = vpd >> 1; m > 0; m >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, m);
            rstd[k] = rsqrtf(sk / (float)a.D + a.eps);
          }
        } else {
#pragma unroll
          for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
          __syncthreads();  // red[] of the previous tensor has been read by everyone
          if (lane == 0) red[warp] = ss;
          __syncthreads();
          float tot = 0.f;
#pragma unroll
          for (int w = 0; w < kThreads / 32; ++w) tot += red[w];
          const float rs = rsqrtf(tot / (float)HD + a.eps);
#pragma unroll
          for (int k = 0; k < kMaxVec; ++k) rstd[k] = rs;
        }
      }
#pragma unroll
      for (int k = 0; k < kMaxVec; ++k) {
        const int idx = threadIdx.x + k * kThreads;
        if (idx >= nvec) continue;
        const int d0 = d0_k[k];
        uint4 o = v[k];
        if (norm || rope) {
          float x[8];
          const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) Cvt<T>::unpack(w[e], x[2 * e], x[2 * e + 1]);
          if (norm) {
            const int wi = a.per_head ? d0 : idx * 8;
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.weight[tns] + (int64_t)wi * 2));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float g0, g1;
              Cvt<T>::unpack(ww[e], g0, g1);
              // one rounding to the storage type after scale and weight, as a fused RMSNorm does
              uint32_t pk = Cvt<T>::pack(x[2 * e] * rstd[k] * g0, x[2 * e + 1] * rstd[k] * g1);
              Cvt<T>::unpack(pk, x[2 * e], x[2 * e + 1]);
            }
          }
          if (rope) {
            float cs[8], sn[8];
            if (same_col) {
#pragma unroll
              for (int e = 0; e < 8; ++e) { cs[e] = cs_row[e]; sn[e] = sn_row[e]; }
            } else {
              const float* cr = a.cos + (int64_t)row * a.cs_stride_row + d0;
              const float* sr = a.sin + (int64_t)row * a.cs_stride_row + d0;
              const float4 c0 = __ldg(reinterpret_cast<const float4*>(cr)), c1 = __ldg(reinterpret_cast<const float4*>(cr) + 1);
              const float4 s0 = __ldg(reinterpret_cast<const float4*>(sr)), s1 = __ldg(reinterpret_cast<const float4*>(sr) + 1);
              cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
              sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // pair (x1, x2) = elements (2e, 2e+1); cosine taken at the even, sine at the odd column
              const float x1 = x[2 * e], x2 = x[2 * e + 1];
              x[2 * e] = x1 * cs[2 * e] - x2 * sn[2 * e + 1];
              x[2 * e + 1] = x1 * sn[2 * e + 1] + x2 * cs[2 * e];
            }
          }
          o.x = Cvt<T>::pack(x[0], x[1]);
          o.y = Cvt<T>::pack(x[2], x[3]);
          o.z = Cvt<T>::pack(x[4], x[5]);
          o.w = Cvt<T>::pack(x[6], x[7]);
        }
        char* d = a.dst[tns] + peer_k[k] * a.dst_peer_stride[tns] + hip_k[k] * a.dst_stride_h[tns] +
                  b * a.dst_stride_b[tns] + row_bytes + d0_k[k] * 2;
        *reinterpret_cast<uint4*>(d) = o;
      }
    }
  }
}

}  // namespace

int launch_prologue(const xdit_prologue_params& p, cudaStream_t stream) {
  PrologueArgs a;
  const void* src[3] = {p.q, p.k, p.v};
  const int64_t sb[3] = {p.q_stride_b, p.k_stride_b, p.v_stride_b};
  const int64_t sr[3] = {p.q_stride_row, p.k_stride_row, p.v_stride_row};
  void* dst[3] = {p.dst_q, p.dst_k, p.dst_v};
  const int64_t dp[3] = {p.dst_q_peer_stride, p.dst_k_peer_stride, p.dst_v_peer_stride};
  for (int i = 0; i < 3; ++i) {
    a.src[i] = (const char*)src[i];
    a.src_stride_b[i] = sb[i] * 2;
    a.src_stride_row[i] = sr[i] * 2;
    a.dst[i] = (char*)dst[i];
    a.dst_peer_stride[i] = dp[i] * 2;
    a.dst_stride_h[i] = (p.dst_stride_h[i] ? p.dst_stride_h[i] : (int64_t)p.B * p.s * p.D) * 2;
    a.dst_stride_b[i] = (p.dst_stride_b[i] ? p.dst_stride_b[i] : (int64_t)p.s * p.D) * 2;
  }
  a.weight[0] = (const char*)p.norm_q_weight;
  a.weight[1] = (const char*)p.norm_k_weight;
  a.cos = p.cos;
  a.sin = p.sin;
  a.cs_stride_row = p.cos_sin_stride_row;
  a.B = p.B; a.H = p.H; a.D = p.D; a.s = p.s; a.U = p.U;
  a.per_head = p.norm_per_head;
  a.eps = p.eps;
  int sms = 0;
  int rc = check_device(&sms);
  if (rc) return rc;
  const int64_t rows = (int64_t)p.B * p.s;
  const int64_t nruns = (rows + kRowRun - 1) / kRowRun;
  const int grid = (int)(nruns < (int64_t)sms * 8 ? nruns : (int64_t)sms * 8);
  if (p.dtype == XDIT_BF16) qk_norm_rope_pack_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(a);
  else qk_norm_rope_pack_kernel<__half><<<grid, kThreads, 0, stream>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "qk_norm_rope_pack_kernel launch");
  return XDIT_OK;
}

}  // namespace xdit
