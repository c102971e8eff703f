// Attention prologue of the DiT processors fused with the Ulysses pack: RMSNorm of the q and k
// projections (over all heads, as Wan does, or per head, as Flux does), rotary embedding of
// interleaved pairs, head split, and the write into the all-to-all send layout -- one pass over
// q, k and v instead of a norm, a rotary, a transpose and a pack kernel per tensor.
//
// HBM-bound: per token row the kernel reads 3 x H*D elements (+ D cos and D sin values, + the two
// weight vectors, which stay in L2) and writes 3 x H*D elements.  One warp per token row: lane l owns
// the 16-byte vectors l, l+32, ... of the row and keeps them in registers between the sum of squares
// and the normalised write, so the row sum is a warp butterfly and no block-wide barrier sits between
// a row's loads and its stores; a warp has all of a row's loads in flight at once.  Where a vector
// goes (peer block, head, column) does not depend on the row and is read from a table in shared
// memory built once per CTA.  The arithmetic runs on packed pairs (f32x2).
#include "common.cuh"

namespace xdit {
namespace {

constexpr int kWarps = 4;     // token rows in flight per CTA
constexpr int kMaxVpl = 32;   // vectors of 8 elements per lane: H*D <= 8192

__device__ __forceinline__ uint64_t f2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_get(uint64_t x, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(x));
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

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

// VPL = vectors per lane (a row's H*D/8 vectors over 32 lanes, rounded up to an instantiated size).
#ifndef XDIT_PROLOGUE_CTAS20
#define XDIT_PROLOGUE_CTAS20 3
#endif
constexpr int min_ctas(int vpl) { return vpl <= 4 ? 5 : vpl <= 8 ? 4 : vpl <= 16 ? 3 : vpl <= 20 ? XDIT_PROLOGUE_CTAS20 : 2; }

template <typename T, int VPL, bool SAME_COL>
__global__ void __launch_bounds__(kWarps * 32, min_ctas(VPL))
qk_norm_rope_pack_kernel(const __grid_constant__ PrologueArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int HD = a.H * a.D;
  const int nvec = HD / 8;
  const int vpd = a.D / 8;  // vectors per head
  const int Hl = a.H / a.U;
  int32_t* dst16 = reinterpret_cast<int32_t*>(smem);              // [3][nvec]: destination of a vector, in 16-byte units
  uint16_t* col = reinterpret_cast<uint16_t*>(dst16 + 3 * nvec);  // [nvec]: its first column inside the head
  for (int idx = threadIdx.x; idx < nvec; idx += blockDim.x) {
    const int head = idx / vpd, d0 = (idx - head * vpd) * 8;
    const int peer = head / Hl, hip = head - peer * Hl;
    col[idx] = (uint16_t)d0;
#pragma unroll
    for (int t = 0; t < 3; ++t)
      dst16[t * nvec + idx] = (int32_t)((peer * a.dst_peer_stride[t] + hip * a.dst_stride_h[t] + d0 * 2) >> 4);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t rows = (int64_t)a.B * a.s;
  // With D/8 dividing 32 every vector of a lane starts at the same column of its head, so the lane
  // needs one set of cos and sin values per token row, for q and k alike.
  constexpr bool same_col = SAME_COL;  // (32 % vpd) == 0
  const int d0_lane = (lane % vpd) * 8;
  // A lane's vectors of the next (row, tensor) item are requested as soon as the registers of the
  // current item's vectors have been consumed, so a warp's loads stay in flight while it computes.
  const int64_t r_first = (int64_t)blockIdx.x * kWarps + warp, r_step = (int64_t)gridDim.x * kWarps;
  uint4 v[VPL];
  if (r_first < rows) {
    const int b0 = (int)(r_first / a.s), row0 = (int)(r_first - (int64_t)b0 * a.s);
    const char* src0 = a.src[0] + b0 * a.src_stride_b[0] + row0 * a.src_stride_row[0];
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int idx = lane + 32 * k;
      if (idx < nvec) v[k] = __ldg(reinterpret_cast<const uint4*>(src0) + idx);
    }
  }
  for (int64_t r = r_first; r < rows; r += r_step) {
    const int b = (int)(r / a.s), row = (int)(r - (int64_t)b * a.s);
    const int64_t row_bytes = (int64_t)row * a.D * 2;  // bytes from a (batch, head)'s first row to this one
    const int64_t rn = r + r_step;
    const int bn = (int)(rn / a.s), rown = (int)(rn - (int64_t)bn * a.s);
    // rotation factors as packed pairs: C = (cos[2e], cos[2e]), S = (-sin[2e+1], sin[2e+1])
    uint64_t c_row[4], s_row[4];
    auto load_cs = [&](int d0, uint64_t* c2, uint64_t* s2) {
      const float* cr = a.cos + (int64_t)row * a.cs_stride_row + d0;
      const float* sr = a.sin + (int64_t)row * a.cs_stride_row + d0;
      const float4 c0 = __ldg(reinterpret_cast<const float4*>(cr)), c1 = __ldg(reinterpret_cast<const float4*>(cr) + 1);
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(sr)), s1 = __ldg(reinterpret_cast<const float4*>(sr) + 1);
      c2[0] = f2(c0.x, c0.x); c2[1] = f2(c0.z, c0.z); c2[2] = f2(c1.x, c1.x); c2[3] = f2(c1.z, c1.z);
      s2[0] = f2(-s0.y, s0.y); s2[1] = f2(-s0.w, s0.w); s2[2] = f2(-s1.y, s1.y); s2[3] = f2(-s1.w, s1.w);
    };
    if (same_col && a.cos != nullptr) load_cs(d0_lane, c_row, s_row);
#pragma unroll 1
    for (int tns = 0; tns < 3; ++tns) {
      const bool norm = tns < 2 && a.weight[tns] != nullptr;
      const bool rope = tns < 2 && a.cos != nullptr;
      // source of the next item: the next tensor of this row, or q of this warp's next row
      const char* nsrc = tns < 2 ? a.src[tns + 1] + b * a.src_stride_b[tns + 1] + row * a.src_stride_row[tns + 1]
                                 : (rn < rows ? a.src[0] + bn * a.src_stride_b[0] + rown * a.src_stride_row[0] : nullptr);
      char* dbase = a.dst[tns] + b * a.dst_stride_b[tns] + row_bytes;
      const int32_t* dtab = dst16 + tns * nvec;
      if (!norm && !rope) {  // v: copied along
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
          const int idx = lane + 32 * k;
          if (idx < nvec) {
            *reinterpret_cast<uint4*>(dbase + ((int64_t)dtab[idx] << 4)) = v[k];
            if (nsrc) v[k] = __ldg(reinterpret_cast<const uint4*>(nsrc) + idx);
          }
        }
        continue;
      }
      float rs_all = 0.f;
      if (norm && !a.per_head) {
        uint64_t ss2 = f2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < VPL; ++k) {
          if (lane + 32 * k < nvec) {
            const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              Cvt<T>::unpack(w[e], lo, hi);
              const uint64_t x2 = f2(lo, hi);
              ss2 = f2_fma(x2, x2, ss2);
            }
          }
        }
        float s0, s1;
        f2_get(ss2, s0, s1);
        float ss = s0 + s1;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        rs_all = rsqrtf(ss / (float)HD + a.eps);
      }
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int idx = lane + 32 * k;
        const bool live = idx < nvec;  // the shuffles below are taken by the whole warp
        const uint32_t w[4] = {live ? v[k].x : 0u, live ? v[k].y : 0u, live ? v[k].z : 0u, live ? v[k].w : 0u};
        uint64_t x2[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi;
          Cvt<T>::unpack(w[e], lo, hi);
          x2[e] = f2(lo, hi);
        }
        if (live && nsrc) v[k] = __ldg(reinterpret_cast<const uint4*>(nsrc) + idx);
        const int d0 = same_col ? d0_lane : (live ? (int)col[idx] : 0);
        if (norm) {
          float rs = rs_all;
          if (a.per_head) {
            // a head's D/8 vectors sit in D/8 consecutive lanes (a power of two): butterfly over them
            uint64_t sk2 = f2_mul(x2[0], x2[0]);
#pragma unroll
            for (int e = 1; e < 4; ++e) sk2 = f2_fma(x2[e], x2[e], sk2);
            float s0, s1;
            f2_get(sk2, s0, s1);
            float sk = s0 + s1;
            for (int m = vpd >> 1; m > 0; m >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, m);
            rs = rsqrtf(sk / (float)a.D + a.eps);
          }
          if (live) {
            const int wi = a.per_head ? d0 : idx * 8;
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(a.weight[tns] + (int64_t)wi * 2));
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
            const uint64_t rs2 = f2(rs, rs);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float g0, g1, y0, y1;
              Cvt<T>::unpack(ww[e], g0, g1);
              // one rounding to the storage type after scale and weight, as a fused RMSNorm does
              f2_get(f2_mul(f2_mul(x2[e], rs2), f2(g0, g1)), y0, y1);
              Cvt<T>::unpack(Cvt<T>::pack(y0, y1), y0, y1);
              x2[e] = f2(y0, y1);
            }
          }
        }
        if (!live) continue;
        if (rope) {
          uint64_t c_vec[4], s_vec[4];
          const uint64_t* c2 = c_row;
          const uint64_t* s2 = s_row;
          if (!same_col) {
            load_cs(d0, c_vec, s_vec);
            c2 = c_vec;
            s2 = s_vec;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // pair (x1, x2) = elements (2e, 2e+1): (x1 cos - x2 sin, x2 cos + x1 sin)
            float x1, xx;
            f2_get(x2[e], x1, xx);
            x2[e] = f2_fma(x2[e], c2[e], f2_mul(f2(xx, x1), s2[e]));
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float lo, hi;
          f2_get(x2[e], lo, hi);
          o[e] = Cvt<T>::pack(lo, hi);
        }
        *reinterpret_cast<uint4*>(dbase + ((int64_t)dtab[idx] << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
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
  const int nvec = p.H * p.D / 8;
  const int Hl = p.H / p.U;
  for (int i = 0; i < 3; ++i) {
    // a vector's place inside the destination is kept as a 32-bit count of 16-byte units
    const int64_t far = (int64_t)(p.U - 1) * a.dst_peer_stride[i] + (int64_t)(Hl - 1) * a.dst_stride_h[i] + p.D * 2;
    if ((far >> 4) > 0x7fffffffll || (a.dst_peer_stride[i] & 15) || (a.dst_stride_h[i] & 15)) {
      set_error("qk_norm_rope_pack: destination strides out of range (32 GB per batch entry, multiples of 8 elements)");
      return XDIT_E_SHAPE;
    }
  }
  const int64_t ctas = (rows + kWarps - 1) / kWarps;
  const int grid = (int)(ctas < (int64_t)sms * 16 ? ctas : (int64_t)sms * 16);
  const int vpl = (nvec + 31) / 32;  // 1..32
  const size_t smem = (size_t)nvec * (3 * sizeof(int32_t) + sizeof(uint16_t));
  const bool bf = p.dtype == XDIT_BF16;
#define XDIT_LAUNCH_PROLOGUE(V)                                                                              \
  do {                                                                                                       \
    if (bf) qk_norm_rope_pack_kernel<__nv_bfloat16, V, SC><<<grid, kWarps * 32, smem, stream>>>(a);           \
    else qk_norm_rope_pack_kernel<__half, V, SC><<<grid, kWarps * 32, smem, stream>>>(a);                     \
  } while (0)
  if (32 % (p.D / 8) == 0) {
    constexpr bool SC = true;
    if (vpl <= 1) XDIT_LAUNCH_PROLOGUE(1);
    else if (vpl <= 2) XDIT_LAUNCH_PROLOGUE(2);
    else if (vpl <= 3) XDIT_LAUNCH_PROLOGUE(3);
    else if (vpl <= 4) XDIT_LAUNCH_PROLOGUE(4);
    else if (vpl <= 6) XDIT_LAUNCH_PROLOGUE(6);
    else if (vpl <= 8) XDIT_LAUNCH_PROLOGUE(8);
    else if (vpl <= 10) XDIT_LAUNCH_PROLOGUE(10);
    else if (vpl <= 12) XDIT_LAUNCH_PROLOGUE(12);
    else if (vpl <= 16) XDIT_LAUNCH_PROLOGUE(16);
    else if (vpl <= 20) XDIT_LAUNCH_PROLOGUE(20);
    else if (vpl <= 24) XDIT_LAUNCH_PROLOGUE(24);
    else XDIT_LAUNCH_PROLOGUE(kMaxVpl);
  } else {  // head_dim such as 72: every vector looks up its own column and rotation factors
    constexpr bool SC = false;
    if (vpl <= 4) XDIT_LAUNCH_PROLOGUE(4);
    else if (vpl <= 8) XDIT_LAUNCH_PROLOGUE(8);
    else if (vpl <= 16) XDIT_LAUNCH_PROLOGUE(16);
    else XDIT_LAUNCH_PROLOGUE(kMaxVpl);
  }
#undef XDIT_LAUNCH_PROLOGUE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "qk_norm_rope_pack_kernel launch");
  return XDIT_OK;
}

}  // namespace xdit
