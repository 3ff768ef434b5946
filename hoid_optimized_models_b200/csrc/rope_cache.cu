// (QK-RMSNorm +) rotate-half RoPE + KV-cache write, one CTA per token, hd/8 lanes per head.
//
// Heads of the packed projection row are laid out q[0..n_q), k[0..n_kv),
// v[0..n_kv).  q heads go to q_out, k heads are normalised/rotated straight
// into the cache row `pos0 + t`, v heads are copied into the cache.
#include "common.cuh"

namespace b200 {

struct RopeArgs {
  void* q_out; uint16_t* kcache; uint16_t* vcache; const void* qkv;
  const uint16_t* qn_w; const uint16_t* kn_w; const float* cos_t; const float* sin_t;
  const int* pos_dev;
  int s, n_q, n_kv, hd, max_seq, q_dtype, qkv_dtype; float eps;
};

__device__ __forceinline__ void ld4(const void* p, int dtype, size_t i, float* f) {
  if (dtype == B200_F32) {
    const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p) + i);
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  }
}
__device__ __forceinline__ void st4(void* p, int dtype, size_t i, const float* f) {
  if (dtype == B200_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    uint2 v;
    v.x = pack_bf16(f[0], f[1]); v.y = pack_bf16(f[2], f[3]);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p) + i) = v;
  }
}

// One CTA per token.  A group of LPH = hd/8 lanes owns one head at a time and walks the token's
// heads (q, then k, then v) with a stride of the CTA's group count: lane l of the group holds
// dims [4l, 4l+4) of the first half and the matching four of the second half, so every access is
// 8 or 16 bytes wide, the token's cos / sin values are loaded once per thread instead of once
// per head, and a thread's loads of successive heads are independent (several in flight).
constexpr int kRopeThreads = 128;

__global__ void __launch_bounds__(kRopeThreads) qk_rope_cache_kernel(RopeArgs a) {
  const int hd = a.hd, half = hd >> 1;
  const int lph = half >> 2;                       // lanes per head: 16 (hd 128) or 8 (hd 64)
  const int grp = threadIdx.x / lph, l = threadIdx.x - grp * lph;
  const int ngrp = kRopeThreads / lph;
  const int lane = threadIdx.x & 31;
  const int sub = lane / lph;                      // group inside the warp
  const int slots = a.n_q + 2 * a.n_kv;
  const int token = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = a.pos_dev[0] + token;
  const bool in_cache = pos >= 0 && pos < a.max_seq;   // never write outside the cache
  float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
  if (in_cache) {                                  // the tables have max_seq rows
    ld4(a.cos_t, B200_F32, (size_t)pos * half + 4 * l, c);
    ld4(a.sin_t, B200_F32, (size_t)pos * half + 4 * l, sn);
  }
  float wq[2][4], wk[2][4];
  const bool normed = a.qn_w != nullptr;           // all q and k heads or none
  if (normed) {
    ld4(a.qn_w, B200_BF16, 4 * l, wq[0]); ld4(a.qn_w, B200_BF16, half + 4 * l, wq[1]);
    ld4(a.kn_w, B200_BF16, 4 * l, wk[0]); ld4(a.kn_w, B200_BF16, half + 4 * l, wk[1]);
  }
  const unsigned gmask = (lph == 32 ? 0xffffffffu : ((1u << lph) - 1u)) << (sub * lph);
  const int n_rot = a.n_q + a.n_kv;
  // every group of a warp runs the same number of iterations (the shuffles below need the
  // group's lanes, not the warp's, but a uniform trip count keeps the code simple)
  for (int h0 = 0; h0 < slots; h0 += ngrp) {
    const int h = h0 + grp;
    if (h >= slots) break;                         // whole groups leave together
    const size_t src0 = ((size_t)token * slots + h) * hd;
    if (h < n_rot) {
      const bool is_q = h < a.n_q;
      float lo[4], hi[4];
      ld4(a.qkv, a.qkv_dtype, src0 + 4 * l, lo);
      ld4(a.qkv, a.qkv_dtype, src0 + half + 4 * l, hi);
      if (normed) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
        for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(gmask, ss, o);
        const float inv = rsqrtf(ss / (float)hd + a.eps);
        const float (*w)[4] = is_q ? wq : wk;
#pragma unroll
        for (int e = 0; e < 4; ++e) { lo[e] = lo[e] * inv * w[0][e]; hi[e] = hi[e] * inv * w[1][e]; }
      }
      if (!is_q && !in_cache) continue;
      float r0[4], r1[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        r0[e] = lo[e] * c[e] - hi[e] * sn[e];
        r1[e] = hi[e] * c[e] + lo[e] * sn[e];
      }
      if (is_q) {
        const size_t d = ((size_t)token * a.n_q + h) * hd;
        st4(a.q_out, a.q_dtype, d + 4 * l, r0);
        st4(a.q_out, a.q_dtype, d + half + 4 * l, r1);
      } else {
        const size_t d = ((size_t)(h - a.n_q) * a.max_seq + pos) * hd;
        st4(a.kcache, B200_BF16, d + 4 * l, r0);
        st4(a.kcache, B200_BF16, d + half + 4 * l, r1);
      }
    } else {
      if (!in_cache) continue;
      const size_t d = ((size_t)(h - n_rot) * a.max_seq + pos) * hd;
      float x[4], y[4];
      ld4(a.qkv, a.qkv_dtype, src0 + 8 * l, x);
      ld4(a.qkv, a.qkv_dtype, src0 + 8 * l + 4, y);
      st4(a.vcache, B200_BF16, d + 8 * l, x);
      st4(a.vcache, B200_BF16, d + 8 * l + 4, y);
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_qk_rope_cache(void* q_out, int q_dtype, void* kcache, void* vcache,
                                  const void* qkv, int qkv_dtype,
                                  const void* qn_w, const void* kn_w,
                                  const float* cos_t, const float* sin_t,
                                  const int* pos_dev, int s, int n_q, int n_kv, int hd,
                                  int max_seq, float eps, int flags, b200_stream_t stream) {
  if (!q_out || !kcache || !vcache || !qkv || !cos_t || !sin_t || !pos_dev) return B200_ERR_ARG;
  if (s <= 0 || n_q <= 0 || n_kv <= 0 || (hd != 64 && hd != 128) || max_seq <= 0)
    return B200_ERR_SHAPE;
  if ((qn_w == nullptr) != (kn_w == nullptr)) return B200_ERR_ARG;
  RopeArgs a{q_out, (uint16_t*)kcache, (uint16_t*)vcache, qkv, (const uint16_t*)qn_w,
             (const uint16_t*)kn_w, cos_t, sin_t, pos_dev, s, n_q, n_kv, hd, max_seq,
             q_dtype, qkv_dtype, eps};
  cudaError_t e = launch(qk_rope_cache_kernel, dim3((unsigned)s), dim3(kRopeThreads), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, a);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
