// (QK-RMSNorm +) rotate-half RoPE + KV-cache write, one warp per (token, head).
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

__device__ __forceinline__ float ld_elem(const void* p, int dtype, size_t i) {
  return dtype == B200_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__global__ void __launch_bounds__(128) qk_rope_cache_kernel(RopeArgs a) {
  const int lane = threadIdx.x & 31;
  const int slots = a.n_q + 2 * a.n_kv;
  const long slot = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  pdl_launch_dependents();
  pdl_wait();
  if (slot >= (long)a.s * slots) return;
  const int token = (int)(slot / slots);
  const int h = (int)(slot - (long)token * slots);
  const int pos = a.pos_dev[0] + token;
  if (pos < 0 || pos >= a.max_seq) return;  // never write outside the cache
  const int hd = a.hd, half = hd >> 1;
  const size_t src0 = ((size_t)token * slots + h) * hd;

  if (h < a.n_q + a.n_kv) {
    const bool is_q = h < a.n_q;
    const uint16_t* nw = is_q ? a.qn_w : a.kn_w;
    float lo[2], hi[2];
    float ss = 0.f;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int p = lane + t * 32;
      lo[t] = hi[t] = 0.f;
      if (p < half) {
        lo[t] = ld_elem(a.qkv, a.qkv_dtype, src0 + p);
        hi[t] = ld_elem(a.qkv, a.qkv_dtype, src0 + p + half);
        ss += lo[t] * lo[t] + hi[t] * hi[t];
      }
    }
    float inv = 1.f;
    if (nw != nullptr) {
      ss = warp_sum(ss);
      inv = rsqrtf(ss / (float)hd + a.eps);
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int p = lane + t * 32;
      if (p < half) {
        float x = lo[t], y = hi[t];
        if (nw != nullptr) {
          x = x * inv * __uint_as_float((uint32_t)nw[p] << 16);
          y = y * inv * __uint_as_float((uint32_t)nw[p + half] << 16);
        }
        const float c = a.cos_t[(size_t)pos * half + p];
        const float sn = a.sin_t[(size_t)pos * half + p];
        const float r0 = x * c - y * sn;
        const float r1 = y * c + x * sn;
        if (is_q) {
          const size_t d = ((size_t)token * a.n_q + h) * hd;
          if (a.q_dtype == B200_F32) {
            reinterpret_cast<float*>(a.q_out)[d + p] = r0;
            reinterpret_cast<float*>(a.q_out)[d + p + half] = r1;
          } else {
            reinterpret_cast<__nv_bfloat16*>(a.q_out)[d + p] = __float2bfloat16(r0);
            reinterpret_cast<__nv_bfloat16*>(a.q_out)[d + p + half] = __float2bfloat16(r1);
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.kcache) +
                               ((size_t)(h - a.n_q) * a.max_seq + pos) * hd;
          dst[p] = __float2bfloat16(r0);
          dst[p + half] = __float2bfloat16(r1);
        }
      }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.vcache) +
                         ((size_t)(h - a.n_q - a.n_kv) * a.max_seq + pos) * hd;
    for (int d = lane; d < hd; d += 32)
      dst[d] = __float2bfloat16(ld_elem(a.qkv, a.qkv_dtype, src0 + d));
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
  const long warps = (long)s * (n_q + 2 * n_kv);
  const unsigned grid = (unsigned)((warps + 3) / 4);
  cudaError_t e = launch(qk_rope_cache_kernel, dim3(grid), dim3(128), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, a);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
