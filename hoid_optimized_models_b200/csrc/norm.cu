// Fused (bias +) residual-add + RMSNorm / LayerNorm over rows.
//
// One CTA per row, eight elements per thread per step, the whole row held in
// registers between the statistics pass and the normalising pass so that every
// input byte is read from HBM exactly once.  Loads and stores are 128-bit.
#include "common.cuh"

namespace b200 {

constexpr int kNormChunkCap = 8;  // 8-element chunks per thread -> N <= threads * 64
// The kernels are instantiated for 1, 2, 4 and 8 chunks per thread so that narrow rows do not
// pay the register (= occupancy) cost of wide ones.

__device__ __forceinline__ void load8(const void* p, int dtype, size_t chunk, float* f) {
  if (dtype == B200_F32) {
    const float4* q = reinterpret_cast<const float4*>(p) + chunk * 2;
    float4 a = q[0], b = q[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    uint4 w = reinterpret_cast<const uint4*>(p)[chunk];
    unpack8(w, f);
  }
}
__device__ __forceinline__ void store8(void* p, int dtype, size_t chunk, const float* f) {
  if (dtype == B200_F32) {
    float4* q = reinterpret_cast<float4*>(p) + chunk * 2;
    q[0] = make_float4(f[0], f[1], f[2], f[3]);
    q[1] = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    uint4 w;
    w.x = pack_bf16(f[0], f[1]); w.y = pack_bf16(f[2], f[3]);
    w.z = pack_bf16(f[4], f[5]); w.w = pack_bf16(f[6], f[7]);
    reinterpret_cast<uint4*>(p)[chunk] = w;
  }
}
__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16(v));
}

// The residual stream (a, resid_out) may be fp32 while the delta b and the normalised output
// are bf16: an fp32 stream keeps the error against an fp32 model flat over depth.
struct RmsArgs {
  void* resid_out; void* norm_out; const void* a; const void* b; const uint16_t* w;
  int N, resid_dtype, b_dtype, out_dtype; float eps;
};

template <int kNormMaxChunks>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(RmsArgs p) {
  __shared__ float red[32];
  const int nchunk = p.N >> 3;
  const size_t row0 = (size_t)blockIdx.x * nchunk;
  pdl_launch_dependents();
  pdl_wait();
  float v[kNormMaxChunks][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nchunk) {
      load8(p.a, p.resid_dtype, row0 + i, v[c]);
      if (p.b != nullptr) {
        float t[8];
        load8(p.b, p.b_dtype, row0 + i, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[c][e] += t[e];
      }
      // normalise the value the residual stream stores
      if (p.resid_dtype == B200_BF16) {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[c][e] = round_bf16(v[c][e]);
      }
      if (p.resid_out != nullptr) store8(p.resid_out, p.resid_dtype, row0 + i, v[c]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(v[c][e], v[c][e], ss);
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / (float)p.N + p.eps);
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nchunk) {
      float g[8], o[8];
      unpack8(reinterpret_cast<const uint4*>(p.w)[i], g);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[c][e] * inv * g[e];
      store8(p.norm_out, p.out_dtype, row0 + i, o);
    }
  }
}

struct LnArgs {
  void* resid_out; void* norm_out; const void* x; const uint16_t* bias; const void* resid;
  const uint16_t* gamma; const uint16_t* beta;
  int N, in_dtype, out_dtype; float eps;
};

template <int kNormMaxChunks>
__global__ void __launch_bounds__(256) add_layernorm_kernel(LnArgs p) {
  __shared__ float red[32];
  const int nchunk = p.N >> 3;
  const size_t row0 = (size_t)blockIdx.x * nchunk;
  pdl_launch_dependents();
  pdl_wait();
  const bool rb = (p.in_dtype == B200_BF16);  // reference rounds each bf16 addition
  float v[kNormMaxChunks][8];
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nchunk) {
      load8(p.x, p.in_dtype, row0 + i, v[c]);
      if (p.bias != nullptr) {
        float t[8];
        unpack8(reinterpret_cast<const uint4*>(p.bias)[i], t);
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[c][e] += t[e]; if (rb) v[c][e] = round_bf16(v[c][e]); }
      }
      if (p.resid != nullptr) {
        float t[8];
        load8(p.resid, p.in_dtype, row0 + i, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) { v[c][e] += t[e]; if (rb) v[c][e] = round_bf16(v[c][e]); }
      }
      if (p.resid_out != nullptr) store8(p.resid_out, p.out_dtype, row0 + i, v[c]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[c][e];
    }
  }
  const float mean = block_sum(s, red) / (float)p.N;
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nchunk) {
#pragma unroll
      for (int e = 0; e < 8; ++e) { const float d = v[c][e] - mean; q = fmaf(d, d, q); }
    }
  }
  const float inv = rsqrtf(block_sum(q, red) / (float)p.N + p.eps);
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < nchunk) {
      float g[8], b[8], o[8];
      unpack8(reinterpret_cast<const uint4*>(p.gamma)[i], g);
      unpack8(reinterpret_cast<const uint4*>(p.beta)[i], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[c][e] - mean) * inv * g[e] + b[e];
      store8(p.norm_out, p.out_dtype, row0 + i, o);
    }
  }
}

static int norm_threads(int N) {
  int t = ((N >> 3) + 31) & ~31;       // one chunk per thread if it fits
  if (t > 256) t = 256;
  if (t < 32) t = 32;
  return t;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_add_rmsnorm(void* resid_out, void* norm_out, int out_dtype,
                                const void* a, int resid_dtype, const void* b, int b_dtype,
                                const void* w, int rows, int N, float eps,
                                int flags, b200_stream_t stream) {
  if (!norm_out || !a || !w) return B200_ERR_ARG;
  if (rows <= 0 || N <= 0 || (N & 7) != 0) return B200_ERR_SHAPE;
  const int threads = norm_threads(N);
  if ((N >> 3) > threads * kNormChunkCap) return B200_ERR_SHAPE;
  RmsArgs p{resid_out, norm_out, a, b, (const uint16_t*)w, N, resid_dtype, b_dtype, out_dtype, eps};
  const int cpt = ((N >> 3) + threads - 1) / threads;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (cpt <= 1) e = launch(add_rmsnorm_kernel<1>, dim3(rows), dim3(threads), 0, st, pdl, p);
  else if (cpt <= 2) e = launch(add_rmsnorm_kernel<2>, dim3(rows), dim3(threads), 0, st, pdl, p);
  else if (cpt <= 4) e = launch(add_rmsnorm_kernel<4>, dim3(rows), dim3(threads), 0, st, pdl, p);
  else e = launch(add_rmsnorm_kernel<8>, dim3(rows), dim3(threads), 0, st, pdl, p);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int b200_add_layernorm(void* resid_out, void* norm_out, int out_dtype,
                                  const void* x, const void* bias, const void* resid, int in_dtype,
                                  const void* gamma, const void* beta,
                                  int rows, int N, float eps, int flags, b200_stream_t stream) {
  if (!norm_out || !x || !gamma || !beta) return B200_ERR_ARG;
  if (rows <= 0 || N <= 0 || (N & 7) != 0) return B200_ERR_SHAPE;
  const int threads = norm_threads(N);
  if ((N >> 3) > threads * kNormChunkCap) return B200_ERR_SHAPE;
  LnArgs p{resid_out, norm_out, x, (const uint16_t*)bias, resid, (const uint16_t*)gamma,
           (const uint16_t*)beta, N, in_dtype, out_dtype, eps};
  const int cpt = ((N >> 3) + threads - 1) / threads;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (cpt <= 1) e = launch(add_layernorm_kernel<1>, dim3(rows), dim3(threads), 0, st, pdl, p);
  else if (cpt <= 2) e = launch(add_layernorm_kernel<2>, dim3(rows), dim3(threads), 0, st, pdl, p);
  else if (cpt <= 4) e = launch(add_layernorm_kernel<4>, dim3(rows), dim3(threads), 0, st, pdl, p);
  else e = launch(add_layernorm_kernel<8>, dim3(rows), dim3(threads), 0, st, pdl, p);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
