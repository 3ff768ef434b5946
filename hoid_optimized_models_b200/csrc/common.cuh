// Shared device helpers for the sm_100a kernels in this directory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/b200ops.h"

#define B200_CHECK_LAUNCH()                                   \
  do {                                                        \
    cudaError_t e__ = cudaPeekAtLastError();                  \
    if (e__ != cudaSuccess) return B200_ERR_LAUNCH;           \
  } while (0)

namespace b200 {

constexpr int kNumSMs = 148;
constexpr int kMaxDevices = 64;   // per-device host-side caches are indexed by cudaGetDevice()

// Tuning knobs set through b200_set_tuning (defined in misc.cu).
extern int g_tuning[16];

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 128-bit streaming load that bypasses L1 allocation (weights / KV rows are used once).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// Two bf16 packed in a 32-bit word -> two fp32 (exact).
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void unpack8(const uint4& w, float* f) {
  f[0] = bf16lo(w.x); f[1] = bf16hi(w.x);
  f[2] = bf16lo(w.y); f[3] = bf16hi(w.y);
  f[4] = bf16lo(w.z); f[5] = bf16hi(w.z);
  f[6] = bf16lo(w.w); f[7] = bf16hi(w.w);
}

// Exact-erf GELU: erf by Abramowitz & Stegun 7.1.26 (absolute error <= 1.5e-7 plus the ~1e-7
// of the approximate reciprocal / exp2, far below bf16 resolution): two special-function-unit
// operations and about a dozen FMAs per element, so that it fits in a GEMM epilogue.
__device__ __forceinline__ float gelu_erf(float v) {
  const float z = fabsf(v) * 0.70710678118654752440f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  float poly = fmaf(t, 1.061405429f, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z * z * 1.4426950408889634f));
  const float erf_abs = 1.f - poly * t * e;
  return 0.5f * v * (1.f + copysignf(erf_abs, v));
}

// Programmatic dependent launch: let the next kernel in the stream start its
// independent prologue, and wait for the previous kernel's results.  Both are
// no-ops when the launch carries no programmatic-serialization attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Block-wide sum for blockDim.x <= 1024; `red` is >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protect `red` from a previous use
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float t = 0.f;
  // fixed order: every thread adds the warp partials in index order
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

// Opt a kernel in to `bytes` of dynamic shared memory, once per device: the attribute belongs to
// the (function, device) pair, so a process that drives several GPUs must set it on each.
// `done` is a per-call-site array of kMaxDevices flags.
template <typename... KArgs>
inline cudaError_t opt_in_smem(void (*kernel)(KArgs...), int bytes, bool* done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[dev] = true;
  return e;
}

// Launch helper that optionally attaches the programmatic-stream-serialization
// attribute (flag B200_FLAG_PDL).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200
