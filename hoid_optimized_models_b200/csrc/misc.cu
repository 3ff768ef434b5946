// Small ops of the token loop: embedding gather, SwiGLU activation, greedy argmax.
#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embed_gather_kernel(void* out, int out_dtype,
                                                           const uint16_t* table, const int* ids,
                                                           int rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int cpr = H >> 3;  // 8-element chunks per row
  const long total = (long)rows * cpr;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / cpr), c = (int)(i - (long)r * cpr);
    const uint4 w = reinterpret_cast<const uint4*>(table + (size_t)ids[r] * H)[c];
    if (out_dtype == B200_F32) {
      float f[8];
      unpack8(w, f);
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)r * H) + c * 2;
      o[0] = make_float4(f[0], f[1], f[2], f[3]);
      o[1] = make_float4(f[4], f[5], f[6], f[7]);
    } else {
      reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + (size_t)r * H)[c] = w;
    }
  }
}

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) silu_mul_kernel(uint4* out, const uint4* gate,
                                                       const uint4* up, long nchunk) {
  pdl_launch_dependents();
  pdl_wait();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nchunk;
       i += (long)gridDim.x * blockDim.x) {
    float g[8], u[8];
    unpack8(gate[i], g);
    unpack8(up[i], u);
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    uint4 w;
    w.x = pack_bf16(o[0], o[1]); w.y = pack_bf16(o[2], o[3]);
    w.z = pack_bf16(o[4], o[5]); w.w = pack_bf16(o[6], o[7]);
    out[i] = w;
  }
}

// ---------------------------------------------------------------------------
// argmax with lowest-index tie-break; two levels in one launch (last CTA finishes).
struct Best { float v; int i; };
__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__global__ void __launch_bounds__(256) argmax_kernel(int* idx_out, float* max_out,
                                                     const float* x, int n, int idx_base,
                                                     int* counter, Best* partial) {
  __shared__ Best sb[8];
  __shared__ int s_last;
  pdl_launch_dependents();
  pdl_wait();
  Best b{-INFINITY, 0x7fffffff};
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float v = x[i];
    if (v > b.v) { b.v = v; b.i = i; }
  }
  auto block_best = [&](Best t) -> Best {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best u{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
      t = better(t, u);
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sb[threadIdx.x >> 5] = t;
    __syncthreads();
    Best r = sb[0];
    for (int w = 1; w < 8; ++w) r = better(r, sb[w]);
    return r;
  };
  b = block_best(b);
  if (threadIdx.x == 0) {
    partial[blockIdx.x] = b;
    __threadfence();
    s_last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  Best f{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
    Best u{__ldcg(&partial[i].v), __ldcg(&partial[i].i)};
    f = better(f, u);
  }
  f = block_best(f);
  if (threadIdx.x == 0) {
    idx_out[0] = (f.i == 0x7fffffff ? 0 : f.i) + idx_base;
    if (max_out != nullptr) max_out[0] = f.v;
    *counter = 0;
  }
}

// out[b, :] = x[b * row_stride : +H] / max(||x||_2, eps): first-token pooling + L2 normalisation.
__global__ void __launch_bounds__(256) cls_pool_l2_kernel(float* out, const uint16_t* x,
                                                          long row_stride, int H, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const uint16_t* row = x + (size_t)blockIdx.x * row_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = __uint_as_float((uint32_t)row[i] << 16);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / fmaxf(sqrtf(block_sum(ss, red)), eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    out[(size_t)blockIdx.x * H + i] = __uint_as_float((uint32_t)row[i] << 16) * inv;
}

// Pick the best of n (value, index) candidates (one per tensor-parallel rank; n = 1 on a
// single GPU), publish it as the next input token, append it to the token log and advance
// the step state {position, kv_len, tokens generated}.
__global__ void greedy_select_kernel(int* tok_out, const Best* cand, int n, int* state, int* log,
                                     int log_cap) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x != 0) return;
  Best b = cand[0];
  for (int i = 1; i < n; ++i) b = better(b, cand[i]);
  tok_out[0] = b.i;
  if (state != nullptr) {
    const int k = state[2];
    if (log != nullptr && k < log_cap) log[k] = b.i;
    state[0] += 1; state[1] += 1; state[2] = k + 1;
  }
}

}  // namespace b200

using namespace b200;

namespace b200 { int g_tuning[16] = {0}; }

extern "C" int b200_set_tuning(int key, int value) {
  if (key < 0 || key >= 16) return B200_ERR_ARG;
  g_tuning[key] = value;
  return B200_OK;
}

extern "C" int b200_version(void) { return 100; }
extern "C" int b200_sm_count(void) { return kNumSMs; }

extern "C" int b200_embed_gather(void* out, int out_dtype, const void* table, const int* ids,
                                 int rows, int H, int flags, b200_stream_t stream) {
  if (!out || !table || !ids) return B200_ERR_ARG;
  if (rows <= 0 || H <= 0 || (H & 7) != 0) return B200_ERR_SHAPE;
  const long total = (long)rows * (H >> 3);
  int grid = (int)((total + 255) / 256);
  if (grid > kNumSMs * 8) grid = kNumSMs * 8;
  cudaError_t e = launch(embed_gather_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, out, out_dtype, (const uint16_t*)table, ids,
                         rows, H);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int b200_silu_mul(void* out, const void* gate, const void* up, int64_t n, int flags,
                             b200_stream_t stream) {
  if (!out || !gate || !up) return B200_ERR_ARG;
  if (n <= 0 || (n & 7) != 0) return B200_ERR_SHAPE;
  const long nchunk = n >> 3;
  int grid = (int)((nchunk + 255) / 256);
  if (grid > kNumSMs * 8) grid = kNumSMs * 8;
  cudaError_t e = launch(silu_mul_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, (uint4*)out, (const uint4*)gate,
                         (const uint4*)up, nchunk);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int b200_cls_pool_l2(float* out, const void* x, int batch, int64_t row_stride, int H,
                                float eps, int flags, b200_stream_t stream) {
  if (!out || !x) return B200_ERR_ARG;
  if (batch <= 0 || H <= 0) return B200_ERR_SHAPE;
  cudaError_t e = launch(cls_pool_l2_kernel, dim3(batch), dim3(256), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, out, (const uint16_t*)x, (long)row_stride, H,
                         eps);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int64_t b200_argmax_workspace_bytes(int n) {
  (void)n;
  return 256 + (int64_t)kNumSMs * sizeof(Best);
}

extern "C" int b200_greedy_select(int* tok_out, const void* cand, int n, int* state, int* log,
                                  int log_cap, int flags, b200_stream_t stream) {
  if (!tok_out || !cand || n <= 0) return B200_ERR_ARG;
  cudaError_t e = launch(greedy_select_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, tok_out, (const Best*)cand, n, state, log,
                         log_cap);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int b200_argmax_f32(int* idx_out, float* max_out, const float* logits, int n,
                               int idx_base, void* workspace, int flags, b200_stream_t stream) {
  if (!idx_out || !logits || !workspace) return B200_ERR_ARG;
  if (n <= 0) return B200_ERR_SHAPE;
  int grid = (n + 2047) / 2048;
  if (grid > kNumSMs) grid = kNumSMs;
  cudaError_t e = launch(argmax_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, idx_out, max_out, logits, n, idx_base,
                         (int*)workspace, (Best*)((char*)workspace + 256));
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
