// Mixture-of-experts routing: top-k softmax router, stable expert-major permutation
// (counting sort), row gather and weighted un-permute.  All index work is integer and
// deterministic; the permutation equals a stable argsort of the flattened expert ids.
#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// Router: softmax over E logits (fp32), top-k with lowest-index tie-break,
// weights renormalised over the selected experts.  One warp per token; lane l
// owns experts l, l + 32, ...
constexpr int kMaxEPL = 8;  // experts per lane -> E <= 256

// Softmax + top-k of one token's logits by one warp: v[j] is the logit of expert lane + 32 j
// (-inf beyond E).  A non-finite logit (NaN, +inf) would turn every probability into NaN and no
// comparison below would ever hold; such probabilities are replaced by zero, so the ids written
// are always valid expert numbers, and the caller's status word (nullable) gets B200_ERR_NUMERIC.
__device__ __forceinline__ void router_select(const float* v, int epl, int top_k, int round_bf16,
                                              int lane, int* ids, float* wts, int* status) {
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxEPL; ++j) mx = fmaxf(mx, v[j]);
  mx = warp_max(mx);
  float p[kMaxEPL];
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxEPL; ++j) {
    p[j] = j < epl ? expf(v[j] - mx) : 0.f;
    sum += p[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  bool bad = false;
#pragma unroll
  for (int j = 0; j < kMaxEPL; ++j) {
    p[j] *= inv;                                   // softmax probabilities
    if (!(p[j] >= 0.f && p[j] <= 1.f)) { p[j] = 0.f; bad = true; }
  }
  if (__any_sync(0xffffffffu, bad) && lane == 0 && status != nullptr)
    atomicExch(status, B200_ERR_NUMERIC);

  float sel_w = 0.f;   // lane k keeps the k-th selection
  int sel_i = 0;
  float wsum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    // lane-local best (lowest index wins ties), then warp argmax with the same rule
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxEPL; ++j) {
      if (j < epl && p[j] > bv) { bv = p[j]; bi = lane + 32 * j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == k) { sel_w = bv; sel_i = bi; }
    wsum += bv;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kMaxEPL; ++j)
        if (j == (bi >> 5)) p[j] = -1.f;   // taken
    }
  }
  if (lane < top_k) {
    float w = wsum > 0.f ? sel_w / wsum : 0.f;
    if (round_bf16) w = __bfloat162float(__float2bfloat16(w));
    ids[lane] = sel_i;
    wts[lane] = w;
  }
}

__global__ void __launch_bounds__(128) moe_router_kernel(int* ids, float* wts, const void* logits,
                                                         int logits_dtype, int s, int E, int top_k,
                                                         int round_bf16, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= s) return;
  const int epl = E >> 5;
  float v[kMaxEPL];
#pragma unroll
  for (int j = 0; j < kMaxEPL; ++j) {
    v[j] = -INFINITY;
    if (j < epl) {
      const size_t i = (size_t)t * E + lane + 32 * j;
      v[j] = logits_dtype == B200_F32
                 ? reinterpret_cast<const float*>(logits)[i]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[i]);
    }
  }
  router_select(v, epl, top_k, round_bf16, lane, ids + (size_t)t * top_k, wts + (size_t)t * top_k,
                status);
}

// ---------------------------------------------------------------------------
// Stable counting sort of `pairs` (token, slot) entries by expert id.
//   pass 1: per-block histograms                     hist[block][E]
//   pass 2: per-expert scan over blocks -> offsets[E+1], hist becomes each block's first
//           output position per expert
//   pass 3: thread e of a block walks the block's entries in order and places those of
//           expert e, which keeps equal keys in their original order.
constexpr int kSortBlock = 1024;  // entries per block

// An id outside [0, E) (a caller error) must not index shared memory: it is sorted as expert 0,
// consistently in both passes, and the status word (nullable) receives B200_ERR_ARG.
__device__ __forceinline__ int moe_checked_id(int id, int E, int* status) {
  if ((unsigned)id < (unsigned)E) return id;
  if (status != nullptr) atomicExch(status, B200_ERR_ARG);
  return 0;
}

__global__ void __launch_bounds__(256) moe_hist_kernel(int* hist, const int* ids, int pairs, int E,
                                                       int* status) {
  extern __shared__ int sh[];
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortBlock;
  for (int i = threadIdx.x; i < kSortBlock && base + i < pairs; i += blockDim.x)
    atomicAdd(&sh[moe_checked_id(ids[base + i], E, status)], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[blockIdx.x * E + e] = sh[e];
}

__global__ void __launch_bounds__(256) moe_scan_kernel(int* hist, int* offsets, int nblocks, int E) {
  extern __shared__ int tot[];   // [E + 1]
  pdl_launch_dependents();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int b = 0; b < nblocks; ++b) {
      const int h = hist[b * E + e];
      hist[b * E + e] = c;     // position of the block's first entry inside the expert
      c += h;
    }
    tot[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = 0;
    for (int e = 0; e < E; ++e) { const int h = tot[e]; tot[e] = c; offsets[e] = c; c += h; }
    tot[E] = c;
    offsets[E] = c;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nblocks * E; i += blockDim.x) hist[i] += tot[i % E];
}

__global__ void __launch_bounds__(256) moe_place_kernel(int* order, int* inv, const int* hist,
                                                        const int* ids, int pairs, int E) {
  __shared__ int sid[kSortBlock];
  pdl_launch_dependents();
  pdl_wait();
  const int base = blockIdx.x * kSortBlock;
  const int n = min(kSortBlock, pairs - base);
  for (int i = threadIdx.x; i < n; i += blockDim.x) sid[i] = moe_checked_id(ids[base + i], E, nullptr);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int pos = hist[blockIdx.x * E + e];
    for (int i = 0; i < n; ++i) {
      if (sid[i] == e) {
        order[pos] = base + i;
        if (inv != nullptr) inv[base + i] = pos;
        ++pos;
      }
    }
  }
}

// xg[r, :] = x[order[r] / top_k, :]
__global__ void __launch_bounds__(256) moe_gather_kernel(uint4* xg, const uint4* x, const int* order,
                                                         int rows, int top_k, int cpr) {
  pdl_launch_dependents();
  pdl_wait();
  const long total = (long)rows * cpr;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / cpr), c = (int)(i - (long)r * cpr);
    xg[i] = x[(size_t)(order[r] / top_k) * cpr + c];
  }
}

// out[t, :] = (resid[t, :] +) sum_slot w[t, slot] * y[inv[t * top_k + slot], :]   (fp32 sum, slot order)
__global__ void __launch_bounds__(256) moe_combine_kernel(uint4* out, const uint4* y, const int* inv,
                                                          const float* w, const uint4* resid,
                                                          const int* ids, int expert_lo, int n_local,
                                                          int tokens, int top_k, int cpr) {
  pdl_launch_dependents();
  pdl_wait();
  const long total = (long)tokens * cpr;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long)gridDim.x * blockDim.x) {
    const int t = (int)(i / cpr), c = (int)(i - (long)t * cpr);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (resid != nullptr) unpack8(resid[i], acc);
    for (int k = 0; k < top_k; ++k) {
      if (ids != nullptr) {   // expert parallel: rows of experts held elsewhere were not computed
        const int e = ids[(size_t)t * top_k + k] - expert_lo;
        if (e < 0 || e >= n_local) continue;
      }
      const float wk = w[(size_t)t * top_k + k];
      float f[8];
      unpack8(y[(size_t)inv[(size_t)t * top_k + k] * cpr + c], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(wk, f[e], acc[e]);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    out[i] = o;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_router(int* ids, float* wts, const void* logits, int logits_dtype, int s,
                               int E, int top_k, int round_bf16, int* status, int flags,
                               b200_stream_t stream) {
  if (!ids || !wts || !logits) return B200_ERR_ARG;
  if (s <= 0 || E <= 0 || (E & 31) != 0 || E > 32 * kMaxEPL || top_k <= 0 || top_k > 32 ||
      top_k > E)
    return B200_ERR_SHAPE;
  cudaError_t e = launch(moe_router_kernel, dim3((s + 3) / 4), dim3(128), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, ids, wts, logits, logits_dtype, s, E, top_k,
                         round_bf16, status);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int64_t b200_moe_permute_workspace_bytes(int pairs, int E) {
  if (pairs <= 0 || E <= 0) return 0;
  return (int64_t)((pairs + kSortBlock - 1) / kSortBlock) * E * 4;
}

extern "C" int b200_moe_permute(int* order, int* inv, int* offsets, const int* ids, int pairs,
                                int E, void* workspace, int* status, int flags,
                                b200_stream_t stream) {
  if (!order || !offsets || !ids || !workspace) return B200_ERR_ARG;
  if (pairs <= 0 || E <= 0 || E > 4096) return B200_ERR_SHAPE;
  const int nblocks = (pairs + kSortBlock - 1) / kSortBlock;
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  int* hist = (int*)workspace;
  if (launch(moe_hist_kernel, dim3(nblocks), dim3(256), (size_t)E * 4, st, pdl, hist, ids, pairs,
             E, status) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (launch(moe_scan_kernel, dim3(1), dim3(256), (size_t)(E + 1) * 4, st, pdl, hist, offsets,
             nblocks, E) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (launch(moe_place_kernel, dim3(nblocks), dim3(256), 0, st, pdl, order, inv, (const int*)hist,
             ids, pairs, E) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return B200_OK;
}

extern "C" int b200_moe_gather_rows(void* xg, const void* x, const int* order, int rows, int top_k,
                                    int H, int flags, b200_stream_t stream) {
  if (!xg || !x || !order) return B200_ERR_ARG;
  if (rows <= 0 || top_k <= 0 || H <= 0 || (H & 7) != 0) return B200_ERR_SHAPE;
  const long total = (long)rows * (H >> 3);
  int grid = (int)((total + 255) / 256);
  if (grid > kNumSMs * 16) grid = kNumSMs * 16;
  cudaError_t e = launch(moe_gather_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, (uint4*)xg, (const uint4*)x, order, rows,
                         top_k, H >> 3);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int b200_moe_combine(void* out, const void* y, const int* inv, const float* wts,
                                const void* resid, const int* ids, int expert_lo, int n_local,
                                int tokens, int top_k, int H, int flags, b200_stream_t stream) {
  if (!out || !y || !inv || !wts) return B200_ERR_ARG;
  if (tokens <= 0 || top_k <= 0 || H <= 0 || (H & 7) != 0) return B200_ERR_SHAPE;
  const long total = (long)tokens * (H >> 3);
  int grid = (int)((total + 255) / 256);
  if (grid > kNumSMs * 16) grid = kNumSMs * 16;
  cudaError_t e = launch(moe_combine_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, (uint4*)out, (const uint4*)y, inv, wts,
                         (const uint4*)resid, ids, expert_lo, n_local, tokens, top_k, H >> 3);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
