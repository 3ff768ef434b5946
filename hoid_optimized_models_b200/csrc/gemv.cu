// Decode GEMV  y[N] = W[N,K] x[K]  — HBM-bound weight streaming for sm_100a.
//
// Work split: each CTA owns a contiguous block of rows.  Inside the CTA the
// block's weights are one flat run of 512-byte "segments" (32 lanes x 16 B =
// 256 bf16 of one row); the run is cut into eight equal pieces, one per warp,
// so every warp streams a contiguous address range with perfectly coalesced
// 128-bit loads and the load imbalance is at most one segment.  A lane keeps a
// private fp32 partial for the row it is in; when the warp crosses a row
// boundary it shuffle-reduces and parks the value in shared memory.  Row sums
// are finished in a fixed order (warp 0..7), so results are bit-reproducible.
//
// The first batch of weight loads is issued before the programmatic-dependent-
// launch wait, so under B200_FLAG_PDL weight streaming overlaps the tail of
// the previous kernel in the stream.  Loads go out in bursts of U per lane
// (4 KB contiguous per warp): bursts measured much faster than a rolling window.
#include <string.h>

#include "common.cuh"
#include "tp_link.cuh"

namespace b200 {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

struct GemvArgs {
  const void* x;
  const uint16_t* w;
  void* y;
  const uint16_t* norm_w;
  const uint16_t* norm_b;    // non-null: LayerNorm (mean / variance, norm_w = gamma, norm_b = beta)
  const uint16_t* bias;
  const void* resid;
  int K, N, ldw, rpc;  // rpc = rows per CTA
  int x_dtype, y_dtype, resid_dtype, epilogue;
  float eps;
  // mixture-of-experts modes (see MODE below)
  const int* expert_ids;     // [n_slots] expert chosen for each routing slot
  const float* slot_scale;   // [n_slots] routing weight folded into the SwiGLU output (MODE 1)
  long expert_stride;        // elements between consecutive experts' matrices
  int segs_per_expert;       // MODE 2: 256-element segments of one expert's K range
  int expert_lo, n_local;    // experts [expert_lo, expert_lo + n_local) live in w (expert parallel)
  // tensor-parallel fusion (see the comment above tp_consume / tp_publish)
  TpLink tp;
  int tp_in, tp_out;         // sequence offsets of the all-reduce to consume / to feed (-1 = none)
  int norm_in_smem;          // RMSNorm: 1 = normalise the staged vector, 0 = scale the row sums
  float* x_out;              // consumer: CTA 0 stores the reduced vector here (nullable)
  int* status;
};

constexpr int kMaxExpertSegs = 256;

// U    : 16-byte loads per lane per batch (two batches are in flight)
// MINB : CTAs per SM the register budget is sized for
// Measured on B200 (graph replay, 32 different weight matrices per case): U = 8 / MINB = 2
// streams 5.9 TB/s on the 235 MB gate|up matrix; deeper prefetch (U = 16, or both batches
// before the wait), a CTA-interleaved segment order and a bulk L2 prefetch of the slice were
// all slower.
// MODE : 0 = dense matrix.
//        1 = expert rows: blockIdx.y is a routing slot, the matrix of expert
//            expert_ids[slot] is used and the output goes to y + slot * (N or N/2).
//        2 = expert columns: x is the concatenation of the slots' activations and row r
//            of the virtual matrix is the concatenation of row r of every chosen
//            expert's matrix, so the sum over the selected experts happens in the dot
//            product itself (one pass, no partial buffers, fixed order).
template <int U, int MINB, int MODE, bool TP = false>
__global__ void __launch_bounds__(kGemvThreads, MINB) gemv_kernel(GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long seg_off[MODE == 2 ? kMaxExpertSegs : 1];
  float* xs = reinterpret_cast<float*>(smem_raw);          // K floats, segment-swizzled
  float* part = xs + a.K;                                    // rpc * kGemvWarps
  float* red = part + a.rpc * kGemvWarps;                    // 32

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = a.K, spr = K >> 8;
  const int r0 = blockIdx.x * a.rpc;
  const int nrows = min(a.N - r0, a.rpc);

  pdl_launch_dependents();
  if (nrows <= 0) return;

  const int S = nrows * spr;  // 512-byte segments owned by the CTA
  // every warp streams its own contiguous eighth of the CTA's segments
  const int s0 = (int)((long)S * warp / kGemvWarps);
  const int s1 = (int)((long)S * (warp + 1) / kGemvWarps);
  const int nbatch = (s1 - s0 + U - 1) / U;
  auto batch_first = [&](int b) -> int { return s0 + b * U; };

  const unsigned char* wb =
      reinterpret_cast<const unsigned char*>(a.w) + (size_t)r0 * a.ldw * 2 + lane * 16;
  const size_t row_bytes = (size_t)a.ldw * 2;
  if (MODE != 0) {
    // the expert choice is produced by the previous kernel
    pdl_wait();
    if (MODE == 1) {
      const int e = a.expert_ids[blockIdx.y] - a.expert_lo;
      if (e < 0 || e >= a.n_local) {
        // the slot's expert lives on another rank: its activations are zero here
        float* o = reinterpret_cast<float*>(a.y) + (size_t)blockIdx.y * (a.N >> 1) + (r0 >> 1);
        for (int t = tid; t < (nrows >> 1); t += kGemvThreads) o[t] = 0.f;
        return;
      }
      wb += (size_t)e * a.expert_stride * 2;
    } else {
      for (int k = tid; k < spr; k += kGemvThreads) {
        const int slot = k / a.segs_per_expert, within = k - slot * a.segs_per_expert;
        const int e = a.expert_ids[slot] - a.expert_lo;
        seg_off[k] = (e < 0 || e >= a.n_local)
                         ? -1 : ((long)e * a.expert_stride + (long)within * 256) * 2;
      }
      __syncthreads();
    }
  }

  auto load_batch = [&](uint4* dst, int b) {
    const int f = batch_first(b);
    int row = f / spr, k = f - row * spr;
#pragma unroll
    for (int j = 0; j < U; ++j) {
      if (f + j < s1) {
        if (MODE == 2) {
          const long off = seg_off[k];
          dst[j] = off < 0 ? make_uint4(0, 0, 0, 0) : ldg_stream(wb + row * row_bytes + off);
        } else {
          dst[j] = ldg_stream(wb + row * row_bytes + (size_t)k * 512);
        }
        if (++k == spr) { k = 0; ++row; }
      }
    }
  };

  uint4 wc[U];
  if (nbatch > 0) load_batch(wc, 0);

  // ---- everything below may depend on the previous kernel ----
  pdl_wait();

  // stage x (fp32, segment-swizzled: [seg][half][lane] float4) and zero the row partials
  float ss = 0.f, sm = 0.f;
  float4* xs4 = reinterpret_cast<float4*>(xs);
  const bool rms_deferred = a.norm_w != nullptr && a.norm_b == nullptr && !a.norm_in_smem;
  unsigned tp_slot = 0, tp_tag = 0;
  if (TP && a.tp_in >= 0) {
    // all-reduce number seq: a few CTAs sum the ranks' contributions, one slice each, and publish
    // the sums locally as tagged pairs; every CTA then polls that one vector (every wait bounded).
    // The inbox is read once per GPU instead of once per CTA.
    const unsigned seq = (unsigned)(a.tp.seq_base[0] + a.tp_in);
    tp_slot = seq & 1u;
    tp_tag = seq + 1u;
    tp_reduce_slice<kGemvThreads>(a.tp, tp_slot, tp_tag, a.x_out, a.status);
  }
  for (int i = tid; i < (K >> 2); i += kGemvThreads) {
    float4 v;
    if (TP && a.tp_in >= 0) {
      v = tp_read_reduced(a.tp, tp_slot, tp_tag, i, a.status);
    } else if (a.x_dtype == B200_F32) {
      v = reinterpret_cast<const float4*>(a.x)[i];
    } else {
      uint2 u = reinterpret_cast<const uint2*>(a.x)[i];
      v = make_float4(bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y));
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    sm += (v.x + v.y) + (v.z + v.w);
    if (rms_deferred) {
      // rmsnorm(x) = (x * w) * rsqrt(mean(x^2) + eps): stage x * w now, the scalar multiplies the
      // row sums in the epilogue, so nothing waits for the sum of squares before the weight loop
      const uint2 u = reinterpret_cast<const uint2*>(a.norm_w)[i];
      v.x *= bf16lo(u.x); v.y *= bf16hi(u.x); v.z *= bf16lo(u.y); v.w *= bf16hi(u.y);
    }
    const int k = i << 2, seg = k >> 8, within = k & 255;
    xs4[seg * 64 + ((within >> 2) & 1) * 32 + (within >> 3)] = v;
  }
  float out_scale = 1.f;
  for (int i = tid; i < a.rpc * kGemvWarps; i += kGemvThreads) part[i] = 0.f;
  if (a.norm_w != nullptr && a.norm_b != nullptr) {
    // LayerNorm prologue: two-pass statistics over the staged vector, like the stand-alone kernel
    const float mean = block_sum(sm, red) / (float)K;
    float qv = 0.f;
    for (int i = tid; i < (K >> 2); i += kGemvThreads) {
      const int k = i << 2, seg = k >> 8, within = k & 255;
      const float4 v = xs4[seg * 64 + ((within >> 2) & 1) * 32 + (within >> 3)];
      const float d0 = v.x - mean, d1 = v.y - mean, d2 = v.z - mean, d3 = v.w - mean;
      qv += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
    }
    const float scale = rsqrtf(block_sum(qv, red) / (float)K + a.eps);
    for (int i = tid; i < (K >> 2); i += kGemvThreads) {
      const int k = i << 2, seg = k >> 8, within = k & 255;
      const int si = seg * 64 + ((within >> 2) & 1) * 32 + (within >> 3);
      const uint2 g = reinterpret_cast<const uint2*>(a.norm_w)[i];
      const uint2 b = reinterpret_cast<const uint2*>(a.norm_b)[i];
      float4 v = xs4[si];
      v.x = (v.x - mean) * scale * bf16lo(g.x) + bf16lo(b.x);
      v.y = (v.y - mean) * scale * bf16hi(g.x) + bf16hi(b.x);
      v.z = (v.z - mean) * scale * bf16lo(g.y) + bf16lo(b.y);
      v.w = (v.w - mean) * scale * bf16hi(g.y) + bf16hi(b.y);
      xs4[si] = v;
    }
  } else if (rms_deferred) {
    out_scale = rsqrtf(block_sum(ss, red) / (float)K + a.eps);   // its barriers also publish xs
  } else if (a.norm_w != nullptr) {
    const float tot = block_sum(ss, red);
    const float scale = rsqrtf(tot / (float)K + a.eps);
    for (int i = tid; i < (K >> 2); i += kGemvThreads) {
      const int k = i << 2, seg = k >> 8, within = k & 255;
      const int si = seg * 64 + ((within >> 2) & 1) * 32 + (within >> 3);
      uint2 u = reinterpret_cast<const uint2*>(a.norm_w)[i];
      float4 v = xs4[si];
      v.x = v.x * scale * bf16lo(u.x);
      v.y = v.y * scale * bf16hi(u.x);
      v.z = v.z * scale * bf16lo(u.y);
      v.w = v.w * scale * bf16hi(u.y);
      xs4[si] = v;
    }
  }
  __syncthreads();

  float acc = 0.f;
  int crow = 0, ck = 0;
  auto flush = [&]() {
    const float v = warp_sum(acc);
    if (lane == 0) part[crow * kGemvWarps + warp] = v;   // a warp meets every row at most once
    acc = 0.f;
  };
  for (int b = 0; b < nbatch; ++b) {
    uint4 wn[U];
    if (b + 1 < nbatch) load_batch(wn, b + 1);
    const int f = batch_first(b);
    if (b == 0) { crow = f / spr; ck = f - crow * spr; }
#pragma unroll
    for (int j = 0; j < U; ++j) {
      if (f + j < s1) {
        const float4 xa = xs4[ck * 64 + lane];
        const float4 xb = xs4[ck * 64 + 32 + lane];
        const uint4 w = wc[j];
        acc = fmaf(bf16lo(w.x), xa.x, acc);
        acc = fmaf(bf16hi(w.x), xa.y, acc);
        acc = fmaf(bf16lo(w.y), xa.z, acc);
        acc = fmaf(bf16hi(w.y), xa.w, acc);
        acc = fmaf(bf16lo(w.z), xb.x, acc);
        acc = fmaf(bf16hi(w.z), xb.y, acc);
        acc = fmaf(bf16lo(w.w), xb.z, acc);
        acc = fmaf(bf16hi(w.w), xb.w, acc);
        if (++ck == spr) { flush(); ck = 0; ++crow; }
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) wc[j] = wn[j];
  }
  if (ck != 0 && s1 > s0) flush();
  __syncthreads();

  // ---- epilogue: fixed-order row sums ----
  auto row_value = [&](int r) -> float {
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kGemvWarps; ++i) v += part[r * kGemvWarps + i];
    v *= out_scale;
    if (a.bias != nullptr) v += __uint_as_float((uint32_t)a.bias[r0 + r] << 16);
    return v;
  };
  if (a.epilogue == B200_EPI_SWIGLU) {
    for (int t = tid; t < (nrows >> 1); t += kGemvThreads) {
      const float g = row_value(2 * t), u = row_value(2 * t + 1);
      float o = silu_f(g) * u;
      if (MODE == 1 && a.slot_scale != nullptr) o *= a.slot_scale[blockIdx.y];
      const int oi = (r0 >> 1) + t + (MODE == 1 ? (int)blockIdx.y * (a.N >> 1) : 0);
      if (a.y_dtype == B200_F32) reinterpret_cast<float*>(a.y)[oi] = o;
      else reinterpret_cast<__nv_bfloat16*>(a.y)[oi] = __float2bfloat16(o);
    }
  } else {
    for (int t = tid; t < nrows; t += kGemvThreads) {
      float v = row_value(t);
      if (a.epilogue == B200_EPI_GELU) v = gelu_erf(v);
      const int oi = r0 + t + (MODE == 1 ? (int)blockIdx.y * a.N : 0);
      if (a.resid != nullptr) {
        v += (a.resid_dtype == B200_F32)
                 ? reinterpret_cast<const float*>(a.resid)[oi]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.resid)[oi]);
      }
      if (TP && a.tp_out >= 0) {
        // partial row (+ residual on the lead rank) into slot `rank` of every rank's inbox
        tp_publish(a.tp, (unsigned)(a.tp.seq_base[0] + a.tp_out), oi, v);
      } else if (a.y_dtype == B200_F32) reinterpret_cast<float*>(a.y)[oi] = v;
      else reinterpret_cast<__nv_bfloat16*>(a.y)[oi] = __float2bfloat16(v);
    }
  }
}

template <int U, int MINB, int MODE = 0, bool TP = false>
static cudaError_t gemv_launch(GemvArgs a, bool swiglu, cudaStream_t st, bool pdl, int n_slots = 1) {
  // MINB CTAs per SM (shared between the routing slots in MODE 1); grow the grid in whole
  // waves until the per-CTA row block is small
  const int wave = (MINB * kNumSMs + n_slots - 1) / n_slots;
  int grid = wave;
  int rpc = (a.N + grid - 1) / grid;
  while (rpc > 1024) { grid += wave; rpc = (a.N + grid - 1) / grid; }
  if (swiglu && (rpc & 1)) ++rpc;
  grid = (a.N + rpc - 1) / rpc;
  a.rpc = rpc;
  const size_t smem = (size_t)a.K * 4 + (size_t)rpc * kGemvWarps * 4 + 128;
  static bool attr_set[kMaxDevices] = {false};
  const cudaError_t ea = opt_in_smem(gemv_kernel<U, MINB, MODE, TP>, 200 * 1024, attr_set);
  if (ea != cudaSuccess) return ea;
  return launch(gemv_kernel<U, MINB, MODE, TP>, dim3(grid, n_slots), dim3(kGemvThreads), smem, st, pdl, a);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gemv_bf16(const void* x, int x_dtype, const void* w, void* y, int y_dtype,
                              int K, int N, int ldw, const void* norm_w, const void* norm_beta,
                              float eps,
                              const void* bias, const void* resid, int resid_dtype,
                              int epilogue, int flags, b200_stream_t stream) {
  if (norm_beta != nullptr && norm_w == nullptr) return B200_ERR_ARG;
  if (!x || !w || !y) return B200_ERR_ARG;
  if (K <= 0 || N <= 0 || (K & 255) != 0 || ldw < K) return B200_ERR_SHAPE;
  if ((ldw & 7) != 0 || ((uintptr_t)w & 15) != 0 || ((uintptr_t)x & 15) != 0) return B200_ERR_ALIGN;
  if (epilogue == B200_EPI_SWIGLU && ((N & 1) != 0 || resid != nullptr)) return B200_ERR_SHAPE;
  if (epilogue < B200_EPI_NONE || epilogue > B200_EPI_GELU) return B200_ERR_ARG;
  if (K > 32768) return B200_ERR_SHAPE;

  GemvArgs a{};
  a.norm_in_smem = g_tuning[B200_TUNE_GEMV_NORM] == 1;
  a.x = x; a.w = (const uint16_t*)w; a.y = y;
  a.norm_w = (const uint16_t*)norm_w; a.norm_b = (const uint16_t*)norm_beta;
  a.bias = (const uint16_t*)bias; a.resid = resid;
  a.K = K; a.N = N; a.ldw = ldw; a.rpc = 0;
  a.x_dtype = x_dtype; a.y_dtype = y_dtype; a.resid_dtype = resid_dtype; a.epilogue = epilogue;
  a.eps = eps;
  a.expert_ids = nullptr; a.slot_scale = nullptr; a.expert_stride = 0; a.segs_per_expert = 0;
  a.expert_lo = 0; a.n_local = 0;
  a.tp_in = -1; a.tp_out = -1; a.x_out = nullptr; a.status = nullptr;
  const bool sw = epilogue == B200_EPI_SWIGLU;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  switch (g_tuning[B200_TUNE_GEMV]) {
    case 1: e = gemv_launch<4, 4>(a, sw, st, pdl); break;
    case 2: e = gemv_launch<4, 3>(a, sw, st, pdl); break;
    default: e = gemv_launch<8, 2>(a, sw, st, pdl); break;
  }
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

/* Decode-time expert MLP, first half: for each of the top_k routing slots
 *   act[slot, j] = wt[slot] * silu(g_j) * u_j,   (g, u) = rows (2j, 2j+1) of w_gu[ids[slot]] . xn
 * with xn = x or rmsnorm(x) * norm_w. */
extern "C" int b200_moe_decode_gate_up(void* act, const void* x, int x_dtype, const void* norm_w,
                                       float eps, const void* w_gu, const int* ids,
                                       const float* wts, int top_k, int inter, int hidden,
                                       int expert_lo, int n_local, int flags,
                                       b200_stream_t stream) {
  if (!act || !x || !w_gu || !ids) return B200_ERR_ARG;
  if (top_k <= 0 || inter <= 0 || hidden <= 0 || (hidden & 255) != 0 || hidden > 32768)
    return B200_ERR_SHAPE;
  if (((uintptr_t)w_gu & 15) != 0 || ((uintptr_t)x & 15) != 0) return B200_ERR_ALIGN;
  GemvArgs a{};
  a.norm_in_smem = g_tuning[B200_TUNE_GEMV_NORM] == 1;
  a.x = x; a.w = (const uint16_t*)w_gu; a.y = act; a.norm_w = (const uint16_t*)norm_w;
  a.bias = nullptr; a.resid = nullptr;
  a.K = hidden; a.N = 2 * inter; a.ldw = hidden; a.rpc = 0;
  a.x_dtype = x_dtype; a.y_dtype = B200_F32; a.resid_dtype = 0; a.epilogue = B200_EPI_SWIGLU;
  a.eps = eps;
  a.expert_ids = ids; a.slot_scale = wts; a.expert_stride = (long)2 * inter * hidden;
  a.segs_per_expert = 0; a.expert_lo = expert_lo; a.n_local = n_local;
  a.tp_in = -1; a.tp_out = -1; a.x_out = nullptr; a.status = nullptr;
  cudaError_t e = gemv_launch<8, 2, 1>(a, true, (cudaStream_t)stream,
                                       (flags & B200_FLAG_PDL) != 0, top_k);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

/* Decode-time expert MLP, second half: y[d] = (resid[d] +) sum_slot w_down[ids[slot]][d, :] . act[slot, :]. */
static int moe_down_impl(const b200::TpLink* link, int tp_out, int* status,
                         void* y, int y_dtype, const void* act, const void* w_down,
                                    const int* ids, int top_k, int inter, int hidden,
                                    int expert_lo, int n_local,
                                    const void* resid, int resid_dtype, int flags,
                                    b200_stream_t stream) {
  if ((!y && link == nullptr) || !act || !w_down || !ids) return B200_ERR_ARG;
  if (top_k <= 0 || inter <= 0 || hidden <= 0 || (inter & 255) != 0) return B200_ERR_SHAPE;
  const int segs = inter >> 8;
  if (top_k * segs > kMaxExpertSegs || (long)top_k * inter > 32768) return B200_ERR_SHAPE;
  if (((uintptr_t)w_down & 15) != 0 || ((uintptr_t)act & 15) != 0) return B200_ERR_ALIGN;
  GemvArgs a{};
  a.norm_in_smem = g_tuning[B200_TUNE_GEMV_NORM] == 1;
  a.x = act; a.w = (const uint16_t*)w_down; a.y = y; a.norm_w = nullptr; a.bias = nullptr;
  a.resid = resid;
  a.K = top_k * inter; a.N = hidden; a.ldw = inter; a.rpc = 0;
  a.x_dtype = B200_F32; a.y_dtype = y_dtype; a.resid_dtype = resid_dtype; a.epilogue = B200_EPI_NONE;
  a.eps = 0.f;
  a.expert_ids = ids; a.slot_scale = nullptr; a.expert_stride = (long)hidden * inter;
  a.segs_per_expert = segs; a.expert_lo = expert_lo; a.n_local = n_local;
  a.tp_in = -1; a.tp_out = -1; a.x_out = nullptr; a.status = nullptr;
  cudaError_t e;
  if (link != nullptr) {
    if (hidden != link->H) return B200_ERR_SHAPE;
    a.tp = *link; a.tp_out = tp_out; a.status = status;
    a.tp.wait_ticks = wait_ticks_from_tuning();
    e = gemv_launch<8, 2, 2, true>(a, false, (cudaStream_t)stream, (flags & B200_FLAG_PDL) != 0);
  } else {
    e = gemv_launch<8, 2, 2>(a, false, (cudaStream_t)stream, (flags & B200_FLAG_PDL) != 0);
  }
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

extern "C" int b200_moe_decode_down(void* y, int y_dtype, const void* act, const void* w_down,
                                    const int* ids, int top_k, int inter, int hidden,
                                    int expert_lo, int n_local,
                                    const void* resid, int resid_dtype, int flags,
                                    b200_stream_t stream) {
  return moe_down_impl(nullptr, -1, nullptr, y, y_dtype, act, w_down, ids, top_k, inter, hidden,
                       expert_lo, n_local, resid, resid_dtype, flags, stream);
}

// ---------------------------------------------------------------------------------------------
// Tensor-parallel link: peer-mapped inboxes set up once per process.
namespace {
struct TpContext { b200::TpLink link; void* local; bool used; };
constexpr int kTpMaxContexts = 16;   // links per process (an engine holds one for its lifetime)
TpContext g_tp[kTpMaxContexts];
constexpr size_t kTpAlign = 256;   // the buffer starts with one aligned block of scalars (seq_base)
}  // namespace

/* Bytes of the per-rank communication buffer: [scalars | inbox pairs | reduced-vector pairs]. */
extern "C" int64_t b200_tp_buffer_bytes(int world, int H) {
  if (world <= 0 || world > kTpMaxRanks || H <= 0) return 0;
  return (int64_t)(kTpAlign + (size_t)2 * world * H * 8 + (size_t)2 * H * 8);
}

/* cudaMalloc + zero the communication buffer (set-up time only) and return its IPC handle. */
extern "C" int b200_tp_alloc(void** ptr, void* ipc_handle_64, int64_t bytes) {
  if (!ptr || !ipc_handle_64 || bytes <= 0) return B200_ERR_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return B200_ERR_LAUNCH;
  if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess) return B200_ERR_LAUNCH;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return B200_ERR_LAUNCH;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(ipc_handle_64, &h, 64);
  *ptr = p;
  return cudaDeviceSynchronize() == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

/* Map a peer's buffer from its IPC handle. */
extern "C" int b200_tp_open(void** ptr, const void* ipc_handle_64) {
  if (!ptr || !ipc_handle_64) return B200_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess
             ? B200_OK : B200_ERR_LAUNCH;
}

/* Register the link: bufs[p] is rank p's buffer as mapped in THIS process (bufs[rank] = own). */
extern "C" int b200_tp_create(void* const* bufs, int world, int rank, int H) {
  if (!bufs || world <= 0 || world > kTpMaxRanks || rank < 0 || rank >= world || H <= 0 || (H & 3))
    return B200_ERR_ARG;
  int id = -1;
  for (int i = 0; i < kTpMaxContexts; ++i) if (!g_tp[i].used) { id = i; break; }
  if (id < 0) return B200_ERR_ARG;
  TpLink& l = g_tp[id].link;
  for (int p = 0; p < world; ++p) {
    if (!bufs[p]) return B200_ERR_ARG;
    l.inbox[p] = (float*)((char*)bufs[p] + kTpAlign);
  }
  l.seq_base = (const int*)((char*)bufs[rank] + 64);
  l.world = world; l.rank = rank; l.H = H;
  l.xr = (uint4*)((char*)l.inbox[rank] + (size_t)2 * world * H * 8);
  l.wait_ticks = kDefaultWaitTicks;
  g_tp[id].local = bufs[rank];
  g_tp[id].used = true;
  return id;
}

namespace b200 {
const TpLink* tp_link_get(int ctx) {
  return (ctx >= 0 && ctx < kTpMaxContexts && g_tp[ctx].used) ? &g_tp[ctx].link : nullptr;
}
}  // namespace b200

__global__ void tp_advance_kernel(int* seq_base, int inc) {
  b200::pdl_launch_dependents();
  b200::pdl_wait();
  if (threadIdx.x == 0) seq_base[0] += inc;
}

/* seq_base += inc (number of fused all-reduces issued since the last advance): once per step. */
extern "C" int b200_tp_advance(int ctx, int inc, int flags, b200_stream_t stream) {
  if (ctx < 0 || ctx >= kTpMaxContexts || !g_tp[ctx].used) return B200_ERR_ARG;
  cudaError_t e = launch(tp_advance_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream,
                         (flags & B200_FLAG_PDL) != 0, (int*)g_tp[ctx].link.seq_base, inc);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

/* b200_gemv_bf16 with the all-reduce fused in (fp32 activations, dense weights):
 *   tp_in  >= 0 : x is ignored; x = sum over ranks of the inbox of all-reduce (seq_base + tp_in),
 *                 K must equal the link's H; x_out (nullable) receives the reduced vector
 *   tp_out >= 0 : y is ignored; y (+ bias + resid) is pushed to every rank as this rank's share of
 *                 all-reduce (seq_base + tp_out); N must equal the link's H */
extern "C" int b200_gemv_bf16_tp(const void* x, const void* w, void* y, int K, int N, int ldw,
                                 const void* norm_w, float eps, const void* bias,
                                 const void* resid, int epilogue, int ctx, int tp_in, int tp_out,
                                 void* x_out, int* status, int flags, b200_stream_t stream) {
  if (ctx < 0 || ctx >= kTpMaxContexts || !g_tp[ctx].used) return B200_ERR_ARG;
  if (!w || (tp_in < 0 && !x) || (tp_out < 0 && !y)) return B200_ERR_ARG;
  if (K <= 0 || N <= 0 || (K & 255) != 0 || ldw < K || K > 32768) return B200_ERR_SHAPE;
  if ((ldw & 7) != 0 || ((uintptr_t)w & 15) != 0) return B200_ERR_ALIGN;
  const TpLink& l = g_tp[ctx].link;
  if ((tp_in >= 0 && K != l.H) || (tp_out >= 0 && (N != l.H || epilogue != B200_EPI_NONE)))
    return B200_ERR_SHAPE;
  if (epilogue == B200_EPI_SWIGLU && ((N & 1) != 0 || resid != nullptr)) return B200_ERR_SHAPE;
  GemvArgs a{};
  a.norm_in_smem = g_tuning[B200_TUNE_GEMV_NORM] == 1;
  a.x = x; a.w = (const uint16_t*)w; a.y = y;
  a.norm_w = (const uint16_t*)norm_w; a.bias = (const uint16_t*)bias; a.resid = resid;
  a.K = K; a.N = N; a.ldw = ldw; a.rpc = 0;
  a.x_dtype = B200_F32; a.y_dtype = B200_F32; a.resid_dtype = B200_F32; a.epilogue = epilogue;
  a.eps = eps;
  a.expert_ids = nullptr; a.slot_scale = nullptr; a.expert_stride = 0; a.segs_per_expert = 0;
  a.expert_lo = 0; a.n_local = 0;
  a.tp = l; a.tp_in = tp_in; a.tp_out = tp_out;
  a.x_out = (float*)x_out; a.status = status;
  a.tp.wait_ticks = wait_ticks_from_tuning();
  cudaError_t e = gemv_launch<8, 2, 0, true>(a, epilogue == B200_EPI_SWIGLU, (cudaStream_t)stream,
                                    (flags & B200_FLAG_PDL) != 0);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

/* b200_moe_decode_down under expert parallelism with the all-reduce fused in: this rank's experts'
 * share of the layer output (+ fp32 resid on one rank) is pushed to every rank as all-reduce
 * (seq_base + tp_out); the next b200_gemv_bf16_tp with the same tp_in reduces it. */
extern "C" int b200_moe_decode_down_tp(const void* act, const void* w_down, const int* ids,
                                       int top_k, int inter, int hidden, int expert_lo,
                                       int n_local, const void* resid, int ctx, int tp_out,
                                       int* status, int flags, b200_stream_t stream) {
  if (ctx < 0 || ctx >= kTpMaxContexts || !g_tp[ctx].used || tp_out < 0) return B200_ERR_ARG;
  return moe_down_impl(&g_tp[ctx].link, tp_out, status, nullptr, B200_F32, act, w_down, ids, top_k,
                       inter, hidden, expert_lo, n_local, resid, B200_F32, flags, stream);
}
