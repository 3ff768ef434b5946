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

namespace b200 {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

// ---------------------------------------------------------------------------------------------
// All-reduce fused into the GEMVs of a tensor-parallel decode step (one process per GPU, peer
// memory over NVLink, no collective library call):
//   * a row-parallel GEMV (o_proj, down_proj, the expert down projection) does not write y.
//     Each finished row of its partial sum goes into slot `rank` of EVERY rank's inbox as an
//     8-byte {fp32 value, sequence tag} pair with one 8-byte peer store: the pair arrives
//     atomically, so the data validates itself and no fence, flag or counter is needed;
//   * the NEXT GEMV on each rank consumes it while it stages its input vector anyway: a few
//     reducer CTAs poll (bounded) the ranks' pairs of their slice, add them in rank order and
//     publish the sum locally as tagged pairs again; all CTAs poll that one vector.  Every rank
//     adds the same values in the same order, so all ranks stay bit-identical.
// Two inbox slots alternate by sequence parity: a rank can be at most one all-reduce ahead of
// its slowest peer, because the next one needs that peer's contribution.
// Two measured alternatives stay selectable (B200_TUNE_TP_PROTOCOL): every CTA summing the inboxes
// itself (world x 32 KB of L2 reads per CTA), and plain stores followed by a system fence and one
// release flag per rank (slower than a collective library: the fence waits out the NVLink round
// trip).
constexpr int kTpMaxRanks = 8;
constexpr int kTpReducers = 8;     // CTAs that sum the ranks' contributions (hierarchical mode)
constexpr long long kTpWaitTicks = 4000000000LL;   // ~2 s: every wait on a peer is bounded
struct TpLink {
  float* inbox[kTpMaxRanks];        // inbox of rank p (peer-mapped): [2 slots][world][H] fp32, or
                                    // [2 slots][world][H] {fp32 value, u32 tag} pairs (ll)
  unsigned* flags[kTpMaxRanks];     // flags of rank p: [2 slots][world] published sequence numbers
  int* local_counter;               // CTA arrival counter of the publishing kernel (this rank)
  const int* seq_base;              // device scalar: sequence number of the step's first all-reduce
  int world, rank, H;
  int ll;                           // 1: tagged-pair protocol, 0: data + sequence flags
  int hier;                         // tagged pairs: a few CTAs reduce, the others read their sums
  uint4* xr;                        // local staging of the reduced vector: [2 slots][H] pairs
};

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

// B200_TUNE_TP_PROTOCOL: 0 default (tagged pairs summed by a few reducer CTAs), 1 data + flags,
// 2 tagged pairs read directly by every CTA, 3 tagged pairs through the reducer CTAs
static void tp_apply_tuning(TpLink& l) {
  const int t = g_tuning[B200_TUNE_TP_PROTOCOL];
  if (t == 1) l.ll = 0;
  else if (t == 2) l.hier = 0;
  else if (t == 3) l.hier = 1;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Sum over n tagged-pair vectors (stride in uint4) of the float4 at q0: every 8-byte
// {value, tag} pair arrives atomically, so the data itself is polled (bounded) - no flag, no fence.
__device__ __forceinline__ float4 ll_reduce(const uint4* q0, int n, int stride, unsigned tag,
                                            int* status) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  long long t0 = 0;
  for (int r = 0; r < n; ++r) {
    const uint4* q = q0 + (size_t)r * stride;
    uint4 e0, e1;
    int spins = 0;
    while (true) {
      e0 = ld_volatile_v4(q);
      e1 = ld_volatile_v4(q + 1);
      if (e0.y == tag && e0.w == tag && e1.y == tag && e1.w == tag) break;
      if ((++spins & 63) == 0) {
        // an earlier wait already gave up: do not spend the budget again
        if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) break;
        if (t0 == 0) t0 = clock64();
        if (clock64() - t0 > kTpWaitTicks) {
          if (status != nullptr) atomicExch(status, B200_ERR_TIMEOUT);
          break;
        }
      }
    }
    v.x += __uint_as_float(e0.x); v.y += __uint_as_float(e0.z);
    v.z += __uint_as_float(e1.x); v.w += __uint_as_float(e1.z);
  }
  return v;
}
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_volatile_v2(uint2* p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

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
    // wait for every rank's contribution to all-reduce number seq (bounded, like every wait)
    const unsigned seq = (unsigned)(a.tp.seq_base[0] + a.tp_in);
    tp_slot = seq & 1u;
    tp_tag = seq + 1u;
    if (!a.tp.ll) {
      if (tid < a.tp.world) {
        const volatile unsigned* f = a.tp.flags[a.tp.rank] + tp_slot * a.tp.world + tid;
        const long long t0 = clock64();
        int spins = 0;
        while (*f != seq + 1u) {
          if ((++spins & 63) == 0) {
            // an earlier wait already gave up: do not spend the budget again
            if (a.status != nullptr && *reinterpret_cast<volatile int*>(a.status) != 0) break;
            if (clock64() - t0 > kTpWaitTicks) {
              if (a.status != nullptr) atomicExch(a.status, B200_ERR_TIMEOUT);
              break;
            }
          }
        }
        __threadfence_system();
      }
      __syncthreads();
    }
  }
  if (TP && a.tp_in >= 0 && a.tp.ll && a.tp.hier) {
    // A few CTAs sum the ranks' contributions, one slice each, and publish the sums locally as
    // tagged pairs; every CTA then polls that one vector.  The inbox is read once per GPU instead
    // of once per CTA (which costs world x 32 KB of L2 traffic per CTA).
    const int nred = min(kTpReducers, (int)gridDim.x);
    if ((int)blockIdx.x < nred) {
      const int n4 = K >> 2, per = (n4 + nred - 1) / nred;
      const int lo = blockIdx.x * per, hi = min(n4, lo + per);
      const uint4* box = reinterpret_cast<const uint4*>(a.tp.inbox[a.tp.rank]) +
                         (size_t)tp_slot * a.tp.world * (K >> 1);
      uint4* dst = a.tp.xr + (size_t)tp_slot * (K >> 1);
      for (int i = lo + tid; i < hi; i += kGemvThreads) {
        const float4 v = ll_reduce(box + 2 * i, a.tp.world, K >> 1, tp_tag, a.status);
        st_volatile_v4(dst + 2 * i, make_uint4(__float_as_uint(v.x), tp_tag, __float_as_uint(v.y), tp_tag));
        st_volatile_v4(dst + 2 * i + 1, make_uint4(__float_as_uint(v.z), tp_tag, __float_as_uint(v.w), tp_tag));
        if (a.x_out != nullptr) reinterpret_cast<float4*>(a.x_out)[i] = v;
      }
    }
  }
  for (int i = tid; i < (K >> 2); i += kGemvThreads) {
    float4 v;
    if (TP && a.tp_in >= 0) {
      if (a.tp.ll) {
        const uint4* src = a.tp.hier
            ? a.tp.xr + (size_t)tp_slot * (K >> 1) + 2 * i
            : reinterpret_cast<const uint4*>(a.tp.inbox[a.tp.rank]) +
                  (size_t)tp_slot * a.tp.world * (K >> 1) + 2 * i;
        v = ll_reduce(src, a.tp.hier ? 1 : a.tp.world, K >> 1, tp_tag, a.status);
      } else {
        const float4* box = reinterpret_cast<const float4*>(a.tp.inbox[a.tp.rank]) +
                            (size_t)tp_slot * a.tp.world * (K >> 2) + i;
        v = __ldcg(box);                                     // peers wrote this: bypass L1
        for (int r = 1; r < a.tp.world; ++r) {
          const float4 o = __ldcg(box + (size_t)r * (K >> 2));
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
      }
      if (a.x_out != nullptr && blockIdx.x == 0 && !(a.tp.ll && a.tp.hier))
        reinterpret_cast<float4*>(a.x_out)[i] = v;
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
        const unsigned seq = (unsigned)(a.tp.seq_base[0] + a.tp_out);
        const size_t off = ((size_t)(seq & 1u) * a.tp.world + a.tp.rank) * a.tp.H + oi;
        if (a.tp.ll) {
          for (int p = 0; p < a.tp.world; ++p)
            st_volatile_v2(reinterpret_cast<uint2*>(a.tp.inbox[p]) + off,
                           make_uint2(__float_as_uint(v), seq + 1u));
        } else {
          for (int p = 0; p < a.tp.world; ++p) a.tp.inbox[p][off] = v;
        }
      } else if (a.y_dtype == B200_F32) reinterpret_cast<float*>(a.y)[oi] = v;
      else reinterpret_cast<__nv_bfloat16*>(a.y)[oi] = __float2bfloat16(v);
    }
  }
  if (TP && a.tp_out >= 0 && !a.tp.ll) {
    // The CTA that arrives last knows every partial row of this rank has been stored.  One
    // system fence per CTA, by the thread that signals: the barrier orders the other threads'
    // stores before it, and the fence is cumulative.  (A fence in every warp serialises per SM
    // on the NVLink round trip.)
    __syncthreads();
    if (tid == 0) {
      __threadfence_system();
      const int old = atomicAdd(a.tp.local_counter, 1);
      if (old == (int)gridDim.x - 1) {
        *a.tp.local_counter = 0;
        __threadfence_system();
        const unsigned seq = (unsigned)(a.tp.seq_base[0] + a.tp_out);
        for (int p = 0; p < a.tp.world; ++p) {
          unsigned* f = a.tp.flags[p] + (seq & 1u) * a.tp.world + a.tp.rank;
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(seq + 1u) : "memory");
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core variant of the dense GEMV (B200_TUNE_GEMV = 3; EXPERIMENTAL: its data mapping is
// checked against an emulation of the mma fragment layout, it has not been timed yet and is not
// the default).  The SIMT loop above spends 64 instructions per 512 bytes of weights (unpack,
// dependent FMAs, bookkeeping); here a warp multiplies 16 rows x 64 columns of W per step with
// four 16-byte loads per lane and four mma.sync.m16n8k16:
//   * A = W: lane (g, tq) loads 32 contiguous bytes of row g and of row g + 8 (a quad covers one
//     128-byte line per row).  The dot product does not care in which order k is visited, so the
//     16 values of a lane are used as they lie: MMA m takes elements 4m .. 4m+3 of both rows;
//   * B = x: column 0 carries the bf16 high part of x, column 1 the low part (x = hi + lo keeps
//     ~16 mantissa bits), the other six columns are zero; lane (n, tq) reads the 16 matching
//     values of column n from shared memory with two 16-byte loads;
//   * D: column 0 + column 1 of row g / g + 8 meet in lane tq = 0 - no shuffle, no unpack.
// The eight warps of a CTA split K, every warp walks all 16-row groups of the CTA over its K
// slice, and the per-warp partial sums are added in warp order exactly as in the SIMT kernel.
__device__ __forceinline__ void gemv_mma_step(float* c, const uint4& a0, const uint4& a1,
                                              const uint4& b0, const uint4& b1, const uint4& x0,
                                              const uint4& x1) {
  // a0 / a1: elements 0..7 / 8..15 of row g; b0 / b1: the same of row g + 8; x0 / x1: the lane's
  // 16 values of its B column
#define B200_GEMV_MMA(A0, A1, A2, A3, B0, B1)                                                   \
  asm volatile(                                                                                 \
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "      \
      "{%8,%9}, {%0,%1,%2,%3};"                                                                  \
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])                                          \
      : "r"(A0), "r"(A1), "r"(A2), "r"(A3), "r"(B0), "r"(B1))
  B200_GEMV_MMA(a0.x, b0.x, a0.y, b0.y, x0.x, x0.y);
  B200_GEMV_MMA(a0.z, b0.z, a0.w, b0.w, x0.z, x0.w);
  B200_GEMV_MMA(a1.x, b1.x, a1.y, b1.y, x1.x, x1.y);
  B200_GEMV_MMA(a1.z, b1.z, a1.w, b1.w, x1.z, x1.w);
#undef B200_GEMV_MMA
}

template <int MINB>
__global__ void __launch_bounds__(kGemvThreads, MINB) gemv_mma_kernel(GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int K = a.K;
  uint32_t* xh = reinterpret_cast<uint32_t*>(smem_raw);      // K/2 packed bf16 pairs: high parts
  uint32_t* xl = xh + (K >> 1);                               // K/2 pairs: low parts
  const int rpc16 = (a.rpc + 15) & ~15;
  float* part = reinterpret_cast<float*>(xl + (K >> 1));      // [rpc16][kGemvWarps]
  float* red = part + rpc16 * kGemvWarps;                     // 32

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int r0 = blockIdx.x * a.rpc;
  const int nrows = min(a.N - r0, a.rpc);
  pdl_launch_dependents();
  if (nrows <= 0) return;

  // this warp's K slice in units of 64 columns (128 bytes per row)
  const int units = K >> 6;
  const int u0 = units * warp / kGemvWarps, u1 = units * (warp + 1) / kGemvWarps;
  const int nu = u1 - u0;
  const int ngroups = (nrows + 15) >> 4;
  const int total = ngroups * nu;                             // steps of this warp
  const unsigned char* wbase = reinterpret_cast<const unsigned char*>(a.w);
  const size_t row_bytes = (size_t)a.ldw * 2;
  auto load_step = [&](uint4* d, int s) {                     // d[0..1] row g, d[2..3] row g + 8
    const int grp = s / nu, u = u0 + (s - grp * nu);
    const int ra = min(grp * 16 + g, nrows - 1), rb = min(grp * 16 + g + 8, nrows - 1);
    const unsigned char* pa = wbase + (size_t)(r0 + ra) * row_bytes + (size_t)u * 128 + tq * 32;
    const unsigned char* pb = wbase + (size_t)(r0 + rb) * row_bytes + (size_t)u * 128 + tq * 32;
    d[0] = ldg_stream(pa); d[1] = ldg_stream(pa + 16);
    d[2] = ldg_stream(pb); d[3] = ldg_stream(pb + 16);
  };
  // weights do not depend on the previous kernel: two steps are in flight before the wait
  uint4 w0[4], w1[4], w2[4];
  if (0 < total) load_step(w0, 0);
  if (1 < total) load_step(w1, 1);

  pdl_wait();

  // stage x (* norm weight) as bf16 high / low pairs; the RMSNorm scalar multiplies the row sums
  float ss = 0.f;
  for (int i = tid; i < (K >> 2); i += kGemvThreads) {
    float4 v;
    if (a.x_dtype == B200_F32) {
      v = reinterpret_cast<const float4*>(a.x)[i];
    } else {
      const uint2 u = reinterpret_cast<const uint2*>(a.x)[i];
      v = make_float4(bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y));
    }
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (a.norm_w != nullptr) {
      const uint2 u = reinterpret_cast<const uint2*>(a.norm_w)[i];
      v.x *= bf16lo(u.x); v.y *= bf16hi(u.x); v.z *= bf16lo(u.y); v.w *= bf16hi(u.y);
    }
    const __nv_bfloat16 h0 = __float2bfloat16(v.x), h1 = __float2bfloat16(v.y);
    const __nv_bfloat16 h2 = __float2bfloat16(v.z), h3 = __float2bfloat16(v.w);
    uint2 hi, lo;
    hi.x = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
    hi.y = (uint32_t)__bfloat16_as_ushort(h2) | ((uint32_t)__bfloat16_as_ushort(h3) << 16);
    lo.x = pack_bf16(v.x - __bfloat162float(h0), v.y - __bfloat162float(h1));
    lo.y = pack_bf16(v.z - __bfloat162float(h2), v.w - __bfloat162float(h3));
    reinterpret_cast<uint2*>(xh)[i] = hi;
    reinterpret_cast<uint2*>(xl)[i] = lo;
  }
  for (int i = tid; i < rpc16 * kGemvWarps; i += kGemvThreads) part[i] = 0.f;
  const float tot = block_sum(ss, red);                       // its barriers also publish xh / xl
  const float out_scale = a.norm_w != nullptr ? rsqrtf(tot / (float)K + a.eps) : 1.f;
  __syncthreads();

  const uint32_t* xsel = g == 0 ? xh : xl;                    // B column of this lane (g < 2)
  float c[4] = {0.f, 0.f, 0.f, 0.f};
  auto compute = [&](const uint4* d, int s) {
    const int grp = s / nu, u = u0 + (s - grp * nu);
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
    if (g < 2) {
      const uint4* xp = reinterpret_cast<const uint4*>(xsel + ((u * 64 + tq * 16) >> 1));
      x0 = xp[0]; x1 = xp[1];
    }
    gemv_mma_step(c, d[0], d[1], d[2], d[3], x0, x1);
    if (s - grp * nu == nu - 1) {                             // last step of this group: park the sums
      if (tq == 0) {
        part[(grp * 16 + g) * kGemvWarps + warp] = c[0] + c[1];
        part[(grp * 16 + g + 8) * kGemvWarps + warp] = c[2] + c[3];
      }
      c[0] = c[1] = c[2] = c[3] = 0.f;
    }
  };
  for (int s = 0; s < total; s += 3) {                        // three register buffers in rotation
    if (s + 2 < total) load_step(w2, s + 2);
    compute(w0, s);
    if (s + 1 < total) {
      if (s + 3 < total) load_step(w0, s + 3);
      compute(w1, s + 1);
    }
    if (s + 2 < total) {
      if (s + 4 < total) load_step(w1, s + 4);
      compute(w2, s + 2);
    }
  }
  __syncthreads();

  // ---- epilogue: fixed-order row sums (as in the SIMT kernel) ----
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
      const float gv = row_value(2 * t), uv = row_value(2 * t + 1);
      const float o = silu_f(gv) * uv;
      const int oi = (r0 >> 1) + t;
      if (a.y_dtype == B200_F32) reinterpret_cast<float*>(a.y)[oi] = o;
      else reinterpret_cast<__nv_bfloat16*>(a.y)[oi] = __float2bfloat16(o);
    }
  } else {
    for (int t = tid; t < nrows; t += kGemvThreads) {
      float v = row_value(t);
      if (a.epilogue == B200_EPI_GELU) v = gelu_erf(v);
      const int oi = r0 + t;
      if (a.resid != nullptr) {
        v += (a.resid_dtype == B200_F32)
                 ? reinterpret_cast<const float*>(a.resid)[oi]
                 : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.resid)[oi]);
      }
      if (a.y_dtype == B200_F32) reinterpret_cast<float*>(a.y)[oi] = v;
      else reinterpret_cast<__nv_bfloat16*>(a.y)[oi] = __float2bfloat16(v);
    }
  }
}

template <int MINB>
static cudaError_t gemv_mma_launch(GemvArgs a, bool swiglu, cudaStream_t st, bool pdl) {
  const int wave = MINB * kNumSMs;
  int grid = wave;
  int rpc = (a.N + grid - 1) / grid;
  while (rpc > 1024) { grid += wave; rpc = (a.N + grid - 1) / grid; }
  if (swiglu && (rpc & 1)) ++rpc;
  grid = (a.N + rpc - 1) / rpc;
  a.rpc = rpc;
  const size_t smem = (size_t)a.K * 4 + (size_t)((rpc + 15) & ~15) * kGemvWarps * 4 + 128;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemv_mma_kernel<MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    attr_set = true;
  }
  return launch(gemv_mma_kernel<MINB>, dim3(grid), dim3(kGemvThreads), smem, st, pdl, a);
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemv_kernel<U, MINB, MODE, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    attr_set = true;
  }
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
    case 3:   // experimental tensor-core loop; no LayerNorm prologue there
      e = norm_beta != nullptr ? gemv_launch<8, 2>(a, sw, st, pdl) : gemv_mma_launch<2>(a, sw, st, pdl);
      break;
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
    tp_apply_tuning(a.tp);
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
constexpr size_t kTpAlign = 256;
size_t tp_flag_bytes(int world) { return ((size_t)2 * world * 4 + kTpAlign - 1) & ~(kTpAlign - 1); }
}  // namespace

/* Bytes of the per-rank communication buffer: [flags | arrival counter + seq_base | inbox]. */
extern "C" int64_t b200_tp_buffer_bytes(int world, int H) {
  if (world <= 0 || world > kTpMaxRanks || H <= 0) return 0;
  return (int64_t)(tp_flag_bytes(world) + kTpAlign + (size_t)2 * world * H * 8 + (size_t)2 * H * 8);
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
    l.flags[p] = (unsigned*)bufs[p];
    l.inbox[p] = (float*)((char*)bufs[p] + tp_flag_bytes(world) + kTpAlign);
  }
  char* own = (char*)bufs[rank] + tp_flag_bytes(world);
  l.local_counter = (int*)own;
  l.seq_base = (const int*)(own + 64);
  l.world = world; l.rank = rank; l.H = H; l.ll = 1;
  l.hier = 1;
  l.xr = (uint4*)((char*)l.inbox[rank] + (size_t)2 * world * H * 8);
  g_tp[id].local = bufs[rank];
  g_tp[id].used = true;
  return id;
}

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
  tp_apply_tuning(a.tp);
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
