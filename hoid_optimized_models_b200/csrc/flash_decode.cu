// Split-KV GQA flash-decode with the log-sum-exp combine fused into the same launch.
//
// Grid (n_splits, n_kv), about one CTA per SM.  A CTA owns one kv head and one
// contiguous slice of the context and serves all G = n_q / n_kv query heads of the
// group from a single pass over K and V, so each cache byte is read from HBM once.
//
// A CTA of eight warps streams 128-key tiles of K and V through a three-stage cp.async ring;
// each warp owns 16 keys of a tile and runs S = Q K^T and O += P V on mma.sync m16n8k16 (about
// 20 instructions per KB of cache; a SIMT kernel with one shuffle reduction per key and head
// needed ~185 and was issue-bound near 4 TB/s).  The 16-row A operand carries the group's
// G <= 8 query heads twice: rows 0..7 hold the bf16 high part of q (and of P), rows 8..15 the
// bf16 low part, so q and P keep ~16 mantissa bits at no extra MMA and the two halves of an
// accumulator add up inside one thread.  The warps' records are merged through shared memory,
// the CTA publishes ONE record [acc(G x HD), m(G), l(G)] to the workspace, and the CTA that
// arrives last on the per-kv-head counter merges the n_splits records (a handful of coalesced
// float4 loads per thread) in fixed split order and writes the output.  No CTA ever waits on
// another.
#include "common.cuh"
#include "flash_decode_core.cuh"

namespace b200 {

template <int HD, int G, bool ROPE>
__global__ void __launch_bounds__(kFmThreads, 1) flash_decode_mma_kernel(FdArgs a) {
  constexpr int KS = HD / 16;          // k16 steps over the head dim
  constexpr int DB = HD / 8;           // n8 blocks over the head dim
  constexpr int CPR = HD / 8;          // 16-byte chunks per row
  constexpr int TILE = kFmTile * HD * 2;                 // bytes of one K (or V) tile
  constexpr int REC = G * HD + ((2 * G + 3) & ~3);
  extern __shared__ __align__(128) unsigned char fm_smem[];
  const uint32_t ring = smem_u32(fm_smem);               // [stages][K tile | V tile]
  float* srec = reinterpret_cast<float*>(fm_smem);       // re-uses the ring after the loop
  float* sw = reinterpret_cast<float*>(fm_smem + kFmStages * 2 * TILE);   // [WARPS][G]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;                // fragment row (= head) and column pair
  const int split = blockIdx.x, kvh = blockIdx.y;

  pdl_launch_dependents();

  int kv_len, k0, k1, ntiles;
  auto slice = [&](int kvl) {
    kv_len = kvl;
    const int per = (kvl + a.n_splits - 1) / a.n_splits;
    k0 = split * per;
    k1 = min(kvl, k0 + per);
    ntiles = k1 > k0 ? (k1 - k0 + kFmTile - 1) / kFmTile : 0;
  };
  const uint16_t* kb = a.k + (size_t)kvh * a.head_stride;
  const uint16_t* vb = a.v + (size_t)kvh * a.head_stride;
  auto load_tile = [&](int t) {
    const uint32_t sk = ring + (t % kFmStages) * 2 * TILE, sv = sk + TILE;
    const int row0 = k0 + t * kFmTile;
#pragma unroll
    for (int i = tid; i < kFmTile * CPR; i += kFmThreads) {
      const int r = i / CPR, c = i % CPR;
      int gr = row0 + r;
      gr = gr < k1 ? gr : k1 - 1;                        // rows past the slice are masked below
      const size_t off = (size_t)gr * a.row_stride + c * 8;
      fm_cp16(sk + fm_swz<HD>(r, c), kb + off);
      fm_cp16(sv + fm_swz<HD>(r, c), vb + off);
    }
  };
  auto first_tiles = [&]() {
    if (0 < ntiles) load_tile(0);
    fm_commit();
    if (1 < ntiles) load_tile(1);
    fm_commit();
  };
  const volatile int* kvl_p = a.kv_len;
  if (ROPE) {
    // Cache rows of earlier positions never change during a step, so the first tiles are
    // requested before the wait on the previous kernel, with the length as it reads now; the row
    // this launch appends is patched in shared memory anyway.  If the length turns out to have
    // been stale (possible only outside a replayed graph), the copies are simply issued again.
    slice(kvl_p[0]);
    first_tiles();
    pdl_wait();
    const int now = kvl_p[0];
    if (now != kv_len) {                                 // CTA-uniform
      fm_wait<0>();
      slice(now);
      first_tiles();
    }
  } else {
    pdl_wait();
    slice(kvl_p[0]);
    first_tiles();
  }

  // ---- q as A fragments: head g in rows g (high part) and g + 8 (low part) ----
  uint32_t qf[KS][4];
  int pos_own = -1;
  uint4 newk = make_uint4(0, 0, 0, 0), newv = make_uint4(0, 0, 0, 0);
  {
    float x[KS][4];                                      // dims ks*16 + tq*2 + {0, 1, 8, 9}
    const bool live = g < G;
    if (ROPE) {
      const int pos = kv_len - 1;
      const bool in_cache = pos >= 0 && pos < a.max_seq;
      const float* src = a.qkv + (size_t)(kvh * G + (live ? g : 0)) * HD;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const float2 u = *reinterpret_cast<const float2*>(src + ks * 16 + tq * 2);
        const float2 w = *reinterpret_cast<const float2*>(src + ks * 16 + tq * 2 + 8);
        x[ks][0] = u.x; x[ks][1] = u.y; x[ks][2] = w.x; x[ks][3] = w.y;
      }
      if (a.qn_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
          for (int e = 0; e < 4; ++e) ss = fmaf(x[ks][e], x[ks][e], ss);
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        const float inv = rsqrtf(ss / (float)HD + a.eps);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(a.qn_w + ks * 16 + tq * 2);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(a.qn_w + ks * 16 + tq * 2 + 8);
          x[ks][0] = x[ks][0] * inv * bf16lo(w0); x[ks][1] = x[ks][1] * inv * bf16hi(w0);
          x[ks][2] = x[ks][2] * inv * bf16lo(w1); x[ks][3] = x[ks][3] * inv * bf16hi(w1);
        }
      }
      // rotate-half: dim d < HD/2 pairs with d + HD/2, which the same thread holds in step ks + KS/2
      const size_t ci = (size_t)(in_cache ? pos : 0) * (HD / 2);
#pragma unroll
      for (int ks = 0; ks < KS / 2; ++ks) {
        const float2 c0 = *reinterpret_cast<const float2*>(a.cos_t + ci + ks * 16 + tq * 2);
        const float2 c1 = *reinterpret_cast<const float2*>(a.cos_t + ci + ks * 16 + tq * 2 + 8);
        const float2 s0 = *reinterpret_cast<const float2*>(a.sin_t + ci + ks * 16 + tq * 2);
        const float2 s1 = *reinterpret_cast<const float2*>(a.sin_t + ci + ks * 16 + tq * 2 + 8);
        const float cs[4] = {c0.x, c0.y, c1.x, c1.y}, sn[4] = {s0.x, s0.y, s1.x, s1.y};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = x[ks][e], hi = x[ks + KS / 2][e];
          x[ks][e] = lo * cs[e] - hi * sn[e];
          x[ks + KS / 2][e] = hi * cs[e] + lo * sn[e];
        }
      }
      // the new k / v row: (norm +) RoPE in the 8-dims-per-lane layout, by warp 0 of the CTA whose
      // slice ends with it
      if (in_cache && pos >= k0 && pos < k1) {
        pos_own = pos;
        if (warp == 0) {
          constexpr int LPK = HD / 8, HL = LPK / 2;
          const int dl = lane % LPK;
          const bool hi = dl >= HL;
          const float* ks_ = a.qkv + (size_t)(a.n_q + kvh) * HD + dl * 8;
          const float4 x0 = reinterpret_cast<const float4*>(ks_)[0];
          const float4 x1 = reinterpret_cast<const float4*>(ks_)[1];
          float kx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
          if (a.kn_w != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(kx[e], kx[e], ss);
#pragma unroll
            for (int o2 = LPK / 2; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
            const float inv = rsqrtf(ss / (float)HD + a.eps);
            float w[8];
            unpack8(*reinterpret_cast<const uint4*>(a.kn_w + dl * 8), w);
#pragma unroll
            for (int e = 0; e < 8; ++e) kx[e] = kx[e] * inv * w[e];
          }
          const float* cp = a.cos_t + ci + (size_t)(dl - (hi ? HL : 0)) * 8;
          const float* sp = a.sin_t + ci + (size_t)(dl - (hi ? HL : 0)) * 8;
          const float4 c0 = reinterpret_cast<const float4*>(cp)[0], c1 = reinterpret_cast<const float4*>(cp)[1];
          const float4 s0 = reinterpret_cast<const float4*>(sp)[0], s1 = reinterpret_cast<const float4*>(sp)[1];
          const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
          float kr[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, kx[e], HL);
            kr[e] = hi ? (kx[e] * cs[e] + other * sn[e]) : (kx[e] * cs[e] - other * sn[e]);
          }
          const float4* vp = reinterpret_cast<const float4*>(
              a.qkv + (size_t)(a.n_q + a.n_kv + kvh) * HD + dl * 8);
          const float4 v0 = vp[0], v1 = vp[1];
          newk.x = pack_bf16(kr[0], kr[1]); newk.y = pack_bf16(kr[2], kr[3]);
          newk.z = pack_bf16(kr[4], kr[5]); newk.w = pack_bf16(kr[6], kr[7]);
          newv.x = pack_bf16(v0.x, v0.y); newv.y = pack_bf16(v0.z, v0.w);
          newv.z = pack_bf16(v1.x, v1.y); newv.w = pack_bf16(v1.z, v1.w);
          if (lane < LPK) {
            const size_t row = (size_t)kvh * a.head_stride + (size_t)pos * a.row_stride + dl * 8;
            *reinterpret_cast<uint4*>(const_cast<uint16_t*>(a.k) + row) = newk;
            *reinterpret_cast<uint4*>(const_cast<uint16_t*>(a.v) + row) = newv;
          }
        }
      }
    } else {
      const size_t qi = (size_t)(kvh * G + (live ? g : 0)) * HD;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        if (a.q_dtype == B200_F32) {
          const float* src = reinterpret_cast<const float*>(a.q) + qi + ks * 16 + tq * 2;
          const float2 u = *reinterpret_cast<const float2*>(src);
          const float2 w = *reinterpret_cast<const float2*>(src + 8);
          x[ks][0] = u.x; x[ks][1] = u.y; x[ks][2] = w.x; x[ks][3] = w.y;
        } else {
          const uint16_t* src = reinterpret_cast<const uint16_t*>(a.q) + qi + ks * 16 + tq * 2;
          const uint32_t u = *reinterpret_cast<const uint32_t*>(src);
          const uint32_t w = *reinterpret_cast<const uint32_t*>(src + 8);
          x[ks][0] = bf16lo(u); x[ks][1] = bf16hi(u); x[ks][2] = bf16lo(w); x[ks][3] = bf16hi(w);
        }
      }
    }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const float sc = live ? a.scale_log2 : 0.f;        // padding rows carry zeros
      fm_split(x[ks][0] * sc, x[ks][1] * sc, qf[ks][0], qf[ks][1]);
      fm_split(x[ks][2] * sc, x[ks][3] * sc, qf[ks][2], qf[ks][3]);
    }
  }

  float o[DB][4];
#pragma unroll
  for (int d = 0; d < DB; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
  float m = -INFINITY, l = 0.f;

  for (int t = 0; t < ntiles; ++t) {
    fm_wait<1>();                    // tile t has landed (at most tile t + 1 still in flight)
    __syncthreads();                 // ... for every thread, and everyone is done with tile t - 1
    if (t + 2 < ntiles) load_tile(t + 2);
    fm_commit();
    const uint32_t sk = ring + (t % kFmStages) * 2 * TILE, sv = sk + TILE;
    const int row0 = k0 + t * kFmTile;
    if (ROPE && pos_own >= row0 && pos_own < row0 + kFmTile) {   // CTA-uniform
      // the cache row this launch appends must not be read back through the async copies
      if (warp == 0 && lane < HD / 8) {
        const uint32_t off = fm_swz<HD>(pos_own - row0, lane);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sk + off), "r"(newk.x),
                     "r"(newk.y), "r"(newk.z), "r"(newk.w) : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sv + off), "r"(newv.x),
                     "r"(newv.y), "r"(newv.z), "r"(newv.w) : "memory");
      }
      __syncthreads();
    }
    const int key0 = row0 + warp * 16;                   // this warp's 16 keys
    if (key0 >= k1) continue;                            // warp-uniform
    // ---- S = Q K^T : 16 rows x 16 keys ----
    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b0, b1, b2, b3;
      const int key = warp * 16 + ((lane >> 4) << 3) + (lane & 7);
      const int c = ks * 2 + ((lane >> 3) & 1);
      fm_ldsm(sk + fm_swz<HD>(key, c), b0, b1, b2, b3);
      fm_mma(s[0], qf[ks], b0, b1);
      fm_mma(s[1], qf[ks], b2, b3);
    }
    // high + low rows of the same head meet in one thread
    float sv4[4] = {s[0][0] + s[0][2], s[0][1] + s[0][3], s[1][0] + s[1][2], s[1][1] + s[1][3]};
    if (key0 + 16 > k1) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + (e >> 1) * 8 + tq * 2 + (e & 1);
        if (key >= k1) sv4[e] = -INFINITY;
      }
    }
    float mt = fmaxf(fmaxf(sv4[0], sv4[1]), fmaxf(sv4[2], sv4[3]));
    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
    mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
    const float mn = fmaxf(m, mt);
    const float mu = (mn == -INFINITY) ? 0.f : mn;
    const float corr = exp2f(m - mu);
    m = mn;
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) p[e] = exp2f(sv4[e] - mu);
    l = l * corr + (p[0] + p[1]) + (p[2] + p[3]);
    uint32_t pf[4];                  // P as the A fragment of one k16 step: rows g / g + 8 = hi / lo
    fm_split(p[0], p[1], pf[0], pf[1]);
    fm_split(p[2], p[3], pf[2], pf[3]);
#pragma unroll
    for (int d = 0; d < DB; ++d) { o[d][0] *= corr; o[d][1] *= corr; o[d][2] *= corr; o[d][3] *= corr; }
    // ---- O += P V ----
#pragma unroll
    for (int d2 = 0; d2 < DB / 2; ++d2) {
      uint32_t b0, b1, b2, b3;
      const int key = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
      const int c = d2 * 2 + (lane >> 4);
      fm_ldsm_t(sv + fm_swz<HD>(key, c), b0, b1, b2, b3);
      fm_mma(o[d2 * 2], pf, b0, b1);
      fm_mma(o[d2 * 2 + 1], pf, b2, b3);
    }
  }
  fm_wait<0>();
  __syncthreads();                   // the ring is free: it becomes the record area

  // ---- one record per warp ----
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (g < G) {
    float* r = srec + warp * REC;
#pragma unroll
    for (int d = 0; d < DB; ++d)
      *reinterpret_cast<float2*>(r + g * HD + d * 8 + tq * 2) =
          make_float2(o[d][0] + o[d][2], o[d][1] + o[d][3]);
    if (tq == 0) { r[G * HD + g] = m; r[G * HD + G + g] = l; }
  }
  fd_finish<HD, G, kFmThreads>(a, srec, sw, kvh, split);
}

template <int HD, int G>
static size_t fm_smem_bytes() {
  return (size_t)kFmStages * 2 * kFmTile * HD * 2 + (size_t)kFmWarps * G * 4;
}

template <int HD, int G, bool ROPE>
static cudaError_t fm_launch(const FdArgs& a, cudaStream_t st, bool pdl) {
  const size_t smem = fm_smem_bytes<HD, G>();
  static bool attr_set[kMaxDevices] = {false};
  const cudaError_t ea = opt_in_smem(flash_decode_mma_kernel<HD, G, ROPE>, (int)smem, attr_set);
  if (ea != cudaSuccess) return ea;
  return launch(flash_decode_mma_kernel<HD, G, ROPE>, dim3(a.n_splits, a.n_kv), dim3(kFmThreads),
                smem, st, pdl, a);
}

static size_t fd_counter_bytes(int n_kv) { return ((size_t)n_kv * 4 + 255) & ~(size_t)255; }

}  // namespace b200

using namespace b200;

// Argument checks of b200_flash_decode, shared with the variant that brings its own scratch (which
// must refuse a bad call before it enqueues anything).
static int fd_check_args(const void* out, const void* q, const void* kcache, const void* vcache,
                         const int* kv_len_dev, const void* workspace, int n_q, int n_kv, int hd,
                         int64_t kv_head_stride, int64_t kv_row_stride, int n_splits) {
  if (!out || !q || !kcache || !vcache || !kv_len_dev || !workspace) return B200_ERR_ARG;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_splits <= 0 || n_splits > 1024)
    return B200_ERR_SHAPE;
  const int G = n_q / n_kv;
  if ((hd != 64 && hd != 128) || (G != 1 && G != 2 && G != 4 && G != 8)) return B200_ERR_SHAPE;
  if ((kv_row_stride & 7) != 0 || (kv_head_stride & 7) != 0 || ((uintptr_t)kcache & 15) != 0 ||
      ((uintptr_t)vcache & 15) != 0 || ((uintptr_t)q & 15) != 0 || ((uintptr_t)workspace & 15) != 0)
    return B200_ERR_ALIGN;
  return B200_OK;
}

extern "C" int64_t b200_flash_decode_workspace_bytes(int n_q, int n_kv, int hd, int n_splits) {
  if (n_q <= 0 || n_kv <= 0 || n_splits <= 0) return 0;
  const int G = n_q / n_kv;
  // per kv head and split: acc[G][hd], m[G], l[G], padded to 16 bytes
  return (int64_t)fd_counter_bytes(n_kv) + (int64_t)n_kv * n_splits * (G * hd + ((2 * G + 3) & ~3)) * 4;
}

extern "C" int b200_flash_decode(void* out, int out_dtype, const void* q, int q_dtype,
                                 const void* kcache, const void* vcache, const int* kv_len_dev,
                                 void* workspace, int n_q, int n_kv, int hd,
                                 int64_t kv_head_stride, int64_t kv_row_stride,
                                 int n_splits, float scale, int flags, b200_stream_t stream) {
  const int bad = fd_check_args(out, q, kcache, vcache, kv_len_dev, workspace, n_q, n_kv, hd,
                                kv_head_stride, kv_row_stride, n_splits);
  if (bad != B200_OK) return bad;
  FdArgs a{};
  a.out = out; a.q = q; a.k = (const uint16_t*)kcache; a.v = (const uint16_t*)vcache;
  a.kv_len = kv_len_dev;
  a.counters = (int*)workspace;
  a.recs = (float*)((char*)workspace + fd_counter_bytes(n_kv));
  a.n_q = n_q; a.n_kv = n_kv; a.n_splits = n_splits; a.out_dtype = out_dtype; a.q_dtype = q_dtype;
  a.head_stride = kv_head_stride; a.row_stride = kv_row_stride;
  a.scale_log2 = scale * 1.4426950408889634f;
  const int G = n_q / n_kv;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
#define FD_CASE(HD_, G_) if (hd == HD_ && G == G_) e = fm_launch<HD_, G_, false>(a, st, pdl); else
  FD_CASE(128, 1) FD_CASE(128, 2) FD_CASE(128, 4) FD_CASE(128, 8)
  FD_CASE(64, 1) FD_CASE(64, 2) FD_CASE(64, 4) FD_CASE(64, 8)
  return B200_ERR_SHAPE;
#undef FD_CASE
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

/* b200_qk_rope_cache + b200_flash_decode in one launch for the decode step: q, k and v of the
 * new position (row kv_len - 1) are read from the packed fp32 projection row, (QK-RMSNorm +) RoPE
 * is applied in the attention kernel's prologue, the new k / v row is appended to the cache by the
 * CTA whose slice ends with it, and attention runs over rows [0, kv_len). */
extern "C" int b200_rope_flash_decode(void* out, int out_dtype, const float* qkv, void* kcache,
                                      void* vcache, const float* cos_t, const float* sin_t,
                                      const void* qn_w, const void* kn_w, float eps,
                                      const int* kv_len_dev, void* workspace, int n_q, int n_kv,
                                      int hd, int64_t kv_head_stride, int64_t kv_row_stride,
                                      int max_seq, int n_splits, float scale, int flags,
                                      b200_stream_t stream) {
  if (!out || !qkv || !kcache || !vcache || !cos_t || !sin_t || !kv_len_dev || !workspace)
    return B200_ERR_ARG;
  if ((qn_w == nullptr) != (kn_w == nullptr)) return B200_ERR_ARG;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_splits <= 0 || n_splits > 1024 || max_seq <= 0)
    return B200_ERR_SHAPE;
  if ((kv_row_stride & 7) != 0 || (kv_head_stride & 7) != 0 || ((uintptr_t)kcache & 15) != 0 ||
      ((uintptr_t)vcache & 15) != 0 || ((uintptr_t)qkv & 15) != 0 ||
      ((uintptr_t)workspace & 15) != 0 || ((uintptr_t)cos_t & 15) != 0 ||
      ((uintptr_t)sin_t & 15) != 0)
    return B200_ERR_ALIGN;
  FdArgs a{};
  a.out = out; a.q = nullptr; a.k = (const uint16_t*)kcache; a.v = (const uint16_t*)vcache;
  a.kv_len = kv_len_dev;
  a.counters = (int*)workspace;
  a.recs = (float*)((char*)workspace + fd_counter_bytes(n_kv));
  a.n_q = n_q; a.n_kv = n_kv; a.n_splits = n_splits; a.out_dtype = out_dtype; a.q_dtype = B200_F32;
  a.head_stride = kv_head_stride; a.row_stride = kv_row_stride;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.qkv = qkv; a.cos_t = cos_t; a.sin_t = sin_t;
  a.qn_w = (const uint16_t*)qn_w; a.kn_w = (const uint16_t*)kn_w; a.eps = eps; a.max_seq = max_seq;
  const int G = n_q / n_kv;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
#define FD_CASE(HD_, G_) if (hd == HD_ && G == G_) e = fm_launch<HD_, G_, true>(a, st, pdl); else
  FD_CASE(128, 1) FD_CASE(128, 2) FD_CASE(128, 4) FD_CASE(128, 8)
  FD_CASE(64, 1) FD_CASE(64, 2) FD_CASE(64, 4) FD_CASE(64, 8)
  return B200_ERR_SHAPE;
#undef FD_CASE
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// Flash-decode for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they need
// attention: a plugin running inside another framework's memory pool, a real-time serving
// loop that forbids allocation (and the implicit synchronisation it can bring) after
// start-up, or a process whose memory budget was fixed when it was launched.  For them the
// split records and arrival counters live in the fixed array below instead of a
// caller-provided workspace.  Every GPU that loads the library holds these 2 MiB until the
// process exits.
constexpr size_t kFdStaticBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_fd_static_scratch[kFdStaticBytes];

// In host code `g_fd_static_scratch` is only a stand-in for the symbol, never a device
// address; the real address is looked up once per device (with that device current).
static void* g_fd_static_ptr[kMaxDevices] = {nullptr};

static int fd_static_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_ERR_ARG;
  if (g_fd_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fd_static_scratch) != cudaSuccess || p == nullptr)
      return B200_ERR_LAUNCH;
    g_fd_static_ptr[dev] = p;
  }
  *out = g_fd_static_ptr[dev];
  return B200_OK;
}

extern "C" int64_t b200_flash_decode_static_max_bytes(void) { return (int64_t)kFdStaticBytes; }

extern "C" int b200_flash_decode_static(void* out, int out_dtype, const void* q, int q_dtype,
                                        const void* kcache, const void* vcache,
                                        const int* kv_len_dev, int n_q, int n_kv, int hd,
                                        int64_t kv_head_stride, int64_t kv_row_stride,
                                        int n_splits, float scale, int flags,
                                        b200_stream_t stream) {
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_splits <= 0) return B200_ERR_SHAPE;
  // sizes whose records do not fit the fixed array are refused, never truncated
  if (b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits) > (int64_t)kFdStaticBytes)
    return B200_ERR_SCRATCH;
  void* scratch = nullptr;
  const int rc = fd_static_address(&scratch);   // first call on a device resolves the symbol
  if (rc != B200_OK) return rc;
  // every check b200_flash_decode makes, before anything is enqueued on the caller's stream
  const int bad = fd_check_args(out, q, kcache, vcache, kv_len_dev, scratch, n_q, n_kv, hd,
                                kv_head_stride, kv_row_stride, n_splits);
  if (bad != B200_OK) return bad;
  // The array keeps whatever the previous call left; the arrival counters must start at zero.
  if (cudaMemsetAsync(scratch, 0, fd_counter_bytes(n_kv), (cudaStream_t)stream) != cudaSuccess)
    return B200_ERR_LAUNCH;
  return b200_flash_decode(out, out_dtype, q, q_dtype, kcache, vcache, kv_len_dev, scratch, n_q,
                           n_kv, hd, kv_head_stride, kv_row_stride, n_splits, scale, flags, stream);
}
