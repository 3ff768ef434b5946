// Pieces of the split-KV decode attention shared by the stand-alone kernel (flash_decode.cu) and
// the persistent decode kernel (decode_layers.cu): launch arguments, the cp.async / ldmatrix /
// mma.sync helpers, and the record merge + last-arriver combine.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kFdOutPairs = 2;      // FdArgs::out_dtype: {fp32 value, tag} pairs, one 64-bit store each
struct FdArgs {
  void* out; const void* q; const uint16_t* k; const uint16_t* v; const int* kv_len;
  int* counters; float* recs;
  int n_q, n_kv, n_splits, out_dtype, q_dtype;
  long head_stride, row_stride;  // elements
  float scale_log2;
  // ROPE variant: q / k / v of the new position come straight from the packed fp32 projection
  // row; the kernel applies (QK-RMSNorm +) RoPE itself and appends the row to the cache
  const float* qkv; const float* cos_t; const float* sin_t;
  const uint16_t* qn_w; const uint16_t* kn_w;
  float eps; int max_seq;
  unsigned tag;                  // kFdOutPairs: the tag written beside every value
};

// ---- shared tail of both kernels -------------------------------------------------------------
// In: srec[NREC][REC] holds NREC <= 32 records (acc[G][HD], m[G], l[G]), one per warp unless the
// caller says otherwise.  The records are merged,
// the CTA's record goes to the workspace, and the CTA that arrives last on the kv head's counter
// merges the n_splits records.  srec is re-used as scratch by that last step and must hold at
// least 6 * THREADS floats.
template <int HD, int G, int THREADS, int NREC = THREADS / 32>
__device__ __forceinline__ void fd_finish(const FdArgs& a, float* srec, float* sw, int kvh,
                                          int split) {
  constexpr int WARPS = THREADS / 32;
  constexpr int REC = G * HD + ((2 * G + 3) & ~3);
  __shared__ float s_M[G], s_den[G];
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __syncthreads();
  // ---- merge the CTA's warps: warp g' computes the weights of head g' ----
  for (int g = warp; g < G; g += WARPS) {
    const float mv = lane < NREC ? srec[lane * REC + G * HD + g] : -INFINITY;
    const float M = warp_max(mv);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    const float w = lane < NREC ? exp2f(mv - Mu) : 0.f;
    const float den = warp_sum(lane < NREC ? srec[lane * REC + G * HD + G + g] * w : 0.f);
    if (lane < NREC) sw[lane * G + g] = w;
    if (lane == 0) { s_M[g] = M; s_den[g] = den; }
  }
  __syncthreads();
  float* wr = a.recs + (size_t)(kvh * a.n_splits + split) * REC;
  for (int i = tid; i < G * HD; i += THREADS) {
    const int g = i / HD;
    float num = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < NREC; ++w2) num = fmaf(srec[w2 * REC + i], sw[w2 * G + g], num);
    wr[i] = num;
  }
  if (tid < G) { wr[G * HD + tid] = s_M[tid]; wr[G * HD + G + tid] = s_den[tid]; }

  // ---- publish, and let the last-arriving CTA of this kv head finish the job ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&a.counters[kvh], 1);
    s_last = (old == a.n_splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // Every thread owns one float4 column of the output and every PARTS-th split: all its loads
  // are independent (one L2 round trip), the partial results meet in shared memory.
  constexpr int C4 = G * HD / 4;
  constexpr int PARTS = (THREADS / C4) >= 8 ? 8 : ((THREADS / C4) >= 1 ? (THREADS / C4) : 1);
  static_assert(C4 <= THREADS, "one pass over the output columns");
  float4* sp_num = reinterpret_cast<float4*>(srec);             // [PARTS][C4]
  float* sp_m = srec + 4 * PARTS * C4;                          // [PARTS][C4]
  float* sp_d = sp_m + PARTS * C4;
  const float* rb = a.recs + (size_t)kvh * a.n_splits * REC;
  const int ns = a.n_splits;
  if (tid < PARTS * C4) {
    const int c = tid % C4, part = tid / C4, g = (c * 4) / HD;
    float m_run = -INFINITY, den = 0.f;
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int sp = part; sp < ns; sp += PARTS) {
      const float* rec = rb + (size_t)sp * REC;
      const float mv = __ldcg(rec + G * HD + g);
      const float lv = __ldcg(rec + G * HD + G + g);
      const float4 r = __ldcg(reinterpret_cast<const float4*>(rec) + c);
      const float mn = fmaxf(m_run, mv);
      const float mu = (mn == -INFINITY) ? 0.f : mn;
      const float wa = exp2f(m_run - mu), wb = exp2f(mv - mu);
      num.x = num.x * wa + r.x * wb; num.y = num.y * wa + r.y * wb;
      num.z = num.z * wa + r.z * wb; num.w = num.w * wa + r.w * wb;
      den = den * wa + lv * wb;
      m_run = mn;
    }
    sp_num[tid] = num; sp_m[tid] = m_run; sp_d[tid] = den;
  }
  __syncthreads();
  if (tid < C4) {
    float m_run = sp_m[tid], den = sp_d[tid];
    float4 num = sp_num[tid];
#pragma unroll
    for (int p = 1; p < PARTS; ++p) {
      const float mv = sp_m[p * C4 + tid], lv = sp_d[p * C4 + tid];
      const float4 r = sp_num[p * C4 + tid];
      const float mn = fmaxf(m_run, mv);
      const float mu = (mn == -INFINITY) ? 0.f : mn;
      const float wa = exp2f(m_run - mu), wb = exp2f(mv - mu);
      num.x = num.x * wa + r.x * wb; num.y = num.y * wa + r.y * wb;
      num.z = num.z * wa + r.z * wb; num.w = num.w * wa + r.w * wb;
      den = den * wa + lv * wb;
      m_run = mn;
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const size_t oi = (size_t)kvh * G * HD + (size_t)tid * 4;
    if (a.out_dtype == kFdOutPairs) {
      const float r[4] = {num.x * inv, num.y * inv, num.z * inv, num.w * inv};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const unsigned long long w2 = ((unsigned long long)a.tag << 32) | __float_as_uint(r[e]);
        asm volatile("st.global.b64 [%0], %1;" ::"l"(reinterpret_cast<uint2*>(a.out) + oi + e), "l"(w2) : "memory");
      }
    } else if (a.out_dtype == B200_F32) {
      reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + oi)[0] =
          make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
    } else {
      uint2 w2;
      w2.x = pack_bf16(num.x * inv, num.y * inv);
      w2.y = pack_bf16(num.z * inv, num.w * inv);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(a.out) + oi) = w2;
    }
  }
  if (tid == 0) a.counters[kvh] = 0;  // ready for the next launch
}

// ---- tensor-core variant ---------------------------------------------------------------------
// The SIMT kernel above spends ~185 instructions per KB of cache (a 16-lane shuffle reduction per
// key and head) and is issue-bound near 4 TB/s.  Here a CTA of eight warps streams 128-key tiles
// of K and V through a three-stage cp.async ring; each warp owns 16 keys of a tile and runs
// S = Q K^T and O += P V on mma.sync m16n8k16 (about 20 instructions per KB).  The 16-row A
// operand carries the group's G <= 8 query heads twice: rows 0..7 hold the bf16 high part of q
// (and of P), rows 8..15 the bf16 low part, so q and P keep ~16 mantissa bits at no extra MMA and
// the two halves of an accumulator add up inside one thread.
constexpr int kFmThreads = 256, kFmWarps = 8, kFmTile = 128, kFmStages = 3;

__device__ __forceinline__ void fm_cp16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void fm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fm_ldsm(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void fm_ldsm_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void fm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset of 16-byte chunk c of row r in an XOR-swizzled [rows][HD] bf16 tile
template <int HD>
__device__ __forceinline__ uint32_t fm_swz(int r, int c) {
  return (uint32_t)(r * (HD * 2) + ((c ^ (r & 7)) << 4));
}
// bf16 high / low split of two fp32 values, packed for an A fragment
__device__ __forceinline__ void fm_split(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat16 xh = __float2bfloat16(x), yh = __float2bfloat16(y);
  hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
  lo = pack_bf16(x - __bfloat162float(xh), y - __bfloat162float(yh));
}

}  // namespace b200
