// Peer-memory link of a tensor-parallel decode step and the tagged-pair helpers shared by the
// kernels that publish into it or consume from it.
//
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
// Two alternatives were measured and removed: every CTA summing the inboxes itself (world x 32 KB
// of L2 reads per CTA: 1.94 against 1.76 ms per Llama-3.1-8B step on four GPUs), and plain stores
// followed by a system fence and one release flag per rank (slower than a collective library:
// the fence waits out the NVLink round trip).
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kTpMaxRanks = 8;
constexpr int kTpReducers = 8;     // CTAs that sum the ranks' contributions
// Every wait on a peer (and every grid-wide wait of the persistent decode kernel) is bounded by
// a clock budget: ~2 s by default, B200_TUNE_WAIT_KTICKS (units of 1024 ticks) overrides it.
constexpr long long kDefaultWaitTicks = 4000000000LL;
inline long long wait_ticks_from_tuning() {
  const int t = g_tuning[B200_TUNE_WAIT_KTICKS];
  return t > 0 ? (long long)t * 1024 : kDefaultWaitTicks;
}

struct TpLink {
  float* inbox[kTpMaxRanks];        // inbox of rank p (peer-mapped): [2 slots][world][H]
                                    // {fp32 value, u32 tag} pairs
  const int* seq_base;              // device scalar: sequence number of the step's first all-reduce
  int world, rank, H;
  uint4* xr;                        // local staging of the reduced vector: [2 slots][H] pairs
  long long wait_ticks;             // budget of every bounded wait (filled in at launch)
};

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_volatile_v2(uint2* p, uint2 v) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Sum over n tagged-pair vectors (stride in uint4) of the float4 at q0: every 8-byte
// {value, tag} pair arrives atomically, so the data itself is polled (bounded) - no flag, no fence.
__device__ __forceinline__ float4 ll_reduce(const uint4* q0, int n, int stride, unsigned tag,
                                            int* status, long long budget) {
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
        if (clock64() - t0 > budget) {
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

// The reducer CTAs' share of consuming all-reduce `tag - 1` (slot = its parity): CTA b < nred sums
// the ranks' pairs of slice b of the H-vector in rank order, publishes the sums locally as tagged
// pairs in xr and, if x_out is given, stores them there as plain floats.
template <int THREADS>
__device__ __forceinline__ void tp_reduce_slice(const TpLink& l, unsigned slot, unsigned tag,
                                                float* x_out, int* status) {
  const int nred = min(kTpReducers, (int)gridDim.x);
  if ((int)blockIdx.x >= nred) return;
  const int H = l.H, n4 = H >> 2, per = (n4 + nred - 1) / nred;
  const int lo = blockIdx.x * per, hi = min(n4, lo + per);
  const uint4* box = reinterpret_cast<const uint4*>(l.inbox[l.rank]) + (size_t)slot * l.world * (H >> 1);
  uint4* dst = l.xr + (size_t)slot * (H >> 1);
  for (int i = lo + threadIdx.x; i < hi; i += THREADS) {
    const float4 v = ll_reduce(box + 2 * i, l.world, H >> 1, tag, status, l.wait_ticks);
    st_volatile_v4(dst + 2 * i, make_uint4(__float_as_uint(v.x), tag, __float_as_uint(v.y), tag));
    st_volatile_v4(dst + 2 * i + 1, make_uint4(__float_as_uint(v.z), tag, __float_as_uint(v.w), tag));
    if (x_out != nullptr) reinterpret_cast<float4*>(x_out)[i] = v;
  }
}
// Elements 4i .. 4i+3 of the reduced vector, polled from the local staging the reducers fill.
__device__ __forceinline__ float4 tp_read_reduced(const TpLink& l, unsigned slot, unsigned tag, int i,
                                                  int* status) {
  return ll_reduce(l.xr + (size_t)slot * (l.H >> 1) + 2 * i, 1, 0, tag, status, l.wait_ticks);
}
// Element i of the reduced vector (polled, bounded).
__device__ __forceinline__ float tp_read_one(const TpLink& l, unsigned slot, unsigned tag, int i,
                                             int* status) {
  const volatile uint2* p = reinterpret_cast<const volatile uint2*>(l.xr) + (size_t)slot * l.H + i;
  long long t0 = 0;
  int spins = 0;
  while (true) {
    // the pair as one 64-bit word: value and tag cannot be torn apart
    const unsigned long long w = *reinterpret_cast<const volatile unsigned long long*>(p);
    if ((unsigned)(w >> 32) == tag) return __uint_as_float((unsigned)w);
    if ((++spins & 63) == 0) {
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return 0.f;
      if (t0 == 0) t0 = clock64();
      if (clock64() - t0 > l.wait_ticks) {
        if (status != nullptr) atomicExch(status, B200_ERR_TIMEOUT);
        return 0.f;
      }
    }
  }
}
// This rank's share `v` of element `oi` of all-reduce `seq` into every rank's inbox.
__device__ __forceinline__ void tp_publish(const TpLink& l, unsigned seq, int oi, float v) {
  const size_t off = ((size_t)(seq & 1u) * l.world + l.rank) * l.H + oi;
  for (int p = 0; p < l.world; ++p)
    st_volatile_v2(reinterpret_cast<uint2*>(l.inbox[p]) + off, make_uint2(__float_as_uint(v), seq + 1u));
}

// Link registered under context id `ctx` by b200_tp_create, or nullptr (defined in gemv.cu).
const TpLink* tp_link_get(int ctx);

}  // namespace b200
