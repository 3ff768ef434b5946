// All transformer layers of one batch-1 decode step in ONE persistent launch.
//
// A decode step is a chain of small dependent matrix-vector products: launched one by one,
// each pays a dependency wait, a first-byte latency and a tail (3-7 us on B200), which is a
// quarter of the step on one GPU and nearly all of it once tensor parallelism has cut every
// matrix to a few MB.  Here one CTA per SM stays resident for the whole step and walks the
// phases   q|k|v -> attention -> o_proj -> gate|up -> down   of every layer:
//
//   * Weights never depend on the previous phase.  Every warp owns a private ring in shared
//     memory (kDlRing batches of kDlU x 512 bytes per lane-private cp.async) and keeps it full
//     ACROSS phase boundaries: while the CTA waits for the other CTAs and stages the next input
//     vector, the first kDlRing batches of the next matrix are already in flight.  A lane only
//     ever reads back what it copied itself, so the ring needs no barrier.
//   * Work split as in the stand-alone GEMV: a CTA owns a contiguous block of rows, the block is
//     one flat run of 512-byte segments cut into sixteen equal pieces, one per warp; row sums are
//     finished in warp order, so results are bit-reproducible.
//   * Attention is the split-KV tensor-core loop of flash_decode.cu on 128-key tiles, with all
//     sixteen warps busy: warps w and w + 8 share 16 keys of a tile, both compute S = Q K^T, each
//     accumulates P V for one half of the head dimension (32 accumulator registers instead of 64,
//     which is what lets 512 threads fit the register file).  The K/V ring borrows the weight
//     ring and the vector staging area; the first two tiles are requested before the wait on
//     the q|k|v projection.  RoPE, QK-RMSNorm and the cache append run in its prologue.
//   * There is no grid-wide barrier.  A phase hands its output vector to the next one as 8-byte
//     {fp32 value, tag} pairs, each written with one 64-bit store; the tag names the launch and
//     the producing phase, so the data validates itself and a consumer simply polls (bounded)
//     the elements it stages: one L2 round trip from "last row written" to "vector staged",
//     where a barrier costs a fence, an atomic, a poll and then the loads.  A buffer is rewritten
//     only by a phase that (transitively) needed every reader's own rows, so no reader can be
//     overtaken; a CTA without rows in a phase does not read.  Under tensor parallelism o_proj
//     and down push their rows to every rank in the same pair format and the next phase reduces
//     them (tp_link.cuh): no collective library call and no extra launch.
//
// Every wait is bounded by a clock budget; when one expires the status word receives
// B200_ERR_TIMEOUT, all later waits fall through at once and the kernel runs to its end.
#include <vector>

#include "common.cuh"
#include "flash_decode_core.cuh"
#include "tp_link.cuh"

namespace b200 {

constexpr int kDlThreads = 512, kDlWarps = 16;
constexpr int kDlU = 4;                                  // 512-byte segments per batch
constexpr int kDlRing = 4;                               // batches per warp in flight
constexpr int kDlBatchBytes = kDlU * 512;                // 2 KB per warp per batch
constexpr int kDlWarpRing = kDlRing * kDlBatchBytes;     // 8 KB per warp
constexpr int kDlRingBytes = kDlWarps * kDlWarpRing;     // 128 KB: weight rings / K,V stages 0, 1
constexpr int kDlXsBytes = 64 * 1024;                    // staged input vector / K,V stage 2
constexpr int kDlMaxK = kDlXsBytes / 4;                  // 16384
constexpr int kDlMaxRows = 256;                          // rows of one phase per CTA
constexpr int kDlPartBytes = kDlMaxRows * kDlWarps * 4;  // 16 KB
constexpr int kDlSmemBytes = kDlXsBytes + kDlRingBytes + kDlPartBytes + 256;

enum { DL_GEMV = 0, DL_ATT = 1 };
enum { DL_IN_PLAIN = 0, DL_IN_PAIRS = 1, DL_IN_TP = 2 };

// One entry of the phase table (device memory, written once at set-up).
struct DlPhase {
  const uint16_t* w;          // GEMV: [N, K] bf16, rows contiguous
  const uint16_t* norm_w;     // GEMV: RMSNorm weight applied to the input (nullable)
  const float* x;             // GEMV, DL_IN_PLAIN: input vector written before the launch
  const uint2* xp;            // DL_IN_PAIRS: input as {value, tag} pairs of the previous phase
  float* y;                   // GEMV: plain copy of the output (nullable; the residual stream)
  uint2* yp;                  // output as {value, tag} pairs (nullable under tp_out)
  const float* resid;         // GEMV: added to the output (nullable; read by the row's owner only)
  float* x_out;               // GEMV fed by an all-reduce: the reduced vector is stored here
  const uint16_t* kc;         // ATT: this layer's K cache [n_kv, max_seq, hd]
  const uint16_t* vc;         // ATT: V cache
  const uint16_t* qn_w;       // ATT: QK-RMSNorm weights (nullable)
  const uint16_t* kn_w;
  int N, K, rpc;
  int flags;                  // type | input kind << 4 | epilogue << 8
  int tp_in, tp_out;          // all-reduce consumed / fed by this phase (-1: none)
  int resid_tp;               // >= 0: the residual is the reduced vector of this all-reduce
  int pad;
  __device__ __host__ int type() const { return flags & 15; }
  __device__ __host__ int in() const { return (flags >> 4) & 15; }
  __device__ __host__ int epilogue() const { return (flags >> 8) & 15; }
};
static_assert(sizeof(DlPhase) == 128, "phase table layout");

struct DlArgs {
  const DlPhase* phases;
  int n_phases;
  // attention
  const float* cos_t; const float* sin_t;
  const int* kv_len;
  int* fd_counters; float* fd_recs;
  int n_q, n_kv, n_splits, max_seq;
  long head_stride, row_stride;
  float scale_log2, eps;
  // synchronisation
  unsigned* epoch;            // launches so far (device scalar; CTA 0 advances it at its end)
  long long wait_ticks;
  int* status;
  TpLink tp;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
template <int N>
__device__ __forceinline__ void dl_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tagged pairs ---------------------------------------------------------------------------------
// Tag of the vector phase p produces in launch number `epoch`: never 0 (fresh buffers are zero),
// unique for 2^32 / (phases + 1) launches.
__device__ __forceinline__ unsigned dl_tag(unsigned epoch, int n_phases, int p) {
  return epoch * (unsigned)(n_phases + 1) + (unsigned)p + 1u;
}
__device__ __forceinline__ void dl_put(uint2* p, float v, unsigned tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");   // one single-copy-atomic store
}
// Two neighbouring pairs with one 16-byte load; spins (bounded) until both carry `tag`.  A torn
// load is harmless: each pair is checked against its own tag.
__device__ __forceinline__ uint4 dl_poll2(const uint2* p, uint4 e, unsigned tag, const DlArgs& a) {
  long long t0 = 0;
  int spins = 0;
  while (e.y != tag || e.w != tag) {
    if ((++spins & 15) == 0) {
      if (*reinterpret_cast<volatile int*>(a.status) != 0) break;     // an earlier wait gave up
      if (t0 == 0) t0 = clock64();
      if (clock64() - t0 > a.wait_ticks) { atomicExch(a.status, B200_ERR_TIMEOUT); break; }
    }
    e = ld_volatile_v4(reinterpret_cast<const uint4*>(p));
  }
  return e;
}

// The phase table lives in global memory, and an entry's pointers sit in front of every
// dependent load: a cold read would put a DRAM round trip on the critical path of each phase.
// A window of entries is kept in shared memory instead: entries 0 .. kDlAhead - 1 are copied at
// kernel start and every attention phase p requests entries p + 5 .. p + kDlAhead - 1
// (asynchronous copies that its own final wait covers).  A table therefore has an attention
// phase at least every five entries, as the plan builder's layers do.
constexpr int kDlWin = 16, kDlAhead = 10;
__device__ __forceinline__ const DlPhase& dl_ph(const DlPhase* win, int p) { return win[p & (kDlWin - 1)]; }

// ---- the weight stream of one warp ------------------------------------------------------------
// Position of the NEXT batch to request: phase p, segments [f, s1) of this warp's piece of the
// CTA's row block.  The cursor runs up to kDlRing batches ahead of the arithmetic and stops at an
// attention phase (which borrows the ring) and at the end of the table.
struct DlCursor {
  int p, f, s1;
  const unsigned char* base;   // first byte of the CTA's row block + lane * 16
  unsigned issued;             // real batches requested so far (ring slot = issued % kDlRing)
};

__device__ __forceinline__ void dl_piece(const DlPhase& ph, int warp, int& nrows, int& s0, int& s1) {
  const int r0 = blockIdx.x * ph.rpc;
  nrows = max(0, min(ph.N - r0, ph.rpc));
  const int S = nrows * (ph.K >> 8);
  s0 = (int)((long)S * warp / kDlWarps);
  s1 = (int)((long)S * (warp + 1) / kDlWarps);
}

// Move the cursor to the first phase at or after c.p in which this warp has work; stop at an
// attention phase or at the end of the table with nothing to request (f == s1).
__device__ __forceinline__ void dl_seek(DlCursor& c, const DlArgs& a, const DlPhase* win, int warp,
                                        int lane) {
  c.f = c.s1 = 0;
  while (c.p < a.n_phases) {
    const DlPhase& ph = dl_ph(win, c.p);
    if (ph.type() != DL_GEMV) return;
    int nrows, s0, s1;
    dl_piece(ph, warp, nrows, s0, s1);
    if (s1 > s0) {
      c.f = s0; c.s1 = s1;
      c.base = reinterpret_cast<const unsigned char*>(ph.w) +
               (size_t)blockIdx.x * ph.rpc * ph.K * 2 + lane * 16;
      return;
    }
    ++c.p;
  }
}

// Request the next batch (if any) into its ring slot and commit exactly one cp.async group, real
// or empty, so that "all but the newest kDlRing - 1 groups" always covers the batch consumed next.
__device__ __forceinline__ void dl_issue(DlCursor& c, const DlArgs& a, const DlPhase* win,
                                         uint32_t ring_lane, int warp, int lane) {
  if (c.f < c.s1) {
    const uint32_t dst = ring_lane + (c.issued % kDlRing) * kDlBatchBytes;
#pragma unroll
    for (int j = 0; j < kDlU; ++j)
      if (c.f + j < c.s1) fm_cp16(dst + j * 512, c.base + (size_t)(c.f + j) * 512);
    ++c.issued;
    c.f += kDlU;
    if (c.f >= c.s1) { ++c.p; dl_seek(c, a, win, warp, lane); }
  }
  fm_commit();
}

// ---- staging of a phase's input vector -----------------------------------------------------------
// Stages x as fp32, segment-swizzled ([seg][half][lane]
// float4), and leaves each warp's share of sum(x^2) in red[warp].  RMSNorm: x * w is staged, the
// scalar rsqrt(mean(x^2) + eps) multiplies the row sums in the epilogue, so nothing here waits
// for the sum of squares.
__device__ __forceinline__ void dl_stage(const DlArgs& a, const DlPhase* php, float* xs, float* red,
                                      unsigned tag_in) {
  const DlPhase& ph = *php;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = ph.K;
  const uint16_t* norm_w = ph.norm_w;
  float ss = 0.f;
  // element pair (k, k + 1), k even, of the staged vector
  auto put2 = [&](int k, float x0, float x1) {
    ss += x0 * x0 + x1 * x1;
    if (norm_w != nullptr) {
      const uint32_t u = reinterpret_cast<const uint32_t*>(norm_w)[k >> 1];
      x0 *= bf16lo(u); x1 *= bf16hi(u);
    }
    const int seg = k >> 8, within = k & 255;
    const int slot = seg * 64 + ((within >> 2) & 1) * 32 + (within >> 3);
    *reinterpret_cast<float2*>(xs + slot * 4 + (k & 3)) = make_float2(x0, x1);
  };
  if (ph.in() == DL_IN_PAIRS) {
    // the producers' rows arrive as tagged pairs: all loads of a round are in flight together,
    // then each is re-read until its tags are this launch's
    constexpr int R = 8;
    const uint4* src = reinterpret_cast<const uint4*>(ph.xp);
    const int n2 = K >> 1;
    for (int i0 = 0; i0 < n2; i0 += R * kDlThreads) {
      uint4 e[R];
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int i = i0 + tid + j * kDlThreads;
        if (i < n2) e[j] = ld_volatile_v4(src + i);
      }
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const int i = i0 + tid + j * kDlThreads;
        if (i < n2) {
          e[j] = dl_poll2(ph.xp + 2 * i, e[j], tag_in, a);
          put2(2 * i, __uint_as_float(e[j].x), __uint_as_float(e[j].z));
        }
      }
    }
  } else if (ph.in() == DL_IN_TP) {
    const unsigned seq = (unsigned)(a.tp.seq_base[0] + ph.tp_in);
    const unsigned tp_slot = seq & 1u, tp_tag = seq + 1u;
    tp_reduce_slice<kDlThreads>(a.tp, tp_slot, tp_tag, ph.x_out, a.status);
    for (int i = tid; i < (K >> 2); i += kDlThreads) {
      const float4 v = tp_read_reduced(a.tp, tp_slot, tp_tag, i, a.status);
      put2(4 * i, v.x, v.y);
      put2(4 * i + 2, v.z, v.w);
    }
  } else {
    for (int i = tid; i < (K >> 2); i += kDlThreads) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(ph.x) + i);
      put2(4 * i, v.x, v.y);
      put2(4 * i + 2, v.z, v.w);
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
}

// ---- one matrix-vector phase --------------------------------------------------------------------
struct DlStream {
  DlCursor cur;
  unsigned consumed;           // batches taken out of the ring so far
};
// The stream state goes in and comes back by value.  (Everything here is inlined into the
// kernel: out-of-line phases were measured 9 % slower per step - the call ABI keeps the cursor in
// local memory.)
__device__ __forceinline__ DlStream dl_gemv(const DlArgs& a, const DlPhase* win, DlStream st,
                                         unsigned epoch, float* xs, float* part, float* red,
                                         uint32_t ring_lane, int p) {
  DlCursor& cur = st.cur;
  unsigned& consumed = st.consumed;
  const DlPhase& ph = dl_ph(win, p);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = ph.K, spr = K >> 8;
  const int r0 = blockIdx.x * ph.rpc;
  int nrows, s0, s1;
  dl_piece(ph, warp, nrows, s0, s1);

  // ---- the input vector becomes valid ----
  __syncthreads();                            // every warp is done with the staging area
  // a CTA without rows in this phase must not read the vector: readers are what keeps a later
  // phase from overwriting it early (see the top of the file).  Under tensor parallelism the
  // reducer CTAs still have their slice of the all-reduce to sum.
  if (nrows > 0 || ph.in() == DL_IN_TP) dl_stage(a, &ph, xs, red, dl_tag(epoch, a.n_phases, p - 1));
  for (int i = tid; i < nrows; i += kDlThreads) {
#pragma unroll
    for (int w2 = 0; w2 < kDlWarps; ++w2) part[w2 * kDlMaxRows + i] = 0.f;
  }
  __syncthreads();
  const float4* xs4 = reinterpret_cast<const float4*>(xs);
  float* mine = part + warp * kDlMaxRows;     // part is [warp][row]

  // ---- stream this warp's piece ----
  if (s1 > s0) {
    float acc = 0.f;
    int crow = s0 / spr, ck = s0 - crow * spr;
    for (int f = s0; f < s1; f += kDlU) {
      dl_wait_group<kDlRing - 1>();           // the oldest batch in flight has landed
      const uint32_t src = ring_lane + (consumed % kDlRing) * kDlBatchBytes;
      uint4 w[kDlU];
#pragma unroll
      for (int j = 0; j < kDlU; ++j)
        if (f + j < s1) w[j] = lds128(src + j * 512);
      ++consumed;
#pragma unroll
      for (int j = 0; j < kDlU; ++j) {
        if (f + j < s1) {
          const float4 xa = xs4[ck * 64 + lane];
          const float4 xb = xs4[ck * 64 + 32 + lane];
          acc = fmaf(bf16lo(w[j].x), xa.x, acc);
          acc = fmaf(bf16hi(w[j].x), xa.y, acc);
          acc = fmaf(bf16lo(w[j].y), xa.z, acc);
          acc = fmaf(bf16hi(w[j].y), xa.w, acc);
          acc = fmaf(bf16lo(w[j].z), xb.x, acc);
          acc = fmaf(bf16hi(w[j].z), xb.y, acc);
          acc = fmaf(bf16lo(w[j].w), xb.z, acc);
          acc = fmaf(bf16hi(w[j].w), xb.w, acc);
          if (++ck == spr) {
            const float v = warp_sum(acc);
            if (lane == 0) mine[crow] = v;   // a warp meets every row at most once
            acc = 0.f; ck = 0; ++crow;
          }
        }
      }
      // refill the slot just emptied (its values already went through the FMAs above)
      dl_issue(cur, a, win, ring_lane, warp, lane);
    }
    if (ck != 0) {
      const float v = warp_sum(acc);
      if (lane == 0) mine[crow] = v;
    }
  }
  __syncthreads();

  // ---- epilogue: fixed-order row sums; neighbouring threads read neighbouring words ----
  float out_scale = 1.f;
  if (ph.norm_w != nullptr) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kDlWarps; ++i) tot += red[i];
    out_scale = rsqrtf(tot / (float)K + a.eps);
  }
  auto row_value = [&](int r) -> float {
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < kDlWarps; ++i) v += part[i * kDlMaxRows + r];
    return v * out_scale;
  };
  const unsigned tag = dl_tag(epoch, a.n_phases, p);
  if (ph.epilogue() == B200_EPI_SWIGLU) {
    for (int t = tid; t < (nrows >> 1); t += kDlThreads) {
      const float g = row_value(2 * t), u = row_value(2 * t + 1);
      dl_put(ph.yp + (r0 >> 1) + t, silu_f(g) * u, tag);
    }
  } else {
    for (int t = tid; t < nrows; t += kDlThreads) {
      float v = row_value(t);
      const int oi = r0 + t;
      // the residual stream: its plain copy is read and written by the row's owner only; under
      // tensor parallelism it is the (tagged) reduced vector of an earlier all-reduce
      if (ph.resid_tp >= 0) {
        const unsigned seq = (unsigned)(a.tp.seq_base[0] + ph.resid_tp);
        v += tp_read_one(a.tp, seq & 1u, seq + 1u, oi, a.status);
      } else if (ph.resid != nullptr) {
        v += __ldcg(ph.resid + oi);
      }
      if (ph.tp_out >= 0) {
        tp_publish(a.tp, (unsigned)(a.tp.seq_base[0] + ph.tp_out), oi, v);
      } else {
        if (ph.y != nullptr) ph.y[oi] = v;
        if (ph.yp != nullptr) dl_put(ph.yp + oi, v, tag);
      }
    }
  }
  return st;
}

// ---- attention phase ----------------------------------------------------------------------------
// The warp's stream cursor goes in and comes back by value.
template <int HD, int G>
__device__ __forceinline__ DlCursor dl_attention(const DlArgs& a, DlPhase* win, DlCursor cur,
                                              unsigned epoch, int p, unsigned char* smem,
                                              uint32_t ring_lane) {
  const DlPhase& ph = dl_ph(win, p);
  constexpr int KS = HD / 16;          // k16 steps over the head dim
  constexpr int DB = HD / 8;           // n8 blocks over the head dim
  constexpr int DH = DB / 2;           // n8 blocks of this warp's half of the head dim
  constexpr int CPR = HD / 8;          // 16-byte chunks per row
  constexpr int TILE = kFmTile * HD * 2;                 // bytes of one K (or V) tile
  constexpr int REC = G * HD + ((2 * G + 3) & ~3);
  constexpr int NREC = 8;              // one record per group of 16 keys
  static_assert(2 * TILE <= kDlXsBytes && 4 * TILE <= kDlRingBytes, "K/V stages fit the borrowed areas");
  static_assert((NREC * REC + NREC * G) * 4 <= kDlXsBytes && 6 * kDlThreads * 4 <= kDlXsBytes,
                "records fit the staging area");

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;                // fragment row (= head) and column pair
  const int kg = warp & 7, half = warp >> 3;             // 16-key group of a tile, half of the head dim
  const bool active = (int)blockIdx.x < a.n_kv * a.n_splits;
  const int kvh = active ? blockIdx.x / a.n_splits : 0, split = active ? blockIdx.x % a.n_splits : 0;

  // stage s of the K/V ring: 0 and 1 in the weight-ring area, 2 in the vector staging area
  const uint32_t xs_u32 = smem_u32(smem), ring_u32 = xs_u32 + kDlXsBytes;
  auto stage = [&](int t) -> uint32_t {
    const int s = t % 3;
    return s == 2 ? xs_u32 : ring_u32 + s * 2 * TILE;
  };

  // the length is fixed for the whole launch (the previous step's selection kernel wrote it)
  const int kv_len = a.kv_len[0];
  const int per = (kv_len + a.n_splits - 1) / a.n_splits;
  const int k0 = split * per;
  const int k1 = min(kv_len, k0 + per);
  const int ntiles = (active && k1 > k0) ? (k1 - k0 + kFmTile - 1) / kFmTile : 0;
  const uint16_t* kb = ph.kc + (size_t)kvh * a.head_stride;
  const uint16_t* vb = ph.vc + (size_t)kvh * a.head_stride;
  auto load_tile = [&](int t) {
    const uint32_t sk = stage(t), sv = sk + TILE;
    const int row0 = k0 + t * kFmTile;
    for (int i = tid; i < kFmTile * CPR; i += kDlThreads) {
      const int r = i / CPR, c = i % CPR;
      int gr = row0 + r;
      gr = gr < k1 ? gr : k1 - 1;                        // rows past the slice are masked below
      const size_t off = (size_t)gr * a.row_stride + c * 8;
      fm_cp16(sk + fm_swz<HD>(r, c), kb + off);
      fm_cp16(sv + fm_swz<HD>(r, c), vb + off);
    }
  };

  __syncthreads();
  // Every warp has finished the previous phase's arithmetic and the weight stream is parked at
  // this phase, so the weight rings are free: the first two tiles go out before the wait on the
  // q|k|v projection.  Cache rows of earlier positions never change during a step; the row this
  // step appends is patched in shared memory.
  // the next layer's phase entries come into the window too (first group, covered by the waits
  // of the tile loop and by the final one)
  {
    constexpr int C = sizeof(DlPhase) / 16;
    const int first = p + 5, last = min(p + kDlAhead, a.n_phases);
    if (tid < (last - first) * C) {
      const int e = first + tid / C, c = tid % C;
      fm_cp16(smem_u32(win + (e & (kDlWin - 1))) + c * 16,
              reinterpret_cast<const unsigned char*>(a.phases + e) + c * 16);
    }
  }
  if (0 < ntiles) load_tile(0);
  fm_commit();
  if (1 < ntiles) load_tile(1);
  fm_commit();
  // q (G heads), k and v of this kv head for the new position: polled as tagged pairs of the
  // q|k|v phase, once per CTA, into the staging area (free until the third K/V stage is loaded)
  float* sq = reinterpret_cast<float*>(smem);            // [G + 2][HD]
  if (active) {
    const unsigned tag_in = dl_tag(epoch, a.n_phases, p - 1);
    constexpr int HP = HD / 2;                           // 16-byte loads (two pairs) per head
    for (int i = tid; i < (G + 2) * HP; i += kDlThreads) {
      const int hh = i / HP, c = i % HP;
      const int head = hh < G ? kvh * G + hh : (hh == G ? a.n_q + kvh : a.n_q + a.n_kv + kvh);
      const uint2* src = ph.xp + (size_t)head * HD + 2 * c;
      uint4 e = ld_volatile_v4(reinterpret_cast<const uint4*>(src));
      e = dl_poll2(src, e, tag_in, a);
      *reinterpret_cast<float2*>(sq + hh * HD + 2 * c) = make_float2(__uint_as_float(e.x), __uint_as_float(e.z));
    }
  }
  __syncthreads();

  uint32_t qf[KS][4];
  int pos_own = -1;
  uint4 newk = make_uint4(0, 0, 0, 0), newv = make_uint4(0, 0, 0, 0);
  float o[DH][4];
  float m = -INFINITY, l = 0.f;
#pragma unroll
  for (int d = 0; d < DH; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }

  if (active) {
    // ---- q as A fragments: head g in rows g (high part) and g + 8 (low part) ----
    // One pair of k16 steps (ks, ks + KS/2: a rotate-half partner pair) at a time, straight from
    // the staged row, so that only the finished fragments stay in registers.
    const bool live = g < G;
    const int pos = kv_len - 1;
    const bool in_cache = pos >= 0 && pos < a.max_seq;
    const float* src = sq + (live ? g : 0) * HD;         // dims ks*16 + tq*2 + {0, 1, 8, 9}
    float inv = 1.f;
    if (ph.qn_w != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const float2 u = *reinterpret_cast<const float2*>(src + ks * 16 + tq * 2);
        const float2 w = *reinterpret_cast<const float2*>(src + ks * 16 + tq * 2 + 8);
        ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(w.x, w.x, ss); ss = fmaf(w.y, w.y, ss);
      }
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      inv = rsqrtf(ss / (float)HD + a.eps);
    }
    const size_t ci = (size_t)(in_cache ? pos : 0) * (HD / 2);
    const float sc = live ? a.scale_log2 : 0.f;          // padding rows carry zeros
#pragma unroll
    for (int ks = 0; ks < KS / 2; ++ks) {
      float lo[4], hi[4];
      {
        const float2 u = *reinterpret_cast<const float2*>(src + ks * 16 + tq * 2);
        const float2 w = *reinterpret_cast<const float2*>(src + ks * 16 + tq * 2 + 8);
        const float2 u2 = *reinterpret_cast<const float2*>(src + (ks + KS / 2) * 16 + tq * 2);
        const float2 w2 = *reinterpret_cast<const float2*>(src + (ks + KS / 2) * 16 + tq * 2 + 8);
        lo[0] = u.x; lo[1] = u.y; lo[2] = w.x; lo[3] = w.y;
        hi[0] = u2.x; hi[1] = u2.y; hi[2] = w2.x; hi[3] = w2.y;
      }
      if (ph.qn_w != nullptr) {
        const uint32_t w0 = *reinterpret_cast<const uint32_t*>(ph.qn_w + ks * 16 + tq * 2);
        const uint32_t w1 = *reinterpret_cast<const uint32_t*>(ph.qn_w + ks * 16 + tq * 2 + 8);
        const uint32_t w2 = *reinterpret_cast<const uint32_t*>(ph.qn_w + (ks + KS / 2) * 16 + tq * 2);
        const uint32_t w3 = *reinterpret_cast<const uint32_t*>(ph.qn_w + (ks + KS / 2) * 16 + tq * 2 + 8);
        lo[0] *= inv * bf16lo(w0); lo[1] *= inv * bf16hi(w0); lo[2] *= inv * bf16lo(w1); lo[3] *= inv * bf16hi(w1);
        hi[0] *= inv * bf16lo(w2); hi[1] *= inv * bf16hi(w2); hi[2] *= inv * bf16lo(w3); hi[3] *= inv * bf16hi(w3);
      }
      // rotate-half: dim d < HD/2 pairs with d + HD/2
      const float2 c0 = *reinterpret_cast<const float2*>(a.cos_t + ci + ks * 16 + tq * 2);
      const float2 c1 = *reinterpret_cast<const float2*>(a.cos_t + ci + ks * 16 + tq * 2 + 8);
      const float2 s0 = *reinterpret_cast<const float2*>(a.sin_t + ci + ks * 16 + tq * 2);
      const float2 s1 = *reinterpret_cast<const float2*>(a.sin_t + ci + ks * 16 + tq * 2 + 8);
      const float cs[4] = {c0.x, c0.y, c1.x, c1.y}, sn[4] = {s0.x, s0.y, s1.x, s1.y};
      float rl[4], rh[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        rl[e] = (lo[e] * cs[e] - hi[e] * sn[e]) * sc;
        rh[e] = (hi[e] * cs[e] + lo[e] * sn[e]) * sc;
      }
      fm_split(rl[0], rl[1], qf[ks][0], qf[ks][1]);
      fm_split(rl[2], rl[3], qf[ks][2], qf[ks][3]);
      fm_split(rh[0], rh[1], qf[ks + KS / 2][0], qf[ks + KS / 2][1]);
      fm_split(rh[2], rh[3], qf[ks + KS / 2][2], qf[ks + KS / 2][3]);
    }
    // the new k / v row: (norm +) RoPE in the 8-dims-per-lane layout, by warp 0 of the CTA whose
    // slice ends with it
    if (in_cache && pos >= k0 && pos < k1) {
      pos_own = pos;
      if (warp == 0) {
        constexpr int LPK = HD / 8, HL = LPK / 2;
        const int dl = lane % LPK;
        const bool hi = dl >= HL;
        const float* ks_ = sq + G * HD + dl * 8;
        const float4 x0 = reinterpret_cast<const float4*>(ks_)[0];
        const float4 x1 = reinterpret_cast<const float4*>(ks_)[1];
        float kx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        if (ph.kn_w != nullptr) {
          float ss = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) ss = fmaf(kx[e], kx[e], ss);
#pragma unroll
          for (int o2 = LPK / 2; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
          const float inv = rsqrtf(ss / (float)HD + a.eps);
          float w[8];
          unpack8(*reinterpret_cast<const uint4*>(ph.kn_w + dl * 8), w);
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
        const float4* vp = reinterpret_cast<const float4*>(sq + (G + 1) * HD + dl * 8);
        const float4 v0 = vp[0], v1 = vp[1];
        newk.x = pack_bf16(kr[0], kr[1]); newk.y = pack_bf16(kr[2], kr[3]);
        newk.z = pack_bf16(kr[4], kr[5]); newk.w = pack_bf16(kr[6], kr[7]);
        newv.x = pack_bf16(v0.x, v0.y); newv.y = pack_bf16(v0.z, v0.w);
        newv.z = pack_bf16(v1.x, v1.y); newv.w = pack_bf16(v1.z, v1.w);
        if (lane < LPK) {
          const size_t row = (size_t)kvh * a.head_stride + (size_t)pos * a.row_stride + dl * 8;
          *reinterpret_cast<uint4*>(const_cast<uint16_t*>(ph.kc) + row) = newk;
          *reinterpret_cast<uint4*>(const_cast<uint16_t*>(ph.vc) + row) = newv;
        }
      }
    }
  }

  for (int t = 0; t < ntiles; ++t) {                     // ntiles is CTA-uniform
    fm_wait<1>();                    // tile t has landed (at most tile t + 1 still in flight)
    __syncthreads();                 // ... for every thread, and everyone is done with tile t - 1
    if (t + 2 < ntiles) load_tile(t + 2);
    fm_commit();
    const uint32_t sk = stage(t), sv = sk + TILE;
    const int row0 = k0 + t * kFmTile;
    if (pos_own >= row0 && pos_own < row0 + kFmTile) {   // CTA-uniform
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
    const int key0 = row0 + kg * 16;                     // this warp pair's 16 keys
    if (key0 >= k1) continue;                            // warp-uniform
    // ---- S = Q K^T : 16 rows x 16 keys (both warps of the pair) ----
    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t b0, b1, b2, b3;
      const int key = kg * 16 + ((lane >> 4) << 3) + (lane & 7);
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
    float pr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pr[e] = exp2f(sv4[e] - mu);
    l = l * corr + (pr[0] + pr[1]) + (pr[2] + pr[3]);
    uint32_t pf[4];                  // P as the A fragment of one k16 step: rows g / g + 8 = hi / lo
    fm_split(pr[0], pr[1], pf[0], pf[1]);
    fm_split(pr[2], pr[3], pf[2], pf[3]);
#pragma unroll
    for (int d = 0; d < DH; ++d) { o[d][0] *= corr; o[d][1] *= corr; o[d][2] *= corr; o[d][3] *= corr; }
    // ---- O += P V for this warp's half of the head dim ----
#pragma unroll
    for (int d2 = 0; d2 < DH / 2; ++d2) {
      uint32_t b0, b1, b2, b3;
      const int key = kg * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
      const int c = (half * (DH / 2) + d2) * 2 + (lane >> 4);
      fm_ldsm_t(sv + fm_swz<HD>(key, c), b0, b1, b2, b3);
      fm_mma(o[d2 * 2], pf, b0, b1);
      fm_mma(o[d2 * 2 + 1], pf, b2, b3);
    }
  }
  fm_wait<0>();
  __syncthreads();                   // the borrowed areas are free again

  // restart the weight stream behind this phase; it runs while the records are merged
  cur.p = p + 1;
  dl_seek(cur, a, win, warp, lane);
#pragma unroll
  for (int i = 0; i < kDlRing; ++i) dl_issue(cur, a, win, ring_lane, warp, lane);

  if (!active) return cur;           // CTA-uniform
  // ---- one record per 16-key group, in the vector staging area ----
  float* srec = reinterpret_cast<float*>(smem);
  float* sw = srec + NREC * REC;
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (g < G) {
    float* r = srec + kg * REC;
#pragma unroll
    for (int d = 0; d < DH; ++d)
      *reinterpret_cast<float2*>(r + g * HD + (half * DH + d) * 8 + tq * 2) =
          make_float2(o[d][0] + o[d][2], o[d][1] + o[d][3]);
    if (tq == 0 && half == 0) { r[G * HD + g] = m; r[G * HD + G + g] = l; }
  }
  FdArgs fa{};
  fa.out = ph.yp; fa.out_dtype = kFdOutPairs; fa.tag = dl_tag(epoch, a.n_phases, p);
  fa.counters = a.fd_counters; fa.recs = a.fd_recs; fa.n_splits = a.n_splits;
  fd_finish<HD, G, kDlThreads, NREC>(fa, srec, sw, kvh, split);
  return cur;
}

template <int HD, int G>
__global__ void __launch_bounds__(kDlThreads, 1) decode_layers_kernel(const __grid_constant__ DlArgs a) {
  extern __shared__ __align__(128) unsigned char dl_smem[];
  __shared__ __align__(16) DlPhase win[kDlWin];
  float* xs = reinterpret_cast<float*>(dl_smem);
  float* part = reinterpret_cast<float*>(dl_smem + kDlXsBytes + kDlRingBytes);
  float* red = part + kDlMaxRows * kDlWarps;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t ring_lane = smem_u32(dl_smem) + kDlXsBytes + warp * kDlWarpRing + lane * 16;

  // this launch's number: every CTA reads it before CTA 0 can possibly have finished (CTA 0
  // needs every other CTA's rows to get there)
  const unsigned epoch = *reinterpret_cast<const volatile unsigned*>(a.epoch);
  {
    constexpr int W = sizeof(DlPhase) / 4;
    const int n = min(kDlAhead, a.n_phases) * W;
    for (int i = threadIdx.x; i < n; i += kDlThreads)
      reinterpret_cast<uint32_t*>(win)[i] = reinterpret_cast<const uint32_t*>(a.phases)[i];
  }
  __syncthreads();

  DlStream st;
  st.cur.p = 0; st.cur.issued = 0; st.cur.base = nullptr;
  st.consumed = 0;
  dl_seek(st.cur, a, win, warp, lane);
#pragma unroll
  for (int i = 0; i < kDlRing; ++i) dl_issue(st.cur, a, win, ring_lane, warp, lane);

  for (int p = 0; p < a.n_phases; ++p) {
    if (dl_ph(win, p).type() == DL_GEMV) st = dl_gemv(a, win, st, epoch, xs, part, red, ring_lane, p);
    else st.cur = dl_attention<HD, G>(a, win, st.cur, epoch, p, dl_smem, ring_lane);
  }
  dl_wait_group<0>();
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(a.epoch, 1u);
}

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_decode_layers_plan_bytes(int n_layers) {
  return n_layers > 0 ? (int64_t)n_layers * 5 * (int64_t)sizeof(DlPhase) : 0;
}

namespace {
// Layout of the synchronisation workspace: the launch counter, then the pair vectors the phases
// hand to one another (hidden state, q|k|v row, attention output, MLP activation).
struct DlWorkspace {
  size_t h, qkv, attn, act, bytes;
};
DlWorkspace dl_workspace(int hidden, int q_size, int kv_size, int inter) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  DlWorkspace w;
  w.h = 256;
  w.qkv = w.h + up((size_t)hidden * 8);
  w.attn = w.qkv + up((size_t)(q_size + 2 * kv_size) * 8);
  w.act = w.attn + up((size_t)q_size * 8);
  w.bytes = w.act + up((size_t)inter * 8);
  return w;
}
}  // namespace

extern "C" int64_t b200_decode_layers_sync_bytes(int hidden, int q_size, int kv_size, int inter) {
  if (hidden <= 0 || q_size <= 0 || kv_size <= 0 || inter <= 0) return 0;
  return (int64_t)dl_workspace(hidden, q_size, kv_size, inter).bytes;
}

extern "C" int b200_decode_layers_plan(void* plan_dev, void* sync_ws, int n_layers,
                                       const void* const* w_qkv, const void* const* w_o,
                                       const void* const* w_gu, const void* const* w_down,
                                       const void* const* ln1, const void* const* ln2,
                                       const void* const* kcache, const void* const* vcache,
                                       const void* const* qn_w, const void* const* kn_w, float* h,
                                       int hidden, int q_size, int kv_size, int inter, int tp_ctx) {
  if (!plan_dev || !sync_ws || n_layers <= 0 || !w_qkv || !w_o || !w_gu || !w_down || !ln1 || !ln2 ||
      !kcache || !vcache || !h)
    return B200_ERR_ARG;
  if ((qn_w == nullptr) != (kn_w == nullptr)) return B200_ERR_ARG;
  if (hidden <= 0 || q_size <= 0 || kv_size <= 0 || inter <= 0) return B200_ERR_SHAPE;
  if ((hidden & 255) || (q_size & 255) || (inter & 255) || hidden > kDlMaxK || q_size > kDlMaxK ||
      inter > kDlMaxK)
    return B200_ERR_SHAPE;
  if (((uintptr_t)sync_ws & 255) != 0 || ((uintptr_t)h & 15) != 0) return B200_ERR_ALIGN;
  const TpLink* link = nullptr;
  if (tp_ctx >= 0) {
    link = tp_link_get(tp_ctx);
    if (link == nullptr) return B200_ERR_ARG;
    if (link->H != hidden) return B200_ERR_SHAPE;
  }
  const bool tp = link != nullptr;
  const bool lead = !tp || link->rank == 0;
  auto rows_per_cta = [](int N, bool even) {
    int rpc = (N + kNumSMs - 1) / kNumSMs;
    if (even && (rpc & 1)) ++rpc;
    return rpc;
  };
  const int n_qkv = q_size + 2 * kv_size;
  const int rpc_qkv = rows_per_cta(n_qkv, false), rpc_h = rows_per_cta(hidden, false),
            rpc_gu = rows_per_cta(2 * inter, true);
  if (rpc_qkv > kDlMaxRows || rpc_h > kDlMaxRows || rpc_gu > kDlMaxRows) return B200_ERR_SHAPE;
  const DlWorkspace ws = dl_workspace(hidden, q_size, kv_size, inter);
  uint2* p_h = (uint2*)((char*)sync_ws + ws.h);
  uint2* p_qkv = (uint2*)((char*)sync_ws + ws.qkv);
  uint2* p_attn = (uint2*)((char*)sync_ws + ws.attn);
  uint2* p_act = (uint2*)((char*)sync_ws + ws.act);
  auto flags = [](int type, int in, int epi) { return type | (in << 4) | (epi << 8); };

  std::vector<DlPhase> t((size_t)n_layers * 5);
  for (int i = 0; i < n_layers; ++i) {
    for (const void* q : {w_qkv[i], w_o[i], w_gu[i], w_down[i], kcache[i], vcache[i]})
      if (q == nullptr || ((uintptr_t)q & 15) != 0) return B200_ERR_ALIGN;
    if (!ln1[i] || !ln2[i]) return B200_ERR_ARG;
    if (qn_w && (!qn_w[i] || !kn_w[i])) return B200_ERR_ARG;
    DlPhase* ph = &t[(size_t)i * 5];
    for (int k = 0; k < 5; ++k) { ph[k] = DlPhase{}; ph[k].tp_in = ph[k].tp_out = ph[k].resid_tp = -1; }
    // q|k|v = W_qkv rmsnorm(h)
    ph[0].w = (const uint16_t*)w_qkv[i]; ph[0].norm_w = (const uint16_t*)ln1[i];
    ph[0].yp = p_qkv; ph[0].N = n_qkv; ph[0].K = hidden; ph[0].rpc = rpc_qkv;
    if (i == 0) { ph[0].flags = flags(DL_GEMV, DL_IN_PLAIN, B200_EPI_NONE); ph[0].x = h; }
    else if (tp) { ph[0].flags = flags(DL_GEMV, DL_IN_TP, B200_EPI_NONE); ph[0].tp_in = 2 * i - 1; }
    else { ph[0].flags = flags(DL_GEMV, DL_IN_PAIRS, B200_EPI_NONE); ph[0].xp = p_h; }
    // attention over the cache (+ RoPE / QK-norm / append of the new row)
    ph[1].flags = flags(DL_ATT, DL_IN_PAIRS, B200_EPI_NONE);
    ph[1].kc = (const uint16_t*)kcache[i]; ph[1].vc = (const uint16_t*)vcache[i];
    ph[1].qn_w = qn_w ? (const uint16_t*)qn_w[i] : nullptr;
    ph[1].kn_w = kn_w ? (const uint16_t*)kn_w[i] : nullptr;
    ph[1].xp = p_qkv; ph[1].yp = p_attn;
    // h += W_o attn
    ph[2].flags = flags(DL_GEMV, DL_IN_PAIRS, B200_EPI_NONE);
    ph[2].w = (const uint16_t*)w_o[i]; ph[2].xp = p_attn; ph[2].N = hidden; ph[2].K = q_size;
    ph[2].rpc = rpc_h;
    if (tp) {
      ph[2].tp_out = 2 * i;
      if (lead) { if (i == 0) ph[2].resid = h; else ph[2].resid_tp = 2 * i - 1; }
    } else {
      ph[2].y = h; ph[2].yp = p_h; ph[2].resid = h;
    }
    // act = swiglu(W_gu rmsnorm(h))
    ph[3].w = (const uint16_t*)w_gu[i]; ph[3].norm_w = (const uint16_t*)ln2[i];
    ph[3].yp = p_act; ph[3].N = 2 * inter; ph[3].K = hidden; ph[3].rpc = rpc_gu;
    if (tp) { ph[3].flags = flags(DL_GEMV, DL_IN_TP, B200_EPI_SWIGLU); ph[3].tp_in = 2 * i; }
    else { ph[3].flags = flags(DL_GEMV, DL_IN_PAIRS, B200_EPI_SWIGLU); ph[3].xp = p_h; }
    // h += W_down act
    ph[4].flags = flags(DL_GEMV, DL_IN_PAIRS, B200_EPI_NONE);
    ph[4].w = (const uint16_t*)w_down[i]; ph[4].xp = p_act; ph[4].N = hidden; ph[4].K = inter;
    ph[4].rpc = rpc_h;
    if (tp) {
      ph[4].tp_out = 2 * i + 1;
      if (lead) ph[4].resid_tp = 2 * i;
    } else {
      ph[4].y = h; ph[4].yp = p_h; ph[4].resid = h;
    }
  }
  return cudaMemcpy(plan_dev, t.data(), t.size() * sizeof(DlPhase), cudaMemcpyHostToDevice) ==
                 cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

template <int HD, int G>
static cudaError_t dl_launch(const DlArgs& a, cudaStream_t st) {
  static bool attr_set[kMaxDevices] = {false};
  cudaError_t e = opt_in_smem(decode_layers_kernel<HD, G>, kDlSmemBytes, attr_set);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kNumSMs);
  cfg.blockDim = dim3(kDlThreads);
  cfg.dynamicSmemBytes = kDlSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_layers_kernel<HD, G>, a);
}

extern "C" int b200_decode_layers(const void* plan_dev, int n_layers, const float* cos_t,
                                  const float* sin_t, const int* kv_len_dev, void* fd_workspace,
                                  void* sync_ws, int n_q, int n_kv, int hd, int64_t kv_head_stride,
                                  int64_t kv_row_stride, int max_seq, int n_splits, float scale,
                                  float eps, int tp_ctx, int* status, int flags,
                                  b200_stream_t stream) {
  (void)flags;
  if (!plan_dev || !cos_t || !sin_t || !kv_len_dev || !fd_workspace || !sync_ws || !status)
    return B200_ERR_ARG;
  if (n_layers <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_splits <= 0 || max_seq <= 0 ||
      n_kv * n_splits > kNumSMs)
    return B200_ERR_SHAPE;
  if ((kv_row_stride & 7) != 0 || (kv_head_stride & 7) != 0 ||
      ((uintptr_t)fd_workspace & 15) != 0 || ((uintptr_t)cos_t & 15) != 0 ||
      ((uintptr_t)sin_t & 15) != 0 || ((uintptr_t)sync_ws & 255) != 0 ||
      ((uintptr_t)plan_dev & 15) != 0)
    return B200_ERR_ALIGN;
  DlArgs a{};
  a.phases = (const DlPhase*)plan_dev; a.n_phases = n_layers * 5;
  a.cos_t = cos_t; a.sin_t = sin_t; a.kv_len = kv_len_dev;
  a.fd_counters = (int*)fd_workspace;
  a.fd_recs = (float*)((char*)fd_workspace + (((size_t)n_kv * 4 + 255) & ~(size_t)255));
  a.n_q = n_q; a.n_kv = n_kv; a.n_splits = n_splits; a.max_seq = max_seq;
  a.head_stride = kv_head_stride; a.row_stride = kv_row_stride;
  a.scale_log2 = scale * 1.4426950408889634f; a.eps = eps;
  a.epoch = (unsigned*)sync_ws; a.wait_ticks = wait_ticks_from_tuning(); a.status = status;
  if (tp_ctx >= 0) {
    const TpLink* link = tp_link_get(tp_ctx);
    if (link == nullptr) return B200_ERR_ARG;
    a.tp = *link;
    a.tp.wait_ticks = a.wait_ticks;
  }
  const int G = n_q / n_kv;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
#define DL_CASE(HD_, G_) if (hd == HD_ && G == G_) e = dl_launch<HD_, G_>(a, st); else
  DL_CASE(128, 1) DL_CASE(128, 2) DL_CASE(128, 4) DL_CASE(128, 8)
  DL_CASE(64, 1) DL_CASE(64, 2) DL_CASE(64, 4) DL_CASE(64, 8)
  return B200_ERR_SHAPE;
#undef DL_CASE
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
