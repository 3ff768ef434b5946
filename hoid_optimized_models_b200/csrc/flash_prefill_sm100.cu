// Prefill / encoder flash attention on the sm_100a tensor cores (tcgen05 + TMEM + TMA).
//
// Persistent: one CTA per SM walks a list of work items.  An item is 256 query rows of one head,
// handled as two independent streams A and B of 128 rows that share the K / V tiles, so the
// latencies of one stream (score load, barrier hand-overs, MMA completion) are covered by the
// exponentials of the other.  Ten warps:
//   warps 0-3  softmax of stream A, warps 4-7 of stream B: ONE thread per query row (= TMEM
//              lane; warp w may only touch lanes 32 (w % 4) ..).  A thread pulls its whole row
//              of 128 scores with tcgen05.ld, takes the row maximum and sum in registers (no
//              exchange between threads), and writes P = exp2(...) as packed bf16 back into
//              tensor memory: over the first 64 columns of the scores it has just consumed at
//              head dim 128 (S_A, S_B, O_A, O_B fill the 512 columns), into 64 columns of its
//              own at head dim 64, where the next tile's scores are then issued as soon as the
//              current ones are in registers instead of after the O MMA that reads P.
//   warp 8     TMA producer: Q tiles per item and stream, K and V tiles into one ring
//   warp 9     MMA issuer (one lane): S_X = Q_X K^T (M128 N128, K = head dim) into the stream's
//              score accumulator, and O_X += P_X V with P read straight from tensor memory and V
//              consumed in its natural [key][dim] layout as an MN-major operand.
// The output accumulates in tensor memory across key tiles.  The running maximum is raised only
// when a row's tile maximum exceeds it by more than 2^8 (exact after the final division by the
// row sum; P stays within bf16 range), and only then is the row of O rescaled in place, so most
// tiles never touch O.  Scores and probabilities never leave the SM.
// Work order: causal items heaviest first, dealt to the CTAs in alternating direction so every
// CTA gets the same number of key tiles to within one round; bidirectional items with the query
// blocks of one head adjacent, so a head's K / V come from DRAM once and from L2 afterwards.
// Causal tiles above the diagonal are never visited.  Every mbarrier wait is bounded (status
// word + clean TMEM release on expiry).
#include <algorithm>
#include <climits>

#include "sm100.cuh"

namespace b200 {

constexpr int FA_BM = 128, FA_BN = 128;
constexpr int kFaThreads = 320;              // 8 softmax warps, TMA warp, MMA warp
constexpr uint32_t kAtomBytes = 128 * 128;   // a 128-row x 64-column bf16 box: 16 KiB
constexpr float kFaLazy = 8.f;               // log2 of the growth of a row maximum that is tolerated

struct FaArgs {
  uint16_t* o; long o_bs, o_rs, o_hs;
  int* status;
  int S, kv_len, q_pos0, group, causal, n_q;
  int n_mp, n_bh, n_items;          // 256-row query blocks per head, batch x heads, work items
  // row / column bookkeeping of the 2D views the tensor maps cover
  int q_batch_rows, q_head_rows, q_head_cols;
  int k_batch_rows, k_head_rows, k_head_cols;
  int v_batch_rows, v_head_rows, v_head_cols;
  float scale_log2;
};

// One work item: key-tile counts of the two streams (n[1] == 0: the item has no rows for B).
struct FaItem { int b, head, m0, n[2], nt; };

// The work item of this CTA in round r (false: the round has none for it).  All roles call
// this with the same arguments and therefore walk identical lists.
__device__ __forceinline__ bool fa_item(const FaArgs& a, int r, FaItem& it) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const int w = r * G + ((a.causal && (r & 1)) ? G - 1 - c : c);
  if (w >= a.n_items) return false;
  int mp, bh;
  if (a.causal) { mp = a.n_mp - 1 - w / a.n_bh; bh = w % a.n_bh; }
  else { mp = w % a.n_mp; bh = w / a.n_mp; }
  it.head = bh % a.n_q;
  it.b = bh / a.n_q;
  it.m0 = mp * 2 * FA_BM;
  int kv0 = a.kv_len, kv1 = a.kv_len;
  if (a.causal) {
    kv0 = min(kv0, a.q_pos0 + it.m0 + FA_BM);
    kv1 = min(kv1, a.q_pos0 + it.m0 + 2 * FA_BM);
  }
  it.n[0] = (kv0 + FA_BN - 1) / FA_BN;             // >= 1: kv_len >= 1 and q_pos0 >= 0
  it.n[1] = it.m0 + FA_BM < a.S ? (kv1 + FA_BN - 1) / FA_BN : 0;
  it.nt = max(it.n[0], it.n[1]);
  return true;
}

// Position in the flat sequence of key tiles of all my items.
struct FaCursor {
  int r, j;          // round of the item, key tile inside it
  int e;             // ring entry of the tile's K (its V is e + 1) = 2 x the flat tile index
  bool valid;
  FaItem it;
};
__device__ __forceinline__ void fa_cursor_next_item(const FaArgs& a, int n_rounds, FaCursor& c) {
  c.j = 0;
  do { ++c.r; } while (c.r < n_rounds && !fa_item(a, c.r, c.it));
  c.valid = c.r < n_rounds;
}
__device__ __forceinline__ void fa_cursor_init(const FaArgs& a, int n_rounds, FaCursor& c) {
  c.r = -1; c.e = 0;
  fa_cursor_next_item(a, n_rounds, c);
}
__device__ __forceinline__ void fa_cursor_advance(const FaArgs& a, int n_rounds, FaCursor& c) {
  c.e += 2;
  if (++c.j == c.it.nt) fa_cursor_next_item(a, n_rounds, c);
}

// sm_100 arithmetic that halves the instruction count of the softmax inner loops: three-input
// max, and fp32 add / fma on register pairs.
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t fa_pair(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void fa_unpair(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fa_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fa_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Bounded wait without an abort flag, for the teardown of a role that already gave up.
__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity, long long ticks) {
  const long long t0 = clock64();
  while (!mbar_try(bar, parity) && clock64() - t0 < ticks) {}
}

// UMMA descriptor for an MN-major, 128-byte-swizzled operand: 64 contiguous MN elements per
// 128-byte row, rows = K index; 8-row groups SBO bytes apart, 64-element MN blocks LBO apart.
__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint64_t umma_desc_k(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> fp32, M = 128; b_major: 0 = K-major, 1 = MN-major
constexpr uint32_t fa_idesc(int n, int b_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// One key tile of one query row: scores from tensor memory -> row maximum -> (rarely) rescale of
// the output accumulator -> P = exp2(.) as packed bf16 back to tensor memory -> hand-over.
// By itself (one warp per scheduler, nothing else running) this body takes ~1500 clocks per tile,
// 1024 of them the 128 exponentials at 8 clocks each on the special-function unit.  Measured and
// rejected: reading the row from tensor memory twice, 32 columns at a time, to halve the registers
// held (no faster by itself, slower in the kernel); a quarter or half of the exponentials as a
// cubic on the FMA pipe (12 % faster by itself at a quarter, no gain in the kernel, where the
// stream's MMAs and hand-overs are the other half of the period).
struct FaRowState { float m_used, l_run; int ok; };

template <int HD, bool SEP>
__device__ __forceinline__ FaRowState fa_softmax_tile(uint32_t my_s, uint32_t my_p, uint32_t my_o,
                                                   float scale_log2, float m_used, float l_run,
                                                   int first, int valid, uint32_t bar_cf,
                                                   uint32_t bar_of, uint32_t of_parity,
                                                   uint32_t bar_pf, volatile int* abort_flag) {
  const int lane = threadIdx.x & 31;
  FaRowState st;
  st.ok = 0;
  auto ex2 = [](float v) -> float {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(v));
    return y;
  };
  uint32_t sr[FA_BN];                            // the row's scores (fp32 bit patterns)
#pragma unroll
  for (int c = 0; c < FA_BN / 32; ++c) tc_ld32(my_s + c * 32, sr + c * 32);
  tc_wait_ld();
  if (SEP) {   // the scores are in registers: the tensor core may start on the next tile's
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_cf);
  }
#define SV(i) __uint_as_float(sr[i])
  // only the last tile(s) need masking: end of the keys, or the causal diagonal
  if (valid < FA_BN) {
#pragma unroll
    for (int i = 0; i < FA_BN; ++i) sr[i] = (i < valid) ? sr[i] : 0xff800000u;   // -inf
  }
  float mx[4] = {SV(0), SV(1), SV(2), SV(3)};
#pragma unroll
  for (int i = 4; i < FA_BN - 4; i += 8) {
    mx[0] = fa_max3(mx[0], SV(i), SV(i + 1)); mx[1] = fa_max3(mx[1], SV(i + 2), SV(i + 3));
    mx[2] = fa_max3(mx[2], SV(i + 4), SV(i + 5)); mx[3] = fa_max3(mx[3], SV(i + 6), SV(i + 7));
  }
  mx[0] = fa_max3(mx[0], SV(FA_BN - 4), SV(FA_BN - 3));
  mx[1] = fa_max3(mx[1], SV(FA_BN - 2), SV(FA_BN - 1));
  const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;
  if (first) {
    m_used = (mt == -INFINITY) ? 0.f : mt;
  } else if (__any_sync(0xffffffffu, mt > m_used + kFaLazy)) {
    // Some row of this warp outgrew its reference maximum: rescale the warp's rows of O
    // (in tensor memory) once the tensor core has finished the previous tile's O.
    // (waits are voted on so that the warp-collective tensor-memory accesses stay convergent)
    if (!__all_sync(0xffffffffu, mbar_wait(bar_of, of_parity, abort_flag))) return st;
    tc_fence_after();
    const float m_new = fmaxf(m_used, mt);
    const float f = ex2(m_used - m_new);
#pragma unroll
    for (int c = 0; c < HD / 16; ++c) {
      uint32_t rr[16];
      tc_ld16(my_o + c * 16, rr);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * f);
      tc_st16(my_o + c * 16, rr);
    }
    l_run *= f;
    m_used = m_new;
  }
  if (SEP && !first) {
    // P has columns of its own here: the previous tile's O MMA must be done reading them.
    // It was issued a tile of exponentials ago, so this does not normally spin.  (A second
    // wait on the phase the rescale above may have waited for is safe: the barrier cannot
    // move on before this warp's next arrival.)
    if (!__all_sync(0xffffffffu, mbar_wait(bar_of, of_parity, abort_flag))) return st;
  }
  // p = exp2(s * scale - m) as packed bf16 pairs, row sum in fp32; 64 keys at a time so
  // that the first half is on its way to tensor memory while the second is computed
  const uint64_t sc2 = fa_pair(scale_log2, scale_log2), nm2 = fa_pair(-m_used, -m_used);
  uint64_t ps2[2] = {0ull, 0ull};                 // two pairs of partial row sums
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t pk[32];
#pragma unroll
    for (int i = 0; i < 64; i += 4) {
      float t0, t1, t2, t3;
      fa_unpair(fa_fma2(fa_pair(SV(h * 64 + i), SV(h * 64 + i + 1)), sc2, nm2), t0, t1);
      fa_unpair(fa_fma2(fa_pair(SV(h * 64 + i + 2), SV(h * 64 + i + 3)), sc2, nm2), t2, t3);
      const float p0 = ex2(t0), p1 = ex2(t1), p2 = ex2(t2), p3 = ex2(t3);
      ps2[0] = fa_add2(ps2[0], fa_pair(p0, p1));
      ps2[1] = fa_add2(ps2[1], fa_pair(p2, p3));
      pk[i / 2] = pack_bf16(p0, p1);
      pk[i / 2 + 1] = pack_bf16(p2, p3);
    }
    tc_st32(my_p + h * 32, pk);
  }
#undef SV
  {
    float s0, s1, s2, s3;
    fa_unpair(ps2[0], s0, s1);
    fa_unpair(ps2[1], s2, s3);
    l_run += (s0 + s1) + (s2 + s3);
  }
  tc_wait_st();
  // hand P (and a possibly rescaled O) to the tensor core: one arrival per warp
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar_pf);
  st.m_used = m_used; st.l_run = l_run; st.ok = 1;
  return st;
}

template <int HD>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, FaArgs a) {
  constexpr int ATOMS = HD / 64;                        // 64-column boxes per operand tile
  constexpr int NQ = HD == 64 ? 2 : 1;                  // Q buffers per stream
  constexpr int NR = HD == 64 ? 8 : 5;                  // ring entries (a K tile or a V tile each)
  constexpr uint32_t kTile = ATOMS * kAtomBytes;        // Q / K / V tile bytes
  constexpr uint32_t kTiles = (2 * NQ + NR) * kTile;    // 192 KiB at head dim 64, 224 KiB at 128
  // barrier indices: Q full / empty per (buffer, stream), ring full / empty, and per stream
  // S ready, P ready, O ready
  constexpr int QF = 0, QE = 2 * NQ, RF = 4 * NQ, RE = 4 * NQ + NR, SF = 4 * NQ + 2 * NR,
                PF = SF + 2, OF = SF + 4, CF = SF + 6, NBAR = SF + 8;
  // At head dim 64 tensor memory has room for P beside S, so a stream's next scores can be
  // computed as soon as its softmax warps have pulled the current ones into registers.
  constexpr bool SEP = HD == 64;
  static_assert(NBAR <= 32, "barrier block is 32 entries");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // Operand tiles need 1024-byte alignment.  The dynamic window starts 1 KB into the CTA's
  // shared memory (after the system-reserved kilobyte) and is therefore aligned; if a future
  // toolchain breaks that assumption the kernel reports it instead of corrupting tiles.
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, B200_ERR_ALIGN);
    return;
  }
  const uint32_t sQ = base;                             // [NQ][2 streams]
  const uint32_t sR = sQ + 2 * NQ * kTile;              // NR ring entries
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + kTiles);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rounds = (a.n_items + (int)gridDim.x - 1) / (int)gridDim.x;

  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < NBAR; ++i) mbar_init(bar(i), (i >= PF && i < PF + 2) || (i >= CF && i < CF + 2) ? 4 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S_A 0..127, S_B 128..255, O_A, O_B from 256; P_X (64 columns of packed bf16)
  // from 384 at head dim 64, else over the first 64 columns of S_X
  auto tS = [&](int x) { return tmem_base + (uint32_t)x * FA_BN; };
  auto tO = [&](int x) { return tmem_base + 256u + (uint32_t)x * HD; };
  auto tP = [&](int x) { return SEP ? tmem_base + 384u + (uint32_t)x * 64 : tS(x); };

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int qn[2] = {0, 0};          // Q tiles loaded so far, per stream
      int e = 0;                   // ring entries issued so far
      bool ok = true;
      for (int r = 0; r < n_rounds && ok; ++r) {
        FaItem it;
        if (!fa_item(a, r, it)) continue;
        const int kvh = it.head / a.group;
        const int q_col = it.head * a.q_head_cols;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (it.n[x] == 0 || !ok) continue;
          const int qb = qn[x] % NQ, bi = qb * 2 + x;
          if (!mbar_wait(bar(QE + bi), ((qn[x] / NQ) & 1) ^ 1, abort_flag)) { ok = false; continue; }
          const int q_row = it.b * a.q_batch_rows + it.head * a.q_head_rows + it.m0 + x * FA_BM;
          mbar_expect_tx(bar(QF + bi), kTile);
#pragma unroll
          for (int t = 0; t < ATOMS; ++t)
            tma_load_2d(sQ + bi * kTile + t * kAtomBytes, &map_q, bar(QF + bi), q_col + 64 * t, q_row);
          ++qn[x];
        }
        const int k_row0 = it.b * a.k_batch_rows + kvh * a.k_head_rows, k_col = kvh * a.k_head_cols;
        const int v_row0 = it.b * a.v_batch_rows + kvh * a.v_head_rows, v_col = kvh * a.v_head_cols;
        for (int j = 0; j < it.nt && ok; ++j) {
#pragma unroll
          for (int kv = 0; kv < 2; ++kv, ++e) {
            if (!ok) continue;
            const int slot = e % NR;
            if (!mbar_wait(bar(RE + slot), ((e / NR) & 1) ^ 1, abort_flag)) { ok = false; continue; }
            mbar_expect_tx(bar(RF + slot), kTile);
#pragma unroll
            for (int t = 0; t < ATOMS; ++t) {
              if (kv == 0)
                tma_load_2d(sR + slot * kTile + t * kAtomBytes, &map_k, bar(RF + slot), k_col + 64 * t, k_row0 + j * FA_BN);
              else
                tma_load_2d(sR + slot * kTile + t * kAtomBytes, &map_v, bar(RF + slot), v_col + 64 * t, v_row0 + j * FA_BN);
            }
          }
        }
      }
      if (!ok) {
        // give the copies still in flight a bounded time to land before the CTA retires
        for (int i = 1; i <= min(e, NR); ++i)
          mbar_wait_quiet(bar(RF + (e - i) % NR), ((e - i) / NR) & 1, 2000000);
        for (int x = 0; x < 2; ++x)
          for (int i = 1; i <= min(qn[x], NQ); ++i)
            mbar_wait_quiet(bar(QF + ((qn[x] - i) % NQ) * 2 + x), ((qn[x] - i) / NQ) & 1, 2000000);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = fa_idesc(FA_BN, 0);
      constexpr uint32_t idesc_o = fa_idesc(HD, 1);
      // Two positions in the flat tile sequence: `pv` is the tile whose O += P V is issued,
      // `ps` the tile whose S = Q K^T is issued, one tile further on (across item boundaries),
      // so a stream's next scores are being computed while its softmax warps work.
      FaCursor pv, ps;
      fa_cursor_init(a, n_rounds, pv);
      ps = pv;
      int sq[2] = {0, 0};         // Q tiles consumed, per stream
      int pg[2] = {0, 0};         // O tiles issued, per stream
      int k_seen = -1;            // ring entry of the last K tile whose arrival was awaited
      bool ok = pv.valid;
      // 1 issued, 0 operands not there yet (only when !blocking), -1 gave up
      auto issue_s = [&](int x, bool blocking) -> int {
        const int qb = sq[x] % NQ, bi = qb * 2 + x, slot = ps.e % NR;
        const bool new_q = ps.j == 0;
        if (!blocking) {
          if (new_q && !mbar_try(bar(QF + bi), (sq[x] / NQ) & 1)) return 0;
          if (k_seen != ps.e && !mbar_try(bar(RF + slot), (ps.e / NR) & 1)) return 0;
        } else {
          if (new_q && !mbar_wait(bar(QF + bi), (sq[x] / NQ) & 1, abort_flag)) return -1;
          if (k_seen != ps.e && !mbar_wait(bar(RF + slot), (ps.e / NR) & 1, abort_flag)) return -1;
        }
        k_seen = ps.e;
        tc_fence_after();
        const uint32_t sk = sR + slot * kTile, sq_ = sQ + bi * kTile;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
          tc_mma(tS(x), umma_desc_k(sq_ + off), umma_desc_k(sk + off), idesc_s, k != 0 ? 1u : 0u);
        }
        tc_commit(bar(SF + x));
        if (ps.j == ps.it.n[x] - 1) { tc_commit(bar(QE + bi)); ++sq[x]; }   // Q free once these retire
        return 1;
      };
      auto issue_pv = [&](int x) -> bool {
        const int slot = (pv.e + 1) % NR;
        if (!mbar_wait(bar(PF + x), pg[x] & 1, abort_flag)) return false;
        if (!mbar_wait(bar(RF + slot), ((pv.e + 1) / NR) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sv = sR + slot * kTile;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          // A = P from tensor memory: 16 keys = 8 columns of packed bf16 pairs
          // B = V (MN-major over dims): 16 keys = two 8-row groups = 2048 bytes
          const uint64_t db = umma_desc_mn(sv + k * 2048, kAtomBytes, 1024);
          tc_mma_ts(tO(x), tP(x) + k * 8, db, idesc_o, (pv.j != 0 || k != 0) ? 1u : 0u);
        }
        tc_commit(bar(OF + x));
        ++pg[x];
        return true;
      };
      if (ok) {      // scores of the very first tile
        if (issue_s(0, true) != 1) ok = false;
        if (ok && ps.it.n[1] > 0 && issue_s(1, true) != 1) ok = false;
        if (ok) { tc_commit(bar(RE + ps.e % NR)); fa_cursor_advance(a, n_rounds, ps); }
      }
      while (ok && pv.valid) {
        const bool act_a = pv.j < pv.it.n[0], act_b = pv.j < pv.it.n[1];
        bool todo_a = ps.valid && ps.j < ps.it.n[0], todo_b = ps.valid && ps.j < ps.it.n[1];
        const bool any_s = todo_a || todo_b;
        if (SEP) {
          // P has columns of its own: a stream's next scores go out as soon as its softmax warps
          // have the current ones in registers, ahead of the O MMA that waits for P
          if (todo_a && act_a) {
            if (!mbar_wait(bar(CF + 0), pg[0] & 1, abort_flag) || issue_s(0, true) != 1) { ok = false; break; }
            todo_a = false;
          }
          if (act_a) { if (!issue_pv(0)) { ok = false; break; } }
          if (todo_b && act_b) {
            if (!mbar_wait(bar(CF + 1), pg[1] & 1, abort_flag) || issue_s(1, true) != 1) { ok = false; break; }
            todo_b = false;
          }
          if (act_b) { if (!issue_pv(1)) { ok = false; break; } }
        } else {
          if (act_a) { if (!issue_pv(0)) { ok = false; break; } }
          if (todo_a) {
            // stream A's next scores; if their operands have not landed, stream B's O goes first
            const int r = issue_s(0, !act_b);
            if (r < 0) { ok = false; break; }
            if (r == 1) todo_a = false;
          }
          if (act_b) { if (!issue_pv(1)) { ok = false; break; } }
        }
        tc_commit(bar(RE + (pv.e + 1) % NR));          // V tile free once both O MMAs retire
        // (a stream that was idle on this tile, or whose operands were late, gets its scores now;
        // its previous scores were consumed long ago)
        if (todo_a) { if (issue_s(0, true) != 1) { ok = false; break; } }
        if (todo_b) { if (issue_s(1, true) != 1) { ok = false; break; } }
        if (any_s) tc_commit(bar(RE + ps.e % NR));     // K tile free once both S MMAs retire
        fa_cursor_advance(a, n_rounds, pv);
        if (ps.valid) fa_cursor_advance(a, n_rounds, ps);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int x = warp >> 2;                          // stream
    const int row = (warp & 3) * 32 + lane;           // query row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t my_s = tS(x) + lane_addr, my_o = tO(x) + lane_addr, my_p = tP(x) + lane_addr;
    bool ok = true;
    int g = 0;                                        // key tiles of this stream consumed so far
    for (int r = 0; r < n_rounds && ok; ++r) {
      FaItem it;
      if (!fa_item(a, r, it)) continue;
      const int ntiles = it.n[x];
      if (ntiles == 0) continue;
      const int m0 = it.m0 + x * FA_BM;
      const int qpos = a.q_pos0 + m0 + row;           // absolute position for the causal rule
      float m_used = 0.f, l_run = 0.f;

      for (int j = 0; j < ntiles && ok; ++j, ++g) {
        // (waits are voted on so that the warp-collective tensor-memory accesses stay convergent)
        if (!__all_sync(0xffffffffu, mbar_wait(bar(SF + x), g & 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        // only the last tile(s) need masking: end of the keys, or the causal diagonal
        int valid = FA_BN;
        if ((j * FA_BN + FA_BN > a.kv_len) || (a.causal && j * FA_BN + FA_BN - 1 > a.q_pos0 + m0)) {
          valid = a.kv_len - j * FA_BN;
          if (a.causal) valid = min(valid, qpos - j * FA_BN + 1);
          valid = min(valid, FA_BN - 1 + (valid >= FA_BN));   // keeps "== FA_BN" meaning "no mask"
        }
        const FaRowState st = fa_softmax_tile<HD, SEP>(my_s, my_p, my_o, a.scale_log2, m_used, l_run, j == 0,
                                                        valid, bar(CF + x), bar(OF + x), (uint32_t)((g - 1) & 1),
                                                        bar(PF + x), abort_flag);
        if (!st.ok) { ok = false; break; }
        m_used = st.m_used; l_run = st.l_run;
      }
      // item epilogue: O / row sum -> bf16 -> global
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(OF + x), (g - 1) & 1, abort_flag));
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const bool live = m0 + row < a.S;
        uint16_t* dst = a.o + (long)it.b * a.o_bs + (long)(m0 + row) * a.o_rs + (long)it.head * a.o_hs;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t rr[32];
          tc_ld32(my_o + c * 32, rr);
          tc_wait_ld();
          if (live) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(rr[q4 * 8 + 0]) * inv, __uint_as_float(rr[q4 * 8 + 1]) * inv);
              w.y = pack_bf16(__uint_as_float(rr[q4 * 8 + 2]) * inv, __uint_as_float(rr[q4 * 8 + 3]) * inv);
              w.z = pack_bf16(__uint_as_float(rr[q4 * 8 + 4]) * inv, __uint_as_float(rr[q4 * 8 + 5]) * inv);
              w.w = pack_bf16(__uint_as_float(rr[q4 * 8 + 6]) * inv, __uint_as_float(rr[q4 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = w;
            }
          }
        }
        // the next item's first O MMA overwrites this accumulator: order the loads before the
        // arrival that releases it
        tc_fence_before();
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status != nullptr) atomicExch(a.status, B200_ERR_TIMEOUT);
  if (warp == 9) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// Splits element strides (batch, row, head) of a [B, rows, heads, hd]-like view into the 2D
// (row, column) bookkeeping the tensor maps use.  Returns false if the view is not expressible.
static bool split_strides(int64_t bs, int64_t rs, int64_t hs, int* batch_rows, int* head_rows,
                          int* head_cols) {
  if (rs <= 0) return false;
  if (bs % rs != 0) return false;
  *batch_rows = (int)(bs / rs);
  if (hs % rs == 0 && hs >= rs) { *head_rows = (int)(hs / rs); *head_cols = 0; }
  else if (hs < rs) { *head_rows = 0; *head_cols = (int)hs; }
  else return false;
  return true;
}

template <int HD>
static int fa_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                     const FaArgs& a, dim3 grid, cudaStream_t st, bool pdl) {
  // tiles (Q buffers of both streams + the K / V ring) + 32 barriers + TMEM slot / abort flag
  constexpr size_t smem = (size_t)(HD == 64 ? 12 : 7) * (HD / 64) * kAtomBytes + 256 + 16;
  static bool attr_set[kMaxDevices] = {false};
  if (opt_in_smem(flash_prefill_tc_kernel<HD>, (int)smem, attr_set) != cudaSuccess) return B200_ERR_LAUNCH;
  cudaError_t e = launch(flash_prefill_tc_kernel<HD>, grid, dim3(kFaThreads), smem, st, pdl, mq, mk, mv, a);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_flash_prefill_tc(void* out, const void* q, const void* k, const void* v,
                                     int batch, int S, int kv_len, int q_pos0, int n_q, int n_kv,
                                     int hd,
                                     int64_t q_bs, int64_t q_rs, int64_t q_hs,
                                     int64_t k_bs, int64_t k_rs, int64_t k_hs,
                                     int64_t v_bs, int64_t v_rs, int64_t v_hs,
                                     int64_t o_bs, int64_t o_rs, int64_t o_hs,
                                     int causal, float scale, int* status, int flags,
                                     b200_stream_t stream) {
  if (!out || !q || !k || !v || !(scale > 0.f)) return B200_ERR_ARG;
  if (batch <= 0 || S <= 0 || kv_len <= 0 || q_pos0 < 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 ||
      (hd != 64 && hd != 128) || batch > 65535 || n_q > 65535)
    return B200_ERR_SHAPE;
  const int64_t strides[12] = {q_bs, q_rs, q_hs, k_bs, k_rs, k_hs, v_bs, v_rs, v_hs, o_bs, o_rs, o_hs};
  for (int i = 0; i < 12; ++i) if (strides[i] & 7) return B200_ERR_ALIGN;
  if (((uintptr_t)out & 15) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15))
    return B200_ERR_ALIGN;
  FaArgs a;
  a.o = (uint16_t*)out; a.o_bs = o_bs; a.o_rs = o_rs; a.o_hs = o_hs; a.status = status;
  a.S = S; a.kv_len = kv_len; a.q_pos0 = q_pos0; a.group = n_q / n_kv; a.causal = causal ? 1 : 0;
  a.n_q = n_q;
  a.scale_log2 = scale * 1.4426950408889634f;
  if (!split_strides(q_bs, q_rs, q_hs, &a.q_batch_rows, &a.q_head_rows, &a.q_head_cols) ||
      !split_strides(k_bs, k_rs, k_hs, &a.k_batch_rows, &a.k_head_rows, &a.k_head_cols) ||
      !split_strides(v_bs, v_rs, v_hs, &a.v_batch_rows, &a.v_head_rows, &a.v_head_cols))
    return B200_ERR_SHAPE;
  int rc = get_encode();
  if (rc != B200_OK) return rc;
  // 2D views [rows, row_stride]; rows stop at the last valid row so that tiles reaching past
  // it are zero-filled by the TMA unit instead of touching memory the caller does not own
  const uint64_t q_rows = (uint64_t)(batch - 1) * a.q_batch_rows + (uint64_t)(n_q - 1) * a.q_head_rows + S;
  const uint64_t k_rows = (uint64_t)(batch - 1) * a.k_batch_rows + (uint64_t)(n_kv - 1) * a.k_head_rows + kv_len;
  const uint64_t v_rows = (uint64_t)(batch - 1) * a.v_batch_rows + (uint64_t)(n_kv - 1) * a.v_head_rows + kv_len;
  const uint64_t q_cols = a.q_head_cols ? (uint64_t)a.q_head_cols * n_q : (uint64_t)hd;
  const uint64_t k_cols = a.k_head_cols ? (uint64_t)a.k_head_cols * n_kv : (uint64_t)hd;
  const uint64_t v_cols = a.v_head_cols ? (uint64_t)a.v_head_cols * n_kv : (uint64_t)hd;
  CUtensorMap mq, mk, mv;
  if ((rc = make_map(&mq, q, q_rows, q_cols, (uint64_t)q_rs, 128, 64)) != B200_OK) return rc;
  if ((rc = make_map(&mk, k, k_rows, k_cols, (uint64_t)k_rs, 128, 64)) != B200_OK) return rc;
  if ((rc = make_map(&mv, v, v_rows, v_cols, (uint64_t)v_rs, 128, 64)) != B200_OK) return rc;
  a.n_mp = (S + 2 * FA_BM - 1) / (2 * FA_BM);
  a.n_bh = n_q * batch;
  const int64_t n_items = (int64_t)a.n_mp * a.n_bh;
  if (n_items > INT_MAX) return B200_ERR_SHAPE;
  a.n_items = (int)n_items;
  dim3 grid((unsigned)std::min<int64_t>(n_items, kNumSMs));
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  return hd == 128 ? fa_launch<128>(mq, mk, mv, a, grid, (cudaStream_t)stream, pdl)
                   : fa_launch<64>(mq, mk, mv, a, grid, (cudaStream_t)stream, pdl);
}
