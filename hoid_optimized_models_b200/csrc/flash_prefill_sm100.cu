// Prefill / encoder flash attention on the sm_100a tensor cores (tcgen05 + TMEM + TMA).
//
// Persistent: one CTA per SM walks a list of work items (128 query rows of one head each) and,
// inside an item, the keys in tiles of 128.  The three roles run decoupled through mbarrier
// rings that are never drained between items, so the next item's Q / K / V loads and its first
// S = Q K^T are in flight while the softmax warps finish the current one:
//   warp 0     TMA producer: Q per item (two buffers at head dim 64), K and V tiles into a ring
//              of 4 (head dim 64) or 2 (head dim 128) stages
//   warp 1     MMA issuer (one lane): S_j = Q K_j^T (M128 N128, K = head dim) into one of two
//              S accumulators in tensor memory, and O_j = P_j V_j (V consumed in its natural
//              [key][dim] layout as an MN-major operand) into the O-tile accumulator
//   warps 2-17 softmax: four threads per query row (= TMEM lane), each owning 32 key columns
//              and a quarter of the output dims.  A thread pulls its 32 scores with one
//              tcgen05.ld, the row maximum is exchanged between the four through shared memory,
//              P_j = exp2(...) is written as bf16 into the 128-byte-swizzled shared tile the
//              second MMA reads, and only then O_{j-1} is folded from tensor memory into fp32
//              registers with the online-softmax correction.  S and O are double-buffered in
//              tensor memory, so the tensor core works on S_{j+1} and O_j while the softmax
//              warps are busy, and the softmax warps never wait for an MMA they just asked for.
// Work order: causal items heaviest query tile first, dealt to the CTAs in alternating direction
// (round r forwards, round r + 1 backwards) so every CTA gets the same number of key tiles to
// within one round; bidirectional items with the query tiles of one head adjacent, so a head's
// K / V are read from DRAM once and from L2 afterwards.
// The score matrix never leaves the SM.  Causal tiles above the diagonal are never visited.
// Every mbarrier wait is bounded (status word + clean TMEM release on expiry).
#include <algorithm>
#include <climits>

#include "sm100.cuh"

namespace b200 {

constexpr int FA_BM = 128, FA_BN = 128;
constexpr int kFaParts = 4;        // softmax threads per query row
constexpr int kFaThreads = 64 + 128 * kFaParts;   // TMA warp, MMA warp, 16 softmax warps
constexpr uint32_t kAtomBytes = 128 * 128;   // a 128-row x 64-column bf16 box: 16 KiB

struct FaArgs {
  uint16_t* o; long o_bs, o_rs, o_hs;
  int* status;
  int S, kv_len, q_pos0, group, causal, n_q;
  int n_mt, n_bh, n_items;          // query tiles per head, batch x heads, work items
  // row / column bookkeeping of the 2D views the tensor maps cover
  int q_batch_rows, q_head_rows, q_head_cols;
  int k_batch_rows, k_head_rows, k_head_cols;
  int v_batch_rows, v_head_rows, v_head_cols;
  float scale_log2;
};

struct FaItem { int b, head, m0, ntiles; };

// The work item of this CTA in round r (false: the round has none for it).  All three roles
// call this with the same arguments and therefore walk identical lists.
__device__ __forceinline__ bool fa_item(const FaArgs& a, int r, FaItem& it) {
  const int G = (int)gridDim.x, c = (int)blockIdx.x;
  const int w = r * G + ((a.causal && (r & 1)) ? G - 1 - c : c);
  if (w >= a.n_items) return false;
  int mt, bh;
  if (a.causal) { mt = a.n_mt - 1 - w / a.n_bh; bh = w % a.n_bh; }
  else { mt = w % a.n_mt; bh = w / a.n_mt; }
  it.head = bh % a.n_q;
  it.b = bh / a.n_q;
  it.m0 = mt * FA_BM;
  int kv_end = a.kv_len;
  if (a.causal) kv_end = min(kv_end, a.q_pos0 + it.m0 + FA_BM);
  it.ntiles = (kv_end + FA_BN - 1) / FA_BN;      // >= 1: kv_len >= 1 and q_pos0 >= 0
  return true;
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

template <int HD>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, FaArgs a) {
  constexpr int ATOMS = HD / 64;                        // 64-column boxes per operand tile
  constexpr int NQ = HD == 64 ? 2 : 1;                  // Q buffers
  constexpr int NST = HD == 64 ? 4 : 2;                 // K | V stages
  constexpr uint32_t kQBytes = ATOMS * kAtomBytes;      // Q / K / V tile bytes
  constexpr uint32_t kPBytes = 2 * kAtomBytes;          // P tile: 128 rows x 128 keys
  constexpr uint32_t kStage = 2 * kQBytes;              // K + V
  constexpr uint32_t kTiles = NQ * kQBytes + NST * kStage + kPBytes;   // 192 KiB either way
  // barrier indices
  constexpr int QF = 0, QE = NQ, KF = 2 * NQ, KE = 2 * NQ + NST, SF = 2 * NQ + 2 * NST,
                PF = SF + 2, OF = SF + 3, NBAR = SF + 4;
  static_assert(NBAR <= 16, "barrier block is 16 entries");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // Operand tiles need 1024-byte alignment.  The dynamic window starts 1 KB into the CTA's
  // shared memory (after the system-reserved kilobyte) and is therefore aligned; if a future
  // toolchain breaks that assumption the kernel reports it instead of corrupting tiles.
  const uint32_t base = smem_u32(smem_raw);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, B200_ERR_ALIGN);
    return;
  }
  unsigned char* gen = smem_raw;
  const uint32_t sQ = base;                             // NQ buffers
  const uint32_t sKV = sQ + NQ * kQBytes;               // NST stages x (K | V)
  unsigned char* gP = gen + NQ * kQBytes + NST * kStage;   // one buffer (freed by the O_j commit)
  const uint32_t sP = smem_u32(gP);
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kTiles);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xch = reinterpret_cast<float*>(tmem_slot + 4);   // [2 parities][4 parts][128 rows] + seq
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_rounds = (a.n_items + (int)gridDim.x - 1) / (int)gridDim.x;

  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < NBAR; ++i) mbar_init(bar(i), i == PF ? 4 * kFaParts : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = tid; i < 64 * kFaParts; i += kFaThreads)
    reinterpret_cast<int*>(xch + 256 * kFaParts)[i] = 0;   // 16-bit exchange sequence numbers
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;            // S buffers at columns 0 and 128
  const uint32_t tO = tmem_base + 256;      // two O-tile accumulators, HD columns each

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int qi = 0, g = 0;           // items and key tiles issued so far
      bool ok = true;
      for (int r = 0; r < n_rounds && ok; ++r) {
        FaItem it;
        if (!fa_item(a, r, it)) continue;
        const int kvh = it.head / a.group;
        const int qb = qi % NQ;
        if (!mbar_wait(bar(QE + qb), ((qi / NQ) & 1) ^ 1, abort_flag)) { ok = false; break; }
        const int q_row = it.b * a.q_batch_rows + it.head * a.q_head_rows + it.m0;
        const int q_col = it.head * a.q_head_cols;
        mbar_expect_tx(bar(QF + qb), kQBytes);
#pragma unroll
        for (int t = 0; t < ATOMS; ++t)
          tma_load_2d(sQ + qb * kQBytes + t * kAtomBytes, &map_q, bar(QF + qb), q_col + 64 * t, q_row);
        ++qi;
        const int k_row0 = it.b * a.k_batch_rows + kvh * a.k_head_rows, k_col = kvh * a.k_head_cols;
        const int v_row0 = it.b * a.v_batch_rows + kvh * a.v_head_rows, v_col = kvh * a.v_head_cols;
        for (int j = 0; j < it.ntiles; ++j, ++g) {
          const int st = g % NST;
          if (!mbar_wait(bar(KE + st), ((g / NST) & 1) ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t sk = sKV + st * kStage, sv = sk + kQBytes;
          mbar_expect_tx(bar(KF + st), kStage);
#pragma unroll
          for (int t = 0; t < ATOMS; ++t) {
            tma_load_2d(sk + t * kAtomBytes, &map_k, bar(KF + st), k_col + 64 * t, k_row0 + j * FA_BN);
            tma_load_2d(sv + t * kAtomBytes, &map_v, bar(KF + st), v_col + 64 * t, v_row0 + j * FA_BN);
          }
        }
      }
      if (!ok) {
        // give the copies still in flight a bounded time to land before the CTA retires
        for (int i = 1; i <= min(g, NST); ++i)
          mbar_wait_quiet(bar(KF + (g - i) % NST), ((g - i) / NST) & 1, 2000000);
        for (int i = 1; i <= min(qi, NQ); ++i)
          mbar_wait_quiet(bar(QF + (qi - i) % NQ), ((qi - i) / NQ) & 1, 2000000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = fa_idesc(FA_BN, 0);
      constexpr uint32_t idesc_o = fa_idesc(HD, 1);
      // key tiles of all my items
      int total = 0;
      for (int r = 0; r < n_rounds; ++r) { FaItem it; if (fa_item(a, r, it)) total += it.ntiles; }
      // Cursor of the S = Q K^T issue.  It runs one tile ahead of the O = P V issue and crosses
      // item boundaries; when its operands have not landed yet the O MMAs go first.
      int s_r = -1, s_j = 0, s_n = 0, s_qi = -1, s_g = 0;
      bool s_new_q = false;
      // 1 issued, 0 operands not there yet (only when !blocking), -1 gave up
      auto issue_s = [&](bool blocking) -> int {
        if (s_j == s_n) {                     // first tile of the next item
          FaItem it;
          do { ++s_r; } while (s_r < n_rounds && !fa_item(a, s_r, it));
          if (s_r >= n_rounds) return -1;
          s_n = it.ntiles; s_j = 0; ++s_qi; s_new_q = true;
        }
        const int st = s_g % NST, qb = s_qi % NQ;
        if (!blocking) {
          if (s_new_q && !mbar_try(bar(QF + qb), (s_qi / NQ) & 1)) return 0;
          if (!mbar_try(bar(KF + st), (s_g / NST) & 1)) return 0;
        } else {
          if (s_new_q && !mbar_wait(bar(QF + qb), (s_qi / NQ) & 1, abort_flag)) return -1;
          if (!mbar_wait(bar(KF + st), (s_g / NST) & 1, abort_flag)) return -1;
        }
        s_new_q = false;
        tc_fence_after();
        const uint32_t sk = sKV + st * kStage, sq = sQ + qb * kQBytes;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * kAtomBytes + (k & 3) * 32;
          tc_mma(tS + (s_g & 1) * FA_BN, umma_desc_k(sq + off), umma_desc_k(sk + off), idesc_s, k != 0 ? 1u : 0u);
        }
        tc_commit(bar(SF + (s_g & 1)));
        ++s_j; ++s_g;
        if (s_j == s_n) tc_commit(bar(QE + qb));   // Q buffer free once these MMAs retire
        return 1;
      };
      bool ok = total > 0 && issue_s(true) == 1;
      for (int g = 0; g < total && ok; ++g) {
        const int st = g % NST;
        int ahead = 1;
        if (g + 1 < total) { ahead = issue_s(false); if (ahead < 0) { ok = false; break; } }
        if (!mbar_wait(bar(PF), g & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sv = sKV + st * kStage + kQBytes;
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          // A = P (K-major over keys): 16 keys = 32 bytes inside a 64-key atom
          const uint64_t da = umma_desc_k(sP + (k >> 2) * kAtomBytes + (k & 3) * 32);
          // B = V (MN-major over dims): 16 keys = two 8-row groups = 2048 bytes
          const uint64_t db = umma_desc_mn(sv + k * 2048, kAtomBytes, 1024);
          tc_mma(tO + (g & 1) * HD, da, db, idesc_o, k != 0 ? 1u : 0u);
        }
        tc_commit(bar(OF));          // O tile ready, P buffer free
        tc_commit(bar(KE + st));     // K/V stage free
        if (ahead == 0 && issue_s(true) != 1) { ok = false; break; }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    constexpr int NP = kFaParts;
    const int slab = warp & 3;                        // TMEM lanes [32 slab, 32 slab + 32)
    const int part = (warp - 2) >> 2;                 // which 32 key columns / quarter of the dims
    const int row = slab * 32 + lane;                 // query row inside the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(slab * 32) << 16;
    constexpr int OD = HD / NP;                       // output dims owned by this thread (32 / 16)
    bool ok = true;
    auto ex2 = [](float x) -> float {
      float y;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
      return y;
    };
    // Exchange one float per tile between the NP threads of a row: value slots are
    // double-buffered by sequence parity, a per-thread 16-bit sequence number publishes them,
    // and the reader's wait is bounded like every other wait in this kernel.  The sequence
    // runs on across items (equality tests only, so wrapping at 65536 is harmless).
    volatile float* xval = xch;                                                   // [2][NP][128]
    volatile unsigned short* xseq = reinterpret_cast<volatile unsigned short*>(xch + 256 * NP);
    int xs = 0;
    auto publish = [&](int seq, float mine) {
      xval[((seq & 1) * NP + part) * 128 + row] = mine;
      __threadfence_block();
      xseq[part * 128 + row] = (unsigned short)seq;
    };
    auto collect = [&](int seq, float* others) -> bool {   // others[NP - 1]
      const long long t0 = clock64();
#pragma unroll
      for (int o = 1; o < NP; ++o) {
        const int p2 = (part + o) & (NP - 1);
        int spins = 0;
        // a partner is never more than one exchange ahead, so these two values are the only ones
        while (xseq[p2 * 128 + row] != (unsigned short)seq &&
               xseq[p2 * 128 + row] != (unsigned short)(seq + 1)) {
          if ((++spins & 255) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitBudget) { *abort_flag = 1; return false; }
          }
        }
      }
      __threadfence_block();
#pragma unroll
      for (int o = 1; o < NP; ++o)
        others[o - 1] = xval[((seq & 1) * NP + ((part + o) & (NP - 1))) * 128 + row];
      return true;
    };

    int g = 0;                                        // key tiles consumed so far, all items
    for (int r = 0; r < n_rounds && ok; ++r) {
      FaItem it;
      if (!fa_item(a, r, it)) continue;
      const int ntiles = it.ntiles, m0 = it.m0;
      const int qpos = a.q_pos0 + m0 + row;           // absolute position for the causal rule
      float o_acc[OD];
#pragma unroll
      for (int d = 0; d < OD; ++d) o_acc[d] = 0.f;
      float m_run = -INFINITY, l_run = 0.f, corr_prev = 1.f;

      auto fold_o = [&](int gg, float corr) {
        // o_acc = o_acc * corr + O_j  (O_j was produced with the row maximum after tile j).
        // The caller has already waited for that tile's O barrier phase; waiting a second time
        // could meet the barrier two phases further on, where the same parity reads "not yet".
#pragma unroll
        for (int c = 0; c < OD / 16; ++c) {   // 16 columns at a time keeps the register count low
          uint32_t rr[16];
          tc_ld16(tO + (gg & 1) * HD + part * OD + c * 16 + lane_addr, rr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o_acc[c * 16 + i] = fmaf(o_acc[c * 16 + i], corr, __uint_as_float(rr[i]));
        }
      };

      for (int j = 0; j < ntiles && ok; ++j, ++g) {
        const int sb = g & 1;
        if (!mbar_wait(bar(SF + sb), (g >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const int key0 = j * FA_BN + part * 32;          // first key of this thread's columns
        uint32_t rr[32];
        tc_ld32(tS + sb * FA_BN + part * 32 + lane_addr, rr);
        tc_wait_ld();
        float sv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[i] = __uint_as_float(rr[i]);
        // only the last tile(s) need masking: end of the keys, or the causal diagonal
        const bool need_mask = (j * FA_BN + FA_BN > a.kv_len) ||
                               (a.causal && j * FA_BN + FA_BN - 1 > a.q_pos0 + m0);
        if (need_mask) {
          int valid = a.kv_len - key0;
          if (a.causal) valid = min(valid, qpos - key0 + 1);
#pragma unroll
          for (int i = 0; i < 32; ++i) sv[i] = (i < valid) ? sv[i] : -INFINITY;
        }
        float mt = sv[0];
#pragma unroll
        for (int i = 1; i < 32; ++i) mt = fmaxf(mt, sv[i]);
        publish(++xs, mt);
        float mo[NP - 1];
        if (!collect(xs, mo)) { ok = false; break; }
#pragma unroll
        for (int o = 0; o < NP - 1; ++o) mt = fmaxf(mt, mo[o]);
        const float m_new = fmaxf(m_run, mt * a.scale_log2);
        const float mu = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = ex2(m_run - mu);
        // p = exp2(s * scale - m), row sum, P tile (bf16, 128-byte swizzle, K-major): this
        // thread's 32 keys are four 16-byte chunks of atom part / 2
        float ps = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) { sv[i] = ex2(fmaf(sv[i], a.scale_log2, -mu)); ps += sv[i]; }
        // The P buffer is free once the tensor core has finished O_{j-1}; that MMA was issued a
        // whole tile of exponentials ago, so this wait does not normally spin.  (At j = 0 the
        // previous item's last fold already proved it.)
        if (j > 0) {
          if (!mbar_wait(bar(OF), (g - 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        unsigned char* prow = gP + (part >> 1) * kAtomBytes + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 w;
          w.x = pack_bf16(sv[q4 * 8 + 0], sv[q4 * 8 + 1]); w.y = pack_bf16(sv[q4 * 8 + 2], sv[q4 * 8 + 3]);
          w.z = pack_bf16(sv[q4 * 8 + 4], sv[q4 * 8 + 5]); w.w = pack_bf16(sv[q4 * 8 + 6], sv[q4 * 8 + 7]);
          const int chunk = (part & 1) * 4 + q4;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) = w;
        }
        // make the P tile visible to the tensor core (async proxy) and hand it over
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PF));            // one arrival per warp
        // fold the previous tile's output while the tensor core works on this one (the two O
        // accumulators alternate, so O_j may be written while O_{j-1} is read)
        if (j > 0) fold_o(g - 1, corr_prev);
        l_run = l_run * corr + ps;
        m_run = m_new;
        corr_prev = corr;
      }
      if (ok) ok = mbar_wait(bar(OF), (g - 1) & 1, abort_flag);
      if (ok) { tc_fence_after(); fold_o(g - 1, corr_prev); }
      // the row sum is split between the NP threads of the row
      if (ok) {
        publish(++xs, l_run);
        float lo[NP - 1];
        ok = collect(xs, lo);
#pragma unroll
        for (int o = 0; o < NP - 1; ++o) l_run += lo[o];
      }
      if (ok && m0 + row < a.S) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint16_t* dst = a.o + (long)it.b * a.o_bs + (long)(m0 + row) * a.o_rs + (long)it.head * a.o_hs + part * OD;
#pragma unroll
        for (int d = 0; d < OD; d += 8) {
          uint4 w;
          w.x = pack_bf16(o_acc[d] * inv, o_acc[d + 1] * inv);
          w.y = pack_bf16(o_acc[d + 2] * inv, o_acc[d + 3] * inv);
          w.z = pack_bf16(o_acc[d + 4] * inv, o_acc[d + 5] * inv);
          w.w = pack_bf16(o_acc[d + 6] * inv, o_acc[d + 7] * inv);
          *reinterpret_cast<uint4*>(dst + d) = w;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status != nullptr) atomicExch(a.status, B200_ERR_TIMEOUT);
  if (warp == 1) {
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
  // tiles (Q buffers, K | V ring, P: 192 KiB at either head dim) + 16 barriers + TMEM slot /
  // flags + exchange values and sequence numbers
  constexpr size_t smem = (size_t)12 * kAtomBytes + 128 + 16 +
                          (size_t)2 * kFaParts * 128 * 4 + (size_t)kFaParts * 128 * 2;
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
  if (!out || !q || !k || !v) return B200_ERR_ARG;
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
  a.n_mt = (S + FA_BM - 1) / FA_BM;
  a.n_bh = n_q * batch;
  const int64_t n_items = (int64_t)a.n_mt * a.n_bh;
  if (n_items > INT_MAX) return B200_ERR_SHAPE;
  a.n_items = (int)n_items;
  dim3 grid((unsigned)std::min<int64_t>(n_items, kNumSMs));
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  return hd == 128 ? fa_launch<128>(mq, mk, mv, a, grid, (cudaStream_t)stream, pdl)
                   : fa_launch<64>(mq, mk, mv, a, grid, (cudaStream_t)stream, pdl);
}
