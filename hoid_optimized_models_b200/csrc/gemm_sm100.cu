// Dense / grouped bf16 GEMM  Y[M,N] = X[M,K] W[N,K]^T  on the sm_100a tensor cores.
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer: cp.async.bulk.tensor 2D loads of a 128x64 X tile and a
//               256x64 W tile (both K-major, 128-byte swizzle) into a 4-stage ring
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (cta_group::1,
//               kind::f16, M128 N256 K16) with fp32 accumulators in tensor memory;
//               tcgen05.commit releases ring stages and publishes accumulators
//   warps 2..9  epilogue (two warps per 32-lane slab, alternating 64-column groups): tcgen05.ld 32 columns at a time, fused bias / residual /
//               SwiGLU / GELU.  bf16 results leave through a per-warp swizzled staging
//               tile and a TMA store (the residual arrives the same way with a TMA
//               load), so every global access of the epilogue is a full coalesced box
//               instead of 32 row-strided 64-byte pieces.  Two accumulators alternate,
//               so the epilogue of tile i overlaps the main loop of tile i+1.
// The N extent of the tile (256 / 128 / 64) is chosen per problem: 256 unless the problem
// has too few such tiles to occupy even a fraction of the SMs.
//
// GEGLU mode (a stock [2 O, K] projection, value half first): a tile's 256 W rows are 128 rows of
// the value half and the matching 128 rows of the gate half, loaded as two boxes, so ONE N = 256
// MMA produces both and the epilogue writes only (value + bias) * gelu(gate + bias).
//
// Grouped mode (MoE experts): rows of X are sorted by expert, `offsets[e]` is the
// first row of expert e, W is [E, N, K]; M-tiles never straddle an expert for
// stores (loads may read the neighbour's rows, the epilogue masks them).
//
// Every mbarrier wait is bounded: on expiry the CTA records B200_ERR_TIMEOUT in
// the status word, all roles leave their loops, tensor memory is released and
// the kernel returns.
#include "sm100.cuh"

namespace b200 {

constexpr int BM = 128, BK = 64;
constexpr int kGemmThreads = 320;   // TMA warp, MMA warp, 8 epilogue warps
constexpr uint32_t kABytes = BM * BK * 2;   // 16 KiB
constexpr int kMaxExperts = 128;
constexpr uint32_t kStageBoxBytes = 32 * 128;   // epilogue staging box: 32 rows x 64 bf16
constexpr int kEpiWarps = 8;                    // two per TMEM lane slab, alternating column groups
// ring depth: 192 KiB of operand stages whatever the tile width
constexpr int gemm_stages(int bn) { return bn == 256 ? 4 : (bn == 128 ? 6 : 8); }

struct GemmArgs {
  uint16_t* y; const uint16_t* bias; const uint16_t* resid; const int* offsets;
  int tma_epilogue;   // bf16 plain / bias / GELU / residual output goes through TMA boxes
  int* status;
  int M, N, K, ldy, ldr, epilogue, n_groups, y_dtype;
};

// K-major, 128-byte-swizzled operand tile: rows 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);   // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for SW128 K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// bf16 x bf16 -> fp32, both operands K-major, M = BM, N = bn.
constexpr uint32_t gemm_idesc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ---------------------------------------------------------------- tile schedule
struct Tile { int row0, row_end, n0, wrow0; bool valid; };

struct Sched {
  int mt, nt, total, bn;
  const int* cum;      // grouped: smem prefix of tiles per group [n_groups + 1]
  const int* offs;     // grouped: smem row offsets [n_groups + 1]
  int n_groups, M, N;
  __device__ __forceinline__ Tile get(int t) const {
    Tile r;
    r.valid = t < total;
    if (!r.valid) { r.row0 = r.row_end = r.n0 = r.wrow0 = 0; return r; }
    if (n_groups == 0) {
      const int tm = t % mt, tn = t / mt;
      r.row0 = tm * BM; r.row_end = min(M, r.row0 + BM); r.n0 = tn * bn; r.wrow0 = r.n0;
    } else {
      int lo = 0, hi = n_groups - 1;           // last group with cum[g] <= t
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (cum[mid] <= t) lo = mid; else hi = mid - 1; }
      const int local = t - cum[lo];
      const int tn = local % nt, tm = local / nt;
      r.row0 = offs[lo] + tm * BM; r.row_end = min(offs[lo + 1], r.row0 + BM);
      r.n0 = tn * bn; r.wrow0 = lo * N + r.n0;
    }
    return r;
  }
};


template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
            const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_r,
            GemmArgs a) {
  constexpr int kStages = gemm_stages(BN);
  constexpr uint32_t kBBytes = BN * BK * 2;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;   // 512 / 256 / 128: powers of two
  constexpr uint32_t kIdesc = gemm_idesc(BN);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // carve: [stages x (A|B)] 1024-aligned, then barriers and bookkeeping
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t s_stage = base + kStages * kStageBytes;           // 8 warps x 4 KiB staging
  unsigned char* g_stage = gen_base + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen_base + kStages * kStageBytes +
                                               kEpiWarps * kStageBoxBytes);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty, then 8 x resid
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_cum = reinterpret_cast<int*>(tmem_slot + 4);
  int* s_off = s_cum + (kMaxExperts + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  auto full_bar = [&](int s) { return smem_u32(bars + s); };
  auto empty_bar = [&](int s) { return smem_u32(bars + kStages + s); };
  auto tfull_bar = [&](int s) { return smem_u32(bars + 2 * kStages + s); };
  auto tempty_bar = [&](int s) { return smem_u32(bars + 2 * kStages + 2 + s); };

  pdl_launch_dependents();

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(tfull_bar(s), 1); mbar_init(tempty_bar(s), kEpiWarps); }
    for (int s = 0; s < kEpiWarps; ++s) mbar_init(smem_u32(bars + 2 * kStages + 4 + s), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    if (a.tma_epilogue) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_y) : "memory");
      if (a.resid != nullptr) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_r) : "memory");
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  pdl_wait();  // offsets / X / residual come from earlier kernels

  Sched sch;
  sch.M = a.M; sch.N = a.N; sch.n_groups = a.n_groups; sch.bn = BN;
  sch.nt = (a.N + BN - 1) / BN;
  sch.cum = s_cum; sch.offs = s_off;
  if (a.n_groups > 0) {
    for (int g = tid; g <= a.n_groups; g += kGemmThreads) s_off[g] = a.offsets[g];
    __syncthreads();
    if (tid == 0) {
      int c = 0;
      for (int g = 0; g < a.n_groups; ++g) {
        s_cum[g] = c;
        c += ((s_off[g + 1] - s_off[g] + BM - 1) / BM) * sch.nt;
      }
      s_cum[a.n_groups] = c;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  sch.mt = (a.M + BM - 1) / BM;
  sch.total = a.n_groups > 0 ? s_cum[a.n_groups] : sch.mt * sch.nt;
  const int kblocks = (a.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < sch.total; t += gridDim.x) {
        const Tile tl = sch.get(t);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * kStageBytes;
          mbar_expect_tx(full_bar(stage), kStageBytes);
          tma_load_2d(sa, &map_x, full_bar(stage), kb * BK, tl.row0);
          if (a.epilogue == B200_EPI_GEGLU) {
            // value rows [n0 / 2, +128) and gate rows [N / 2 + n0 / 2, +128) through a 128-row box
            tma_load_2d(sa + kABytes, &map_w, full_bar(stage), kb * BK, tl.n0 >> 1);
            tma_load_2d(sa + kABytes + kBBytes / 2, &map_w, full_bar(stage), kb * BK, (a.N >> 1) + (tl.n0 >> 1));
          } else {
            tma_load_2d(sa + kABytes, &map_w, full_bar(stage), kb * BK, tl.wrow0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // drain: give loads already in flight a bounded chance to land before exit
        for (int s = 0; s < kStages; ++s) {
          const long long t0 = clock64();
          while (!mbar_try(full_bar(s), 0) && !mbar_try(full_bar(s), 1) &&
                 clock64() - t0 < 2000000) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < sch.total; t += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * kStageBytes;
          const uint64_t da = umma_desc(sa), db = umma_desc(sa + kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advance 16 elements (32 B) along K inside the 128-byte swizzle atom
            tc_mma(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), kIdesc,
                   (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int slab = warp & 3;  // TMEM lanes [32*slab, 32*slab+32) belong to this warp
    const int half = (warp - 2) >> 2;   // the slab's two warps take alternate column groups
    const int ew = warp - 2;            // epilogue warp index: staging box and residual barrier
    int acc = 0; uint32_t acc_phase = 0, res_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < sch.total; t += gridDim.x) {
      const Tile tl = sch.get(t);
      // bias of the tile's columns, 8 per lane, fetched while the main loop is still running;
      // the per-column value is broadcast with a shuffle later (no dependent global load and no
      // shared memory in the per-chunk path)
      float bias8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (a.bias != nullptr && lane * 8 < BN && tl.n0 + lane * 8 < a.N)
        unpack8(*reinterpret_cast<const uint4*>(a.bias + tl.n0 + lane * 8), bias8);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tl.row0 + slab * 32 + lane;
      const bool row_ok = row < tl.row_end;
      const uint32_t taddr = tmem_base + ((uint32_t)(slab * 32) << 16) + (uint32_t)(acc * BN);
      // TMA boxes clip at the matrix edge but cannot mask rows of the NEXT expert, so a grouped
      // tile that ends inside the matrix takes the direct path
      const bool tma_tile = a.tma_epilogue && (tl.row_end - tl.row0 == BM || tl.row_end == a.M);
      if (tma_tile) {
        const uint32_t rbar = smem_u32(bars + 2 * kStages + 4 + ew);
        const uint32_t sbox = s_stage + ew * kStageBoxBytes;
        unsigned char* myrow = g_stage + ew * kStageBoxBytes + lane * 128;
#pragma unroll 1
        for (int g = half; g < BN / 64; g += 2) {
          const int col0 = tl.n0 + g * 64;
          if (col0 >= a.N) break;  // warp-uniform
          // the previous store from this warp's staging box must have finished READING it
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
          if (a.resid != nullptr) {
            if (lane == 0) {
              mbar_expect_tx(rbar, kStageBoxBytes);
              tma_load_2d(sbox, &map_r, rbar, col0, tl.row0 + slab * 32);
            }
            if (!mbar_wait(rbar, res_phase, abort_flag)) { ok = false; break; }
            res_phase ^= 1;
          }
          uint32_t r[2][32];
          tc_ld32(taddr + g * 64, r[0]);
          tc_ld32(taddr + g * 64 + 32, r[1]);
          tc_wait_ld();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[h][j]);
            if (a.bias != nullptr) {
              const int src = (g * 64 + h * 32) >> 3;   // lane holding the first of these columns
#pragma unroll
              for (int j = 0; j < 32; ++j)
                v[j] += __shfl_sync(0xffffffffu, bias8[j & 7], src + (j >> 3));
            }
            if (a.epilogue == B200_EPI_GELU) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4* slot = reinterpret_cast<uint4*>(myrow + (((h * 4 + q4) ^ (lane & 7)) << 4));
              if (a.resid != nullptr) {
                float r8[8];
                unpack8(*slot, r8);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[q4 * 8 + e] += r8[e];
              }
              uint4 w;
              w.x = pack_bf16(v[q4 * 8 + 0], v[q4 * 8 + 1]); w.y = pack_bf16(v[q4 * 8 + 2], v[q4 * 8 + 3]);
              w.z = pack_bf16(v[q4 * 8 + 4], v[q4 * 8 + 5]); w.w = pack_bf16(v[q4 * 8 + 6], v[q4 * 8 + 7]);
              *slot = w;
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(&map_y), "r"(sbox), "r"(col0), "r"(tl.row0 + slab * 32) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (!ok) break;
      } else if (a.epilogue == B200_EPI_GEGLU) {
        // accumulator columns [0, BN/2) are the value half, [BN/2, BN) the gate half of output
        // columns n0 / 2 ..
        const int O = a.N >> 1;
#pragma unroll 1
        for (int c = half; c < BN / 64; c += 2) {
          const int ocol0 = (tl.n0 >> 1) + c * 32;
          if (ocol0 >= O) break;  // warp-uniform
          uint32_t rv[32], rg[32];
          tc_ld32(taddr + c * 32, rv);
          tc_ld32(taddr + BN / 2 + c * 32, rg);
          tc_wait_ld();
          if (row_ok) {
            uint16_t* dst = a.y + (size_t)row * a.ldy + ocol0;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (ocol0 + j < O) {
                float bv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, bg[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (a.bias != nullptr) {
                  unpack8(*reinterpret_cast<const uint4*>(a.bias + ocol0 + j), bv);
                  unpack8(*reinterpret_cast<const uint4*>(a.bias + O + ocol0 + j), bg);
                }
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  o[e] = (__uint_as_float(rv[j + e]) + bv[e]) * gelu_erf(__uint_as_float(rg[j + e]) + bg[e]);
                uint4 w;
                w.x = pack_bf16(o[0], o[1]); w.y = pack_bf16(o[2], o[3]);
                w.z = pack_bf16(o[4], o[5]); w.w = pack_bf16(o[6], o[7]);
                *reinterpret_cast<uint4*>(dst + j) = w;
              }
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = half; c < BN / 32; c += 2) {
        const int col0 = tl.n0 + c * 32;
        if (col0 >= a.N) break;  // warp-uniform
        uint32_t r[32];
        tc_ld32(taddr + c * 32, r);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (a.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j < a.N) {
              float b8[8];
              unpack8(*reinterpret_cast<const uint4*>(a.bias + col0 + j), b8);
#pragma unroll
              for (int e = 0; e < 8; ++e) v[j + e] += b8[e];
            }
          }
        }
        if (a.epilogue == B200_EPI_SWIGLU) {
          if (row_ok) {
            uint16_t* dst = a.y + (size_t)row * a.ldy + (col0 >> 1);
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              if (col0 + 2 * j < a.N) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float g = v[2 * (j + e)], u = v[2 * (j + e) + 1];
                  o[e] = g / (1.f + __expf(-g)) * u;
                }
                uint4 w;
                w.x = pack_bf16(o[0], o[1]); w.y = pack_bf16(o[2], o[3]);
                w.z = pack_bf16(o[4], o[5]); w.w = pack_bf16(o[6], o[7]);
                *reinterpret_cast<uint4*>(dst + j) = w;
              }
            }
          }
        } else {
          if (a.epilogue == B200_EPI_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
          }
          if (row_ok && a.y_dtype == B200_F32) {
            float* dst = reinterpret_cast<float*>(a.y) + (size_t)row * a.ldy + col0;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              if (col0 + j < a.N)
                *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
          } else if (row_ok) {
            uint16_t* dst = a.y + (size_t)row * a.ldy + col0;
            const uint16_t* rs = a.resid ? a.resid + (size_t)row * a.ldr + col0 : nullptr;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col0 + j < a.N) {
                if (rs != nullptr) {
                  float r8[8];
                  unpack8(*reinterpret_cast<const uint4*>(rs + j), r8);
#pragma unroll
                  for (int e = 0; e < 8; ++e) v[j + e] += r8[e];
                }
                uint4 w;
                w.x = pack_bf16(v[j + 0], v[j + 1]); w.y = pack_bf16(v[j + 2], v[j + 3]);
                w.z = pack_bf16(v[j + 4], v[j + 5]); w.w = pack_bf16(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = w;
              }
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // stores landed
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag && a.status != nullptr) atomicExch(a.status, B200_ERR_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

// ---------------------------------------------------------------- host side
template <int BN>
static int gemm_launch_bn(const CUtensorMap& mx, const void* w, uint64_t wrows, int K, int ldw,
                          const CUtensorMap& my, const CUtensorMap& mr, const GemmArgs& a,
                          int max_tiles_m, cudaStream_t stream, bool pdl) {
  constexpr int kStages = gemm_stages(BN);
  constexpr size_t smem = 1024 + (size_t)kStages * (kABytes + BN * BK * 2) +
                          kEpiWarps * kStageBoxBytes + 256 + 2 * (kMaxExperts + 1) * 4;
  CUtensorMap mw;
  int rc = make_map(&mw, w, wrows, (uint64_t)K, (uint64_t)ldw, a.epilogue == B200_EPI_GEGLU ? BN / 2 : BN, BK);
  if (rc != B200_OK) return rc;
  const int nt = (a.N + BN - 1) / BN;
  long tiles = (long)max_tiles_m * nt;
  int grid = (int)(tiles < kNumSMs ? tiles : kNumSMs);
  if (grid < 1) grid = 1;
  static bool attr_set[kMaxDevices] = {false};
  if (opt_in_smem(gemm_kernel<BN>, (int)smem, attr_set) != cudaSuccess) return B200_ERR_LAUNCH;
  cudaError_t e = launch(gemm_kernel<BN>, dim3(grid), dim3(kGemmThreads), smem, stream, pdl, mx, mw,
                         my, mr, a);
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}

static int gemm_launch(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                       int ldx, int ldw, int ldy, const void* bias, const void* resid, int ldr,
                       int epilogue, const int* offsets, int n_groups, int max_tiles_m, int* status,
                       int flags, cudaStream_t stream) {
  if (!x || !w || !y) return B200_ERR_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || (N & 7)) return B200_ERR_SHAPE;
  if ((ldx & 7) || (ldw & 7) || (ldy & 7) || (resid && (ldr & 7))) return B200_ERR_ALIGN;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)y & 15) ||
      ((uintptr_t)bias & 15) || ((uintptr_t)resid & 15))
    return B200_ERR_ALIGN;
  if (epilogue < B200_EPI_NONE || epilogue > B200_EPI_GEGLU) return B200_ERR_ARG;
  const bool halves = epilogue == B200_EPI_SWIGLU || epilogue == B200_EPI_GEGLU;
  if (halves && (resid != nullptr || (N & 15))) return B200_ERR_SHAPE;
  if (epilogue == B200_EPI_GEGLU && n_groups > 0) return B200_ERR_ARG;
  if (y_dtype == B200_F32 && (resid != nullptr || halves)) return B200_ERR_ARG;
  if (n_groups < 0 || n_groups > kMaxExperts || (n_groups > 0 && !offsets)) return B200_ERR_ARG;
  int rc = get_encode();
  if (rc != B200_OK) return rc;

  GemmArgs a;
  a.y = (uint16_t*)y; a.bias = (const uint16_t*)bias; a.resid = (const uint16_t*)resid;
  a.offsets = offsets; a.status = status;
  a.M = M; a.N = N; a.K = K; a.ldy = ldy; a.ldr = ldr; a.epilogue = epilogue; a.n_groups = n_groups;
  a.y_dtype = y_dtype;
  a.tma_epilogue = (y_dtype == B200_BF16 && !halves) ? 1 : 0;

  CUtensorMap mx, my, mr;
  const uint64_t wrows = n_groups > 0 ? (uint64_t)n_groups * N : (uint64_t)N;
  if ((rc = make_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, BM, BK)) != B200_OK) return rc;
  my = mx; mr = mx;   // placeholders when the TMA epilogue is off
  if (a.tma_epilogue) {
    if ((rc = make_map(&my, y, (uint64_t)M, (uint64_t)N, (uint64_t)ldy, 32, 64)) != B200_OK) return rc;
    if (resid && (rc = make_map(&mr, resid, (uint64_t)M, (uint64_t)N, (uint64_t)ldr, 32, 64)) != B200_OK)
      return rc;
  }
  // Tile width.  Narrow tiles fill more SMs but each moves (128 + bn) rows of operands for
  // 128 x bn outputs and runs the MMA below its rate at N = 64, so 256 wins as soon as it keeps
  // well under half of the SMs busy (measured on M = 1024 / 1500 prefill shapes: 256 beats 128
  // by 1.2-1.5x from 80 tiles up and is within 8 % at 60).
  const long tiles256 = (long)max_tiles_m * ((N + 255) / 256);
  const long tiles128 = (long)max_tiles_m * ((N + 127) / 128);
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  const int forced = g_tuning[B200_TUNE_GEMM_BN];
  int bn = tiles256 >= 64 ? 256 : (tiles128 >= 32 ? 128 : 64);
  if (forced == 256 || forced == 128 || forced == 64) bn = forced;
  if (epilogue == B200_EPI_GEGLU) bn = 256;   // the two halves of a tile are 128 W rows each
  if (bn == 256) return gemm_launch_bn<256>(mx, w, wrows, K, ldw, my, mr, a, max_tiles_m, stream, pdl);
  if (bn == 128) return gemm_launch_bn<128>(mx, w, wrows, K, ldw, my, mr, a, max_tiles_m, stream, pdl);
  return gemm_launch_bn<64>(mx, w, wrows, K, ldw, my, mr, a, max_tiles_m, stream, pdl);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gemm_bf16(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                              int ldx, int ldw, int ldy, const void* bias, const void* resid,
                              int ldr, int epilogue, int* status, int flags,
                              b200_stream_t stream) {
  return gemm_launch(x, w, y, y_dtype, M, N, K, ldx, ldw, ldy, bias, resid, ldr, epilogue, nullptr, 0,
                     (M + BM - 1) / BM, status, flags, (cudaStream_t)stream);
}

extern "C" int b200_moe_grouped_gemm(const void* x, const void* w, void* y, const int* offsets,
                                     int n_experts, int rows, int N, int K, int ldx, int ldy,
                                     int epilogue, int* status, int flags, b200_stream_t stream) {
  if (n_experts <= 0) return B200_ERR_ARG;
  // upper bound on M-tiles: every expert may add one partial tile
  const int max_tiles_m = (rows + BM - 1) / BM + n_experts;
  return gemm_launch(x, w, y, B200_BF16, rows, N, K, ldx, K, ldy, nullptr, nullptr, 0, epilogue, offsets,
                     n_experts, max_tiles_m, status, flags, (cudaStream_t)stream);
}
