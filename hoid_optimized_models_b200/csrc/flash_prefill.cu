// Prefill / encoder flash attention (causal GQA or bidirectional MHA), bf16 in/out.
//
// Grid (ceil(S/64), n_q, batch).  A CTA of four warps owns 64 query rows of one
// head; each warp keeps its 16 rows of Q as tensor-core A fragments in registers
// for the whole pass.  K and V tiles of 64 keys stream through a double-buffered
// shared-memory ring filled with 16-byte cp.async (XOR-swizzled rows, so ldmatrix
// is conflict free); S = Q K^T and O += P V run on mma.sync m16n8k16 with fp32
// accumulators and an exp2 online softmax; the S accumulators are re-used in
// place as the P operand.  Causal tiles beyond the diagonal are never loaded.
// The [S,S] score matrix never exists in memory.
#include "common.cuh"

namespace b200 {

constexpr int FP_BM = 64, FP_BN = 64, FP_THREADS = 128;

struct FpArgs {
  uint16_t* o; const uint16_t* q; const uint16_t* k; const uint16_t* v;
  long q_bs, q_rs, q_hs;     // batch / row / head strides (elements)
  long k_bs, k_rs, k_hs;
  long v_bs, v_rs, v_hs;
  long o_bs, o_rs, o_hs;
  int S, kv_len, q_pos0, group, causal;
  float scale_log2;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of 16-byte chunk `c` of row `r` in a swizzled [rows][HD] bf16 tile
template <int HD>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * (HD * 2) + ((c ^ (r & 7)) << 4));
}

// cooperative load of a [64][HD] tile; rows clamped to [0, max_row]
template <int HD>
__device__ __forceinline__ void load_tile(uint32_t smem, const uint16_t* base, long row_stride,
                                          int row0, int max_row, int tid) {
  constexpr int CPR = HD / 8;  // chunks per row
#pragma unroll
  for (int i = tid; i < 64 * CPR; i += FP_THREADS) {
    const int r = i / CPR, c = i % CPR;
    int gr = row0 + r;
    gr = gr > max_row ? max_row : gr;
    cp_async16(smem + swz<HD>(r, c), base + (long)gr * row_stride + c * 8);
  }
}

template <int HD>
__global__ void __launch_bounds__(FP_THREADS) flash_prefill_kernel(FpArgs a) {
  extern __shared__ __align__(128) unsigned char fp_smem[];
  constexpr int TILE = 64 * HD * 2;
  constexpr int KS = HD / 16;  // k16 steps over the head dim
  constexpr int DB = HD / 8;   // n8 blocks over the head dim
  const uint32_t sQ = smem_u32(fp_smem);
  const uint32_t sK = sQ + TILE, sV = sK + 2 * TILE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, tq = lane & 3;
  // heavier (later) causal tiles first
  const int mtile = a.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int m0 = mtile * FP_BM;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kvh = head / a.group;

  pdl_launch_dependents();
  pdl_wait();

  const uint16_t* qp = a.q + b * a.q_bs + head * a.q_hs;
  const uint16_t* kp = a.k + b * a.k_bs + kvh * a.k_hs;
  const uint16_t* vp = a.v + b * a.v_bs + kvh * a.v_hs;

  // keys visible to this tile
  int kv_end = a.kv_len;
  if (a.causal) kv_end = min(kv_end, a.q_pos0 + m0 + FP_BM);
  const int ntiles = (kv_end + FP_BN - 1) / FP_BN;

  load_tile<HD>(sQ, qp, a.q_rs, m0, a.S - 1, tid);
  cp_async_commit();
  if (ntiles > 0) {
    load_tile<HD>(sK, kp, a.k_rs, 0, a.kv_len - 1, tid);
    load_tile<HD>(sV, vp, a.v_rs, 0, a.kv_len - 1, tid);
  }
  cp_async_commit();
  cp_async_wait<1>();
  __syncthreads();

  // Q fragments: rows warp*16 .. +16
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int r = warp * 16 + (lane & 15);
    const int c = ks * 2 + (lane >> 4);
    ldsm_x4(sQ + swz<HD>(r, c), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  float o[DB][4];
#pragma unroll
  for (int d = 0; d < DB; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int qrow0 = a.q_pos0 + m0 + warp * 16 + g;  // absolute position of this thread's first row

  for (int nt = 0; nt < ntiles; ++nt) {
    const int buf = nt & 1;
    if (nt + 1 < ntiles) {
      load_tile<HD>(sK + (buf ^ 1) * TILE, kp, a.k_rs, (nt + 1) * FP_BN, a.kv_len - 1, tid);
      load_tile<HD>(sV + (buf ^ 1) * TILE, vp, a.v_rs, (nt + 1) * FP_BN, a.kv_len - 1, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t kt = sK + buf * TILE, vt = sV + buf * TILE;

    // ---- S = Q K^T (16 x 64 per warp) ----
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int nb2 = 0; nb2 < 4; ++nb2) {
        uint32_t b0, b1, b2, b3;
        const int key = nb2 * 16 + ((lane >> 4) << 3) + (lane & 7);
        const int c = ks * 2 + ((lane >> 3) & 1);
        ldsm_x4(kt + swz<HD>(key, c), b0, b1, b2, b3);
        mma_bf16(s[nb2 * 2], qf[ks], b0, b1);
        mma_bf16(s[nb2 * 2 + 1], qf[ks], b2, b3);
      }
    }
    // ---- scale, mask, online softmax ----
    const int key0 = nt * FP_BN;
    const bool need_mask = (key0 + FP_BN > a.kv_len) || (a.causal && key0 + FP_BN - 1 > a.q_pos0 + m0);
    float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[nb][e] * a.scale_log2;
        if (need_mask) {
          const int key = key0 + nb * 8 + tq * 2 + (e & 1);
          const int qr = qrow0 + (e >> 1) * 8;
          if (key >= a.kv_len || (a.causal && key > qr)) x = -INFINITY;
        }
        s[nb][e] = x;
        mt[e >> 1] = fmaxf(mt[e >> 1], x);
      }
    }
    float corr[2], mu[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mt[h] = fmaxf(mt[h], __shfl_xor_sync(0xffffffffu, mt[h], 1));
      mt[h] = fmaxf(mt[h], __shfl_xor_sync(0xffffffffu, mt[h], 2));
      const float mn = fmaxf(mrow[h], mt[h]);
      mu[h] = (mn == -INFINITY) ? 0.f : mn;
      corr[h] = exp2f(mrow[h] - mu[h]);
      mrow[h] = mn;
    }
    float ps[2] = {0.f, 0.f};
    uint32_t pf[4][4];  // P as A fragments for the 4 k16 steps over keys
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      const float p0 = exp2f(s[nb][0] - mu[0]), p1 = exp2f(s[nb][1] - mu[0]);
      const float p2 = exp2f(s[nb][2] - mu[1]), p3 = exp2f(s[nb][3] - mu[1]);
      ps[0] += p0 + p1; ps[1] += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) lrow[h] = lrow[h] * corr[h] + ps[h];
#pragma unroll
    for (int d = 0; d < DB; ++d) {
      o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
    // ---- O += P V ----
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int d2 = 0; d2 < DB / 2; ++d2) {
        uint32_t b0, b1, b2, b3;
        const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
        const int c = d2 * 2 + (lane >> 4);
        ldsm_x4_t(vt + swz<HD>(key, c), b0, b1, b2, b3);
        mma_bf16(o[d2 * 2], pf[ks], b0, b1);
        mma_bf16(o[d2 * 2 + 1], pf[ks], b2, b3);
      }
    }
    __syncthreads();  // everyone is done with `buf` before it is refilled
  }
  cp_async_wait<0>();

  // ---- finalise: O / l, stage through the warp's own Q rows, 16-byte stores ----
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
    lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
    lrow[h] = lrow[h] > 0.f ? 1.f / lrow[h] : 0.f;
  }
  __syncwarp();
#pragma unroll
  for (int d = 0; d < DB; ++d) {
    const int r0 = warp * 16 + g;
    const uint32_t w0 = pack_bf16(o[d][0] * lrow[0], o[d][1] * lrow[0]);
    const uint32_t w1 = pack_bf16(o[d][2] * lrow[1], o[d][3] * lrow[1]);
    // element column d*8 + tq*2 -> chunk d, byte (tq*4) inside the chunk
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(sQ + swz<HD>(r0, d) + tq * 4), "r"(w0) : "memory");
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(sQ + swz<HD>(r0 + 8, d) + tq * 4), "r"(w1) : "memory");
  }
  __syncwarp();
  uint16_t* op = a.o + b * a.o_bs + head * a.o_hs;
  constexpr int CPR = HD / 8;
  for (int i = lane; i < 16 * CPR; i += 32) {
    const int r = warp * 16 + i / CPR, c = i % CPR;
    const int gr = m0 + r;
    if (gr < a.S) {
      uint4 w;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(sQ + swz<HD>(r, c)));
      *reinterpret_cast<uint4*>(op + (long)gr * a.o_rs + c * 8) = w;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_flash_prefill(void* out, const void* q, const void* k, const void* v,
                                  int batch, int S, int kv_len, int q_pos0, int n_q, int n_kv, int hd,
                                  int64_t q_bs, int64_t q_rs, int64_t q_hs,
                                  int64_t k_bs, int64_t k_rs, int64_t k_hs,
                                  int64_t v_bs, int64_t v_rs, int64_t v_hs,
                                  int64_t o_bs, int64_t o_rs, int64_t o_hs,
                                  int causal, float scale, int flags, b200_stream_t stream) {
  if (!out || !q || !k || !v) return B200_ERR_ARG;
  if (batch <= 0 || S <= 0 || kv_len <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 ||
      (hd != 64 && hd != 128) || batch > 65535 || n_q > 65535)
    return B200_ERR_SHAPE;
  const int64_t strides[12] = {q_bs, q_rs, q_hs, k_bs, k_rs, k_hs, v_bs, v_rs, v_hs, o_bs, o_rs, o_hs};
  for (int i = 0; i < 12; ++i) if (strides[i] & 7) return B200_ERR_ALIGN;
  if (((uintptr_t)out & 15) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15))
    return B200_ERR_ALIGN;
  FpArgs a;
  a.o = (uint16_t*)out; a.q = (const uint16_t*)q; a.k = (const uint16_t*)k; a.v = (const uint16_t*)v;
  a.q_bs = q_bs; a.q_rs = q_rs; a.q_hs = q_hs; a.k_bs = k_bs; a.k_rs = k_rs; a.k_hs = k_hs;
  a.v_bs = v_bs; a.v_rs = v_rs; a.v_hs = v_hs; a.o_bs = o_bs; a.o_rs = o_rs; a.o_hs = o_hs;
  a.S = S; a.kv_len = kv_len; a.q_pos0 = q_pos0; a.group = n_q / n_kv; a.causal = causal ? 1 : 0;
  a.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((S + FP_BM - 1) / FP_BM, n_q, batch);
  const size_t smem = (size_t)5 * 64 * hd * 2;
  cudaError_t e;
  const bool pdl = (flags & B200_FLAG_PDL) != 0;
  if (hd == 128) {
    static bool set128 = false;
    if (!set128) { cudaFuncSetAttribute(flash_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); set128 = true; }
    e = launch(flash_prefill_kernel<128>, grid, dim3(FP_THREADS), smem, (cudaStream_t)stream, pdl, a);
  } else {
    static bool set64 = false;
    if (!set64) { cudaFuncSetAttribute(flash_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); set64 = true; }
    e = launch(flash_prefill_kernel<64>, grid, dim3(FP_THREADS), smem, (cudaStream_t)stream, pdl, a);
  }
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
