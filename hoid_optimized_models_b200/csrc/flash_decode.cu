// Split-KV GQA flash-decode with the log-sum-exp combine fused into the same launch.
//
// Grid (n_splits, n_kv).  A CTA owns one kv head and one contiguous slice of the
// context and serves all G = n_q / n_kv query heads of the group from a single
// pass over K and V, so each cache byte is read from HBM once per step.
//
// Inside the CTA a key row (HD bf16) is spread over HD/8 lanes, 16 bytes each:
// a warp-wide 128-bit load covers 32/(HD/8) adjacent keys = 512 contiguous
// bytes.  Each lane group keeps its own online-softmax state (m, l, acc) in
// registers and the groups are merged through shared memory at the end.  The
// CTA then publishes its record to the workspace and bumps a per-kv-head
// arrival counter; the CTA that arrives last merges all records of that head
// and writes the output (fixed split order, so results do not depend on
// arrival order).  No CTA ever waits on another.
#include "common.cuh"

namespace b200 {

constexpr int kFdThreads = 128;
constexpr int kFdWarps = kFdThreads / 32;
constexpr int kFdU = 4;  // keys in flight per lane group per iteration

struct FdArgs {
  void* out; const void* q; const uint16_t* k; const uint16_t* v; const int* kv_len;
  int* counters; float* recs;
  int n_q, n_kv, n_splits, out_dtype, q_dtype;
  long head_stride, row_stride;  // elements
  float scale_log2;
};

template <int HD, int G>
__global__ void __launch_bounds__(kFdThreads) flash_decode_kernel(FdArgs a) {
  constexpr int LPK = HD / 8;          // lanes per key
  constexpr int KPW = 32 / LPK;        // keys per warp-wide load
  constexpr int NS = kFdWarps * KPW;   // lane groups ("streams") per CTA
  constexpr int REC = HD + 2;
  __shared__ float srec[NS * G * REC];
  __shared__ float sw[NS * G];
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane / LPK, dl = lane % LPK;
  const int split = blockIdx.x, kvh = blockIdx.y;

  pdl_launch_dependents();
  pdl_wait();

  const int kv_len = a.kv_len[0];
  const int per = (kv_len + a.n_splits - 1) / a.n_splits;
  const int k0 = split * per;
  const int k1 = min(kv_len, k0 + per);

  // q for the group's heads, pre-multiplied by scale * log2(e)
  float q[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const size_t qi = ((size_t)(kvh * G + g) * HD) + dl * 8;
    if (a.q_dtype == B200_F32) {
      const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.q) + qi);
      float4 x = p[0], y = p[1];
      q[g][0] = x.x; q[g][1] = x.y; q[g][2] = x.z; q[g][3] = x.w;
      q[g][4] = y.x; q[g][5] = y.y; q[g][6] = y.z; q[g][7] = y.w;
    } else {
      unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.q) + qi), q[g]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) q[g][e] *= a.scale_log2;
  }

  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }

  const uint16_t* kb = a.k + (size_t)kvh * a.head_stride + dl * 8;
  const uint16_t* vb = a.v + (size_t)kvh * a.head_stride + dl * 8;

  // key handled by this lane group in unroll slot u of iteration `it`:
  //   k0 + ((it * U + u) * WARPS + warp) * KPW + sub
  for (int base = k0 + warp * KPW; base < k1; base += kFdU * kFdWarps * KPW) {
    uint4 kw[kFdU], vw[kFdU];
    bool ok[kFdU];
#pragma unroll
    for (int u = 0; u < kFdU; ++u) {
      const int key = base + u * kFdWarps * KPW + sub;
      ok[u] = key < k1;
      kw[u] = make_uint4(0, 0, 0, 0);
      vw[u] = make_uint4(0, 0, 0, 0);
      if (ok[u]) {
        kw[u] = ldg_stream(kb + (size_t)key * a.row_stride);
        vw[u] = ldg_stream(vb + (size_t)key * a.row_stride);
      }
    }
    float s[kFdU][G];
#pragma unroll
    for (int u = 0; u < kFdU; ++u) {
      float kf[8];
      unpack8(kw[u], kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(q[g][e], kf[e], d);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[u][g] = ok[u] ? d : -INFINITY;
      }
    }
    float p[kFdU][G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mt = s[0][g];
#pragma unroll
      for (int u = 1; u < kFdU; ++u) mt = fmaxf(mt, s[u][g]);
      const float mn = fmaxf(m[g], mt);
      const float mu = (mn == -INFINITY) ? 0.f : mn;
      const float corr = exp2f(m[g] - mu);
      float ps = 0.f;
#pragma unroll
      for (int u = 0; u < kFdU; ++u) { p[u][g] = exp2f(s[u][g] - mu); ps += p[u][g]; }
      l[g] = l[g] * corr + ps;
      m[g] = mn;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] *= corr;
    }
#pragma unroll
    for (int u = 0; u < kFdU; ++u) {
      float vf[8];
      unpack8(vw[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(p[u][g], vf[e], acc[g][e]);
    }
  }

  // ---- merge the CTA's lane groups ----
  const int sid = warp * KPW + sub;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float* r = srec + (sid * G + g) * REC;
#pragma unroll
    for (int e = 0; e < 8; ++e) r[dl * 8 + e] = acc[g][e];
    if (dl == 0) { r[HD] = m[g]; r[HD + 1] = l[g]; }
  }
  __syncthreads();
  // per-(stream, head) weights exp2(m_s - M_g); thread t < G handles head t
  if (tid < G) {
    float M = -INFINITY;
    for (int s2 = 0; s2 < NS; ++s2) M = fmaxf(M, srec[(s2 * G + tid) * REC + HD]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float den = 0.f;
    for (int s2 = 0; s2 < NS; ++s2) {
      const float w = exp2f(srec[(s2 * G + tid) * REC + HD] - Mu);
      sw[s2 * G + tid] = w;
      den += srec[(s2 * G + tid) * REC + HD + 1] * w;
    }
    float* wr = a.recs + ((size_t)(kvh * a.n_splits + split) * G + tid) * REC;
    wr[HD] = M;
    wr[HD + 1] = den;
  }
  __syncthreads();
  for (int i = tid; i < G * HD; i += kFdThreads) {
    const int g = i / HD, d = i - g * HD;
    float num = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < NS; ++s2) num = fmaf(srec[(s2 * G + g) * REC + d], sw[s2 * G + g], num);
    a.recs[((size_t)(kvh * a.n_splits + split) * G + g) * REC + d] = num;
  }

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

  const float* rb = a.recs + (size_t)kvh * a.n_splits * G * REC;
  for (int i = tid; i < G * HD; i += kFdThreads) {
    const int g = i / HD, d = i - g * HD;
    float M = -INFINITY;
    for (int sp = 0; sp < a.n_splits; ++sp) M = fmaxf(M, __ldcg(rb + (sp * G + g) * REC + HD));
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float num = 0.f, den = 0.f;
    for (int sp = 0; sp < a.n_splits; ++sp) {
      const float* r = rb + (sp * G + g) * REC;
      const float w = exp2f(__ldcg(r + HD) - Mu);
      den = fmaf(__ldcg(r + HD + 1), w, den);
      num = fmaf(__ldcg(r + d), w, num);
    }
    const float o = den > 0.f ? num / den : 0.f;
    const size_t oi = (size_t)(kvh * G + g) * HD + d;
    if (a.out_dtype == B200_F32) reinterpret_cast<float*>(a.out)[oi] = o;
    else reinterpret_cast<__nv_bfloat16*>(a.out)[oi] = __float2bfloat16(o);
  }
  if (tid == 0) a.counters[kvh] = 0;  // ready for the next launch
}

template <int HD, int G>
static cudaError_t fd_launch(const FdArgs& a, cudaStream_t st, bool pdl) {
  return launch(flash_decode_kernel<HD, G>, dim3(a.n_splits, a.n_kv), dim3(kFdThreads), 0, st, pdl, a);
}

static size_t fd_counter_bytes(int n_kv) { return ((size_t)n_kv * 4 + 255) & ~(size_t)255; }

}  // namespace b200

using namespace b200;

extern "C" int64_t b200_flash_decode_workspace_bytes(int n_q, int n_kv, int hd, int n_splits) {
  if (n_q <= 0 || n_kv <= 0 || n_splits <= 0) return 0;
  return (int64_t)fd_counter_bytes(n_kv) + (int64_t)n_q * n_splits * (hd + 2) * 4;
}

extern "C" int b200_flash_decode(void* out, int out_dtype, const void* q, int q_dtype,
                                 const void* kcache, const void* vcache, const int* kv_len_dev,
                                 void* workspace, int n_q, int n_kv, int hd,
                                 int64_t kv_head_stride, int64_t kv_row_stride,
                                 int n_splits, float scale, int flags, b200_stream_t stream) {
  if (!out || !q || !kcache || !vcache || !kv_len_dev || !workspace) return B200_ERR_ARG;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0 || n_splits <= 0 || n_splits > 65535)
    return B200_ERR_SHAPE;
  if ((kv_row_stride & 7) != 0 || (kv_head_stride & 7) != 0 || ((uintptr_t)kcache & 15) != 0 ||
      ((uintptr_t)vcache & 15) != 0 || ((uintptr_t)q & 15) != 0 || ((uintptr_t)workspace & 15) != 0)
    return B200_ERR_ALIGN;
  FdArgs a;
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
#define FD_CASE(HD_, G_) if (hd == HD_ && G == G_) e = fd_launch<HD_, G_>(a, st, pdl); else
  FD_CASE(128, 1) FD_CASE(128, 2) FD_CASE(128, 4) FD_CASE(128, 8)
  FD_CASE(64, 1) FD_CASE(64, 2) FD_CASE(64, 4) FD_CASE(64, 8)
  return B200_ERR_SHAPE;
#undef FD_CASE
  return e == cudaSuccess ? B200_OK : B200_ERR_LAUNCH;
}
