/*
 * b200ops — C ABI of the sm_100a inference kernel library.
 *
 * Every entry point:
 *   - takes plain device pointers, explicit sizes and an explicit stream;
 *   - writes only into caller-provided buffers (nothing is allocated, nothing
 *     synchronises, so every call can sit inside a CUDA-graph capture);
 *   - returns B200_OK or a negative B200_ERR_* code (bad shape / alignment /
 *     launch failure) and never throws.
 *
 * "Reference" citations name the file of hoid-ai/hoid-optimized-models whose
 * kernel or library call the entry point replaces (path within that project).
 *
 * Conventions: bf16 tensors are raw uint16 storage; `*_dtype` arguments use
 * B200_BF16 / B200_F32; weight matrices are row-major [N, K] exactly as the
 * HuggingFace checkpoints store them (y = x W^T).  Positions / lengths that
 * change from step to step are read from DEVICE scalars so that one captured
 * graph serves every step (the reference's dyn_dims[14] / dyn_dims[18]).
 */
#ifndef B200OPS_H_
#define B200OPS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b200_stream_t;

enum { B200_BF16 = 0, B200_F32 = 1 };

enum {
  B200_OK = 0,
  B200_ERR_SHAPE = -1,     /* unsupported size / divisibility */
  B200_ERR_ALIGN = -2,     /* pointer or leading dimension not 16-byte aligned */
  B200_ERR_LAUNCH = -3,    /* CUDA reported a launch error */
  B200_ERR_ARG = -4,       /* null pointer / bad enum */
  B200_ERR_TIMEOUT = -5,   /* a bounded device-side wait expired (status word) */
  B200_ERR_DRIVER = -6,    /* driver entry point (tensor-map encode) unavailable */
  B200_ERR_SCRATCH = -7,   /* request needs more scratch than the library's fixed array holds */
  B200_ERR_NUMERIC = -8    /* non-finite input where an index is derived from it (status word) */
};

/* launch flags */
enum {
  B200_FLAG_PDL = 1        /* launch with programmatic stream serialization */
};

/* GEMV / GEMM epilogues */
enum {
  B200_EPI_NONE = 0,
  B200_EPI_SWIGLU = 1,     /* rows interleaved (gate_j, up_j): out[j] = silu(y[2j]) * y[2j+1] */
  B200_EPI_GELU = 2,       /* exact erf GELU on (y + bias) */
  B200_EPI_GEGLU = 3       /* GEMM only. W is a stock [2 O, K] GEGLU projection, value half first:
                              out[M, O] = (x Wv^T + bv) * gelu_erf(x Wg^T + bg) */
};

int b200_version(void);
/* Kernel tuning knobs (process-wide, host side).  Keys 2 and 3 selected kernel variants that
 * were measured slower and removed; they are accepted and ignored. */
enum { B200_TUNE_GEMV = 0 /* GEMV register blocking: 0 = 8 loads per batch, 2 CTAs per SM (the
                             measured best); 1 = 4 loads / 4 CTAs; 2 = 4 loads / 3 CTAs */,
       B200_TUNE_GEMM_BN = 1 /* force the GEMM tile width: 256 / 128 / 64 */,
       B200_TUNE_GEMV_NORM = 4 /* RMSNorm prologue: 0 scale the row sums, 1 normalise x in smem */,
       B200_TUNE_WAIT_KTICKS = 5 /* clock budget of every bounded device-side wait on another rank
                                    or on the other CTAs of a persistent kernel, in units of 1024
                                    ticks; 0 = the default of about two seconds */ };
int b200_set_tuning(int key, int value);
/* Number of SMs the library sizes its grids for (148 on B200). */
int b200_sm_count(void);

/* ---------------------------------------------------------------------------
 * a1. Decode GEMV  y[N] = W[N,K] . x[K]   (bf16 weights, fp32 accumulate)
 * Reference: torch.matmul(h, W.t(), out=) at models/llama31-8b/llama31_optimized.py:391-418,
 * models/qwen3-4b/qwen3_optimized.py:391-419, models/qwen3-30b-a3b/qwen3_optimized.py:472-494,
 * models/whisper-large-v3/whisper_decoder_optimized.py:416-447 and the fused q/k/v GEMV
 * models/whisper-large-v3/kernels/whisper_qkv_prefetch10_raw_b128_k.cu:2-21.
 *
 * Optional fusions (pass NULL to disable):
 *   norm_w  : RMSNorm prologue, x <- x * rsqrt(mean(x^2) + eps) * norm_w   (bf16 [K])
 *             (replaces models/llama31-8b/kernels/rmsnorm_prefetch16_k.cu:4-22 at s = 1)
 *   norm_beta : with norm_w, LayerNorm prologue instead: x <- (x - mean) * rsqrt(var + eps) *
 *             norm_w + norm_beta, two-pass fp32 statistics (replaces the stand-alone LayerNorm
 *             launches of models/whisper-large-v3/whisper_decoder_optimized.py:416-447)
 *   bias    : bf16 [N] added to y
 *   resid   : y = resid + W x; may alias y (replaces kernels/add_bf16_vec8_k.cu:10-21)
 *   epilogue: B200_EPI_SWIGLU over interleaved gate/up rows, output length N/2
 *             (replaces kernels/silu_mul_vec8_fast_k.cu:12-23), or B200_EPI_GELU.
 * K must be a multiple of 256; w rows 16-byte aligned (ldw % 8 == 0).
 */
int b200_gemv_bf16(const void* x, int x_dtype, const void* w, void* y, int y_dtype,
                   int K, int N, int ldw,
                   const void* norm_w, const void* norm_beta, float eps,
                   const void* bias,
                   const void* resid, int resid_dtype,
                   int epilogue, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * (e) Tensor-parallel decode without a collective library call: the all-reduce that follows
 * o_proj / down_proj (no counterpart in the single-GPU reference; its call sites are
 * models/llama31-8b/llama31_optimized.py:407,414) is fused into the GEMVs on both sides of it.
 * Set-up (once per process, may allocate): every rank allocates b200_tp_buffer_bytes() with
 * b200_tp_alloc, exchanges the 64-byte IPC handles, maps its peers with b200_tp_open and
 * registers the table with b200_tp_create (returns a context id >= 0; at most 16 links per
 * process, each lives until the process exits).
 * Per step: b200_gemv_bf16_tp with tp_out >= 0 pushes this rank's partial y into every rank's
 * inbox over NVLink, as 8-byte {value, sequence tag} pairs that arrive atomically (or, with
 * tuning key B200_TUNE_TP_PROTOCOL = 1, as plain stores followed by one system-scope release
 * flag per rank); with tp_in >= 0 it waits - bounded, status receives B200_ERR_TIMEOUT on
 * expiry - for all ranks and stages x as the sum of the inboxes in rank order.  tp_in / tp_out number the all-reduces
 * inside one step; b200_tp_advance adds the per-step count to the device-side base so that a
 * captured graph can be replayed.  All ranks must issue the same sequence of calls.
 */
int64_t b200_tp_buffer_bytes(int world, int H);
int b200_tp_alloc(void** ptr, void* ipc_handle_64, int64_t bytes);
int b200_tp_open(void** ptr, const void* ipc_handle_64);
int b200_tp_create(void* const* bufs, int world, int rank, int H);
int b200_tp_advance(int ctx, int inc, int flags, b200_stream_t stream);
int b200_gemv_bf16_tp(const void* x, const void* w, void* y, int K, int N, int ldw,
                      const void* norm_w, float eps, const void* bias, const void* resid,
                      int epilogue, int ctx, int tp_in, int tp_out, void* x_out, int* status,
                      int flags, b200_stream_t stream);
/* Expert parallelism: b200_moe_decode_down whose output (this rank's experts' share, + fp32 resid
 * on one rank) is pushed as all-reduce tp_out instead of being stored (the all-reduce after the
 * routed experts has no counterpart in the single-GPU reference; its call site is
 * models/qwen3-30b-a3b/qwen3_optimized.py:494, the down projection of the expert MLP). */
int b200_moe_decode_down_tp(const void* act, const void* w_down, const int* ids, int top_k,
                            int inter, int hidden, int expert_lo, int n_local, const void* resid,
                            int ctx, int tp_out, int* status, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a6. (residual add +) RMSNorm over rows.
 *   sum = a (+ b)                       [rows, N]; a and resid_out (the residual stream) have
 *                                       resid_dtype, the delta b has b_dtype, norm_out out_dtype
 *   resid_out <- sum (optional, rounded to resid_dtype first, as the reference does in bf16)
 *   norm_out  <- sum * rsqrt(mean(sum^2) + eps) * w
 * An fp32 residual stream with bf16 deltas keeps the error against an fp32 model flat over depth.
 * Reference: models/qwen3-4b/kernels/fused_residual_rmsnorm_multi_k.cu:2-54,
 * models/qwen3-30b-a3b/kernels/fullcta_add_rmsnorm_k.cu:2-45,
 * models/llama31-8b/kernels/rmsnorm_prefetch16_k.cu:4-22 (b = NULL).
 * N % 8 == 0, N <= 16384.
 */
int b200_add_rmsnorm(void* resid_out, void* norm_out, int out_dtype,
                     const void* a, int resid_dtype, const void* b, int b_dtype,
                     const void* w, int rows, int N, float eps,
                     int flags, b200_stream_t stream);

/* (bias +) (residual add +) LayerNorm over rows, two-pass fp32 statistics.
 *   sum = x (+ bias) (+ resid); with in_dtype bf16 each addition is rounded to bf16 like the reference
 *   resid_out <- sum (optional); norm_out <- (sum - mean) * rsqrt(var + eps) * gamma + beta
 * Reference: models/bge-m3/kernels/bge_bias_residual_ln_warp_packed_k.cu:2-67,
 * models/whisper-large-v3/kernels/whisper_ordered_residual_ln_replicated_k.cu:32-111,
 * whisper_resid_ln_oneshot_vec2_k.cu:2-24, whisper_ln_volatile_warptail_k.cu:6-75.
 */
int b200_add_layernorm(void* resid_out, void* norm_out, int out_dtype,
                       const void* x, const void* bias, const void* resid, int in_dtype,
                       const void* gamma, const void* beta,
                       int rows, int N, float eps, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a7. (QK-RMSNorm +) RoPE + KV-cache write for `s` new tokens.
 *   qkv      : [s, (n_q + 2 n_kv) * hd] packed projections (q heads, k heads, v heads)
 *   q_out    : [s, n_q * hd]
 *   kcache / vcache : [n_kv, max_seq, hd] bf16; rows pos0 + t are written
 *   qn_w/kn_w: optional bf16 [hd] per-head RMSNorm weights (Qwen3)
 *   cos/sin  : fp32 [max_seq, hd/2]; rotate-half convention
 *   pos_dev  : device int32, position of the first new token
 * Reference: models/qwen3-4b/qwen3_native_gen.py:16-92 (prepare_qkv_k),
 * models/qwen3-30b-a3b/kernels/prepare_qkv_k.cu:5-76,
 * models/llama31-8b/llama31_native_gen.py:30-110 (apply_rope_q_k, apply_rope_kv_k, cache_write_k).
 */
int b200_qk_rope_cache(void* q_out, int q_dtype, void* kcache, void* vcache,
                       const void* qkv, int qkv_dtype,
                       const void* qn_w, const void* kn_w,
                       const float* cos_t, const float* sin_t,
                       const int* pos_dev, int s, int n_q, int n_kv, int hd,
                       int max_seq, float eps, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a3 + a4. Split-KV GQA flash-decode with the log-sum-exp combine fused in.
 *   q      : [n_q, hd]; head h uses kv head h / (n_q / n_kv)
 *   kcache : element (kvh, j, d) at kcache[kvh * kv_head_stride + j * kv_row_stride + d]
 *   kv_len_dev : device int32, number of keys to attend to (position + 1)
 *   workspace  : fp32 scratch of b200_flash_decode_workspace_bytes() bytes; its first
 *                n_kv int32 words are arrival counters that must be zero before the
 *                first call (the kernel leaves them zero).
 *   n_splits   : CTAs per kv head (fixed at capture time; idle splits exit early)
 * Reference: models/llama31-8b/kernels/dense_cached_attention_residue_partial_k.cu:19-124 and
 * dense_cached_attention_residue_combine_k.cu:7-36;
 * models/qwen3-30b-a3b/kernels/attn_gqa8_subsplit64_partial_k.cu:2-68 with its three reduce
 * kernels; models/whisper-large-v3/kernels/whisper_cross_bias_partial.triton.py:1-25.
 * hd in {64, 128}; n_q / n_kv in {1, 2, 4, 8}.
 */
int64_t b200_flash_decode_workspace_bytes(int n_q, int n_kv, int hd, int n_splits);
int b200_flash_decode(void* out, int out_dtype, const void* q, int q_dtype,
                      const void* kcache, const void* vcache, const int* kv_len_dev,
                      void* workspace, int n_q, int n_kv, int hd,
                      int64_t kv_head_stride, int64_t kv_row_stride,
                      int n_splits, float scale, int flags, b200_stream_t stream);

/* a2 + a3 + a4 in one launch for the decode step (saves one launch per layer): q, k and v of
 * the new position (row kv_len - 1) are read from the packed fp32 projection row
 * [q heads | k heads | v heads]; the kernel applies (QK-RMSNorm +) rotate-half RoPE in its
 * prologue exactly as b200_qk_rope_cache does, the CTA whose slice ends with the new row appends
 * k / v (bf16) to the cache, and attention runs over rows [0, kv_len).  cos_t / sin_t are the
 * [max_seq, hd / 2] fp32 tables; qn_w / kn_w nullable together.  Same workspace as
 * b200_flash_decode.  Reference: the prepare_qkv + attention pair of
 * models/llama31-8b/llama31_optimized.py:398-405 (qwen3: qwen3_optimized.py:395-404). */
int b200_rope_flash_decode(void* out, int out_dtype, const float* qkv, void* kcache, void* vcache,
                           const float* cos_t, const float* sin_t, const void* qn_w,
                           const void* kn_w, float eps, const int* kv_len_dev, void* workspace,
                           int n_q, int n_kv, int hd, int64_t kv_head_stride,
                           int64_t kv_row_stride, int max_seq, int n_splits, float scale,
                           int flags, b200_stream_t stream);

/* Flash-decode without any allocation (no counterpart in the reference).
 *
 * Same computation and arguments as b200_flash_decode, minus the workspace: the split
 * records and arrival counters live in a 2 MiB array that is part of the library image
 * (b200_flash_decode_static_max_bytes()), so a caller that is not allowed to allocate device
 * memory - a plugin inside another framework's memory pool, an allocation-free serving loop,
 * a process with a fixed memory budget - can still run decode attention.  Every GPU that
 * loads the library holds the array until the process exits.
 *   - Returns B200_ERR_SCRATCH when b200_flash_decode_workspace_bytes(n_q, n_kv, hd, n_splits)
 *     exceeds the array; nothing is launched in that case.
 *   - The first call on each device looks up the array's device address; make that call
 *     with the device current and before any stream capture.
 *   - All calls share the array.  Each call clears the counters it needs on `stream` first,
 *     so calls on one stream are safe back to back; calls that overlap on the GPU (other
 *     streams, other threads) race on the array and give wrong results.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 */
int64_t b200_flash_decode_static_max_bytes(void);
int b200_flash_decode_static(void* out, int out_dtype, const void* q, int q_dtype,
                             const void* kcache, const void* vcache, const int* kv_len_dev,
                             int n_q, int n_kv, int hd,
                             int64_t kv_head_stride, int64_t kv_row_stride,
                             int n_splits, float scale, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a13. All layers of one batch-1 decode step of a dense decoder in ONE persistent launch
 * (cooperative, one CTA per SM): q|k|v GEMV with RMSNorm prologue -> (QK-norm +) RoPE + cache
 * append + split-KV attention + combine -> o_proj + residual -> gate|up GEMV with RMSNorm prologue
 * and SwiGLU -> down + residual, layer after layer.  The phases hand their vectors to one another
 * as self-validating {value, tag} pairs that the next phase polls (no grid-wide barrier), and the
 * next matrix's first weights are already in flight across every wait.
 * Reference: the body of the captured decode graph, models/llama31-8b/llama31_optimized.py:385-419
 * and models/qwen3-4b/qwen3_optimized.py:385-420 (18 launches per layer there).
 *
 * Set-up (once, synchronous copy): b200_decode_layers_plan writes the phase table into plan_dev
 * (b200_decode_layers_plan_bytes(n_layers) bytes of device memory) from host arrays of per-layer
 * device pointers: w_qkv[i] [q_size + 2 kv_size, hidden], w_o[i] [hidden, q_size], w_gu[i]
 * [2 inter, hidden] with gate / up rows interleaved, w_down[i] [hidden, inter] (bf16, HuggingFace
 * [N, K] layout, contiguous), ln1[i] / ln2[i] RMSNorm weights, kcache[i] / vcache[i] the layer's
 * [n_kv, max_seq, hd] bf16 caches, qn_w / kn_w the QK-norm weights (both arrays NULL for models
 * without).  h is the fp32 residual stream [hidden]: the embedded token on entry, the last
 * layer's output on exit.  sync_ws is b200_decode_layers_sync_bytes(...) bytes of device memory,
 * 256-byte aligned, ZERO before the first launch and owned by this plan (launch counter + the
 * pair vectors).  Sizes are the per-rank ones; hidden, q_size, inter % 256 == 0 and <= 16384.
 * tp_ctx >= 0 (a b200_tp_create context): the all-reduces after o_proj and down are the fused
 * peer-memory exchange of b200_gemv_bf16_tp, numbered 2 i and 2 i + 1 within the step; h is then
 * NOT written: the consumer of all-reduce 2 n_layers - 1 (b200_gemv_bf16_tp with tp_in, x_out)
 * produces it.
 *
 * Per step: b200_decode_layers.  kv_len_dev[0] - 1 is the new position; fd_workspace as for
 * b200_flash_decode; status (required) receives B200_ERR_TIMEOUT if a bounded wait expired - the
 * outputs are then invalid.  n_kv * n_splits <= b200_sm_count().  The launch is cooperative and
 * carries no programmatic dependent launch attribute.  Launches that share a plan must not
 * overlap on the GPU.
 */
int64_t b200_decode_layers_plan_bytes(int n_layers);
int64_t b200_decode_layers_sync_bytes(int hidden, int q_size, int kv_size, int inter);
int b200_decode_layers_plan(void* plan_dev, void* sync_ws, int n_layers, const void* const* w_qkv,
                            const void* const* w_o, const void* const* w_gu,
                            const void* const* w_down, const void* const* ln1,
                            const void* const* ln2, const void* const* kcache,
                            const void* const* vcache, const void* const* qn_w,
                            const void* const* kn_w, float* h, int hidden, int q_size,
                            int kv_size, int inter, int tp_ctx);
int b200_decode_layers(const void* plan_dev, int n_layers, const float* cos_t, const float* sin_t,
                       const int* kv_len_dev, void* fd_workspace, void* sync_ws, int n_q, int n_kv,
                       int hd, int64_t kv_head_stride, int64_t kv_row_stride, int max_seq,
                       int n_splits, float scale, float eps, int tp_ctx, int* status, int flags,
                       b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a2. Prefill / encoder GEMM  Y[M,N] = X[M,K] W[N,K]^T  (bf16 in, fp32 accumulate in
 * tensor memory, bf16 out; fp32 out for plain / bias / GELU epilogues, e.g. router logits) on
 * tcgen05 tensor cores fed by TMA.
 *   bias  : optional bf16 [N];  resid : optional bf16 [M, ldr], Y = resid + X W^T (may alias y)
 *   epilogue: B200_EPI_SWIGLU (W rows interleaved gate/up, Y is [M, N/2]), B200_EPI_GELU, or
 *             B200_EPI_GEGLU (W = [value half; gate half] as torch.chunk(2, -1) splits the stock
 *             projection, bias likewise, Y is [M, N/2]; both halves of an output tile come from
 *             one N = 256 MMA.  Replaces the dual-GEMM of
 *             models/sdxl/kernels/dual_geglu.cutedsl.py, called at
 *             models/sdxl/sdxl_optimized.py:380-393)
 *   status: optional device int32; receives B200_ERR_TIMEOUT if a bounded wait expired
 * Reference: torch.matmul at M = P, models/llama31-8b/llama31_optimized.py:479-499;
 * torch.mm(out=) models/bge-m3/bge_optimized.py:340-349; the CuTe-DSL GEMMs
 * models/whisper-large-v3/kernels/fc1_persistent_exact_gelu_entry.cutedsl.py:173-759,
 * triple_qkv_entry.cutedsl.py:150-804, conv2_blackwell_efc_bias_entry.cutedsl.py:1-42.
 * K % 8 == 0, N % 8 == 0 (N % 16 for SwiGLU), all leading dimensions % 8 == 0.
 */
int b200_gemm_bf16(const void* x, const void* w, void* y, int y_dtype, int M, int N, int K,
                   int ldx, int ldw, int ldy, const void* bias, const void* resid, int ldr,
                   int epilogue, int* status, int flags, b200_stream_t stream);

/* a11. Grouped expert GEMM: rows of x are sorted by expert, offsets[e] (device int32
 * [n_experts + 1]) is the first row of expert e, w is [n_experts, N, K]:
 *   y[r, :] = x[r, :] w[e(r)]^T   (+ SwiGLU over interleaved gate/up rows)
 * Reference: torch._grouped_mm, models/qwen3-30b-a3b/qwen3_optimized.py:583-585.
 */
int b200_moe_grouped_gemm(const void* x, const void* w, void* y, const int* offsets,
                          int n_experts, int rows, int N, int K, int ldx, int ldy,
                          int epilogue, int* status, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a5. Prefill / encoder flash attention (never materialises the score matrix).
 *   q, k, v, out are bf16 with explicit element strides (batch, row, head); query row i of
 *   head h uses kv head h / (n_q / n_kv); causal: row i sees keys <= q_pos0 + i;
 *   kv_len keys are valid.  The strides let K/V be read straight from the decode cache
 *   ([n_kv, max_seq, hd]: row stride hd, head stride max_seq * hd) or from a packed
 *   q|k|v projection (encoder).
 * Reference: models/llama31-8b/kernels/fmha_prefill_elastic.triton.py:1-58 (causal GQA),
 * models/bge-m3/kernels/bge_fa2_attention_nokb_postvb_late.ptx:1-2329 (bidirectional d64),
 * flash-attn-4 call at models/whisper-large-v3/whisper_optimized.py:356-360.
 * hd in {64, 128}; all strides multiples of 8 elements; q_pos0 >= 0, kv_len >= 1, scale > 0
 * (B200_ERR_SHAPE / B200_ERR_ARG otherwise).
 * Runs on the tcgen05 tensor cores: persistent CTAs, TMA-fed, two 128-row query streams per
 * CTA, scores, probabilities and output accumulators in tensor memory, 128 x 128 tiles.  The
 * softmax raises a row's reference maximum only when it grows by more than 2^8, which is exact
 * after the final division by the row sum.  Keys are consumed in tiles of 128: the rows of k and
 * v between kv_len and the end of the last tile are masked to probability zero but still enter
 * the second MMA as 0 * v, so v must hold finite values there (rows past the end of the whole
 * view are zero-filled by the TMA unit; a zero-initialised cache, as the engines use, is enough).  Each of q / k / v must be expressible as a 2D row-major view: the batch stride a
 * multiple of the row stride, and the head stride either a multiple of the row stride (heads are
 * row blocks, as in the KV cache) or smaller than it (heads are column blocks, as in packed
 * projections).  status (nullable) receives B200_ERR_TIMEOUT if a bounded wait expired.
 */
int b200_flash_prefill_tc(void* out, const void* q, const void* k, const void* v,
                          int batch, int S, int kv_len, int q_pos0, int n_q, int n_kv, int hd,
                          int64_t q_bs, int64_t q_rs, int64_t q_hs,
                          int64_t k_bs, int64_t k_rs, int64_t k_hs,
                          int64_t v_bs, int64_t v_rs, int64_t v_hs,
                          int64_t o_bs, int64_t o_rs, int64_t o_hs,
                          int causal, float scale, int* status, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a9. MoE router: fp32 softmax over E logits -> top-k (ties: lowest expert index) ->
 * weights renormalised over the selected experts; ids in descending-probability order.
 *   logits: [s, E] fp32 or bf16; ids int32 [s, top_k]; wts fp32 [s, top_k]
 *   round_bf16: round the weights through bf16 like the reference kernel does
 *   status: optional device int32; a token with a non-finite logit gets valid ids (its
 *           probabilities count as zero) and status receives B200_ERR_NUMERIC
 * Reference: models/qwen3-30b-a3b/kernels/moe_router_parallel_topk_k.cu:2-111 (decode) and
 * the torch softmax/topk/renorm at models/qwen3-30b-a3b/qwen3_optimized.py:569-572 (prefill).
 * E % 32 == 0, E <= 256, top_k <= 32.
 */
int b200_moe_router(int* ids, float* wts, const void* logits, int logits_dtype, int s, int E,
                    int top_k, int round_bf16, int* status, int flags, b200_stream_t stream);
/* a11. Expert-major permutation of the s * top_k (token, slot) pairs: a stable counting sort
 * by expert id, identical to torch.argsort(ids.flatten(), stable=True).
 *   order[r]  : flat pair index (token * top_k + slot) at sorted row r
 *   inv[p]    : sorted row of pair p (nullable)
 *   offsets   : int32 [E + 1], first sorted row of every expert (offsets[E] = pairs)
 *   workspace : b200_moe_permute_workspace_bytes(pairs, E) bytes
 *   status    : optional device int32; an id outside [0, E) is sorted as expert 0 (nothing is
 *               indexed out of range) and status receives B200_ERR_ARG
 * Reference: models/qwen3-30b-a3b/qwen3_optimized.py:573-581 (argsort + scatter_add + cumsum).
 */
int64_t b200_moe_permute_workspace_bytes(int pairs, int E);
int b200_moe_permute(int* order, int* inv, int* offsets, const int* ids, int pairs, int E,
                     void* workspace, int* status, int flags, b200_stream_t stream);
/* xg[r, :] = x[order[r] / top_k, :]  (bf16 rows of H elements).
 * Reference: index_select at models/qwen3-30b-a3b/qwen3_optimized.py:582. */
int b200_moe_gather_rows(void* xg, const void* x, const int* order, int rows, int top_k, int H,
                         int flags, b200_stream_t stream);
/* out[t, :] = (resid[t, :] +) sum_slot wts[t, slot] * y[inv[t * top_k + slot], :]
 * (fp32 accumulation in slot order, one bf16 rounding).  With ids != NULL only the pairs whose
 * expert lies in [expert_lo, expert_lo + n_local) are summed (expert parallelism).
 * Reference: mul_ / index_copy_ / sum at models/qwen3-30b-a3b/qwen3_optimized.py:586-590. */
int b200_moe_combine(void* out, const void* y, const int* inv, const float* wts,
                     const void* resid, const int* ids, int expert_lo, int n_local,
                     int tokens, int top_k, int H, int flags, b200_stream_t stream);

/* a10. Decode-time expert MLP on the top_k selected experts (weight streaming, HBM bound).
 *   w_gu  : [E, 2 * inter, hidden] bf16 with gate/up rows INTERLEAVED (row 2j = gate_j,
 *           row 2j + 1 = up_j; a load-time repack of HuggingFace's gate-rows-then-up-rows)
 *   w_down: [E, hidden, inter] bf16
 *   gate_up: act[slot, j] = wts[slot] * silu(g_j) * u_j with optional RMSNorm prologue on x
 *   down  : y[d] = (resid[d] +) sum_slot w_down[ids[slot]][d, :] . act[slot, :]
 * Reference: models/qwen3-30b-a3b/kernels/moe_gate_up_silu_k.cu:2-32 and
 * moe_down_accum_k.cu:2-33.  hidden % 256 == 0, inter % 256 == 0.
 * Expert parallelism: w_gu / w_down hold experts [expert_lo, expert_lo + n_local) only; slots
 * routed elsewhere contribute zero, and the ranks' outputs are summed by the caller.
 */
int b200_moe_decode_gate_up(void* act, const void* x, int x_dtype, const void* norm_w, float eps,
                            const void* w_gu, const int* ids, const float* wts, int top_k,
                            int inter, int hidden, int expert_lo, int n_local, int flags,
                            b200_stream_t stream);
int b200_moe_decode_down(void* y, int y_dtype, const void* act, const void* w_down,
                         const int* ids, int top_k, int inter, int hidden,
                         int expert_lo, int n_local,
                         const void* resid, int resid_dtype, int flags, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * a8 / a12 small ops.
 */
/* out[r, :] = table[ids[r], :]  (bf16 table; out bf16 or fp32).
 * Reference: embedding_k, models/llama31-8b/llama31_native_gen.py:17-27. */
int b200_embed_gather(void* out, int out_dtype, const void* table, const int* ids,
                      int rows, int H, int flags, b200_stream_t stream);
/* out[b, :] = x_b / max(||x_b||_2, eps) with x_b the bf16 row at x + b * row_stride (the first
 * token of sequence b): CLS pooling + L2 normalisation to fp32 [batch, H].
 * Reference: models/bge-m3/kernels/bge_pool_k.cu:1. */
int b200_cls_pool_l2(float* out, const void* x, int batch, int64_t row_stride, int H, float eps,
                     int flags, b200_stream_t stream);
/* out = silu(gate) * up, elementwise over n values (bf16).
 * Reference: models/llama31-8b/kernels/silu_mul_vec8_fast_k.cu:12-23. */
int b200_silu_mul(void* out, const void* gate, const void* up, int64_t n,
                  int flags, b200_stream_t stream);
/* Greedy head: idx_out[0] = argmax(logits[0:n]) (lowest index on ties), fp32 logits.
 * Reference: logits.argmax() on the host side, models/llama31-8b/llama31_optimized.py:517-518. */
/* workspace: b200_argmax_workspace_bytes() bytes, first word zero before the first call
 * (the kernel leaves it zero); max_out (nullable) receives the winning logit; idx_base is
 * added to the index (vocabulary shard offset). */
int b200_argmax_f32(int* idx_out, float* max_out, const float* logits, int n, int idx_base,
                    void* workspace, int flags, b200_stream_t stream);
/* On-device greedy step: cand is n records {float value; int32 index} (one per tensor-parallel
 * rank); the best (highest value, lowest index on ties) becomes tok_out[0], is appended to
 * log[state[2]] and state = {position, kv_len, generated} is advanced by one.  Removes the
 * per-token host round trip of models/llama31-8b/llama31_optimized.py:438-442,517-518. */
int b200_greedy_select(int* tok_out, const void* cand, int n, int* state, int* log, int log_cap,
                       int flags, b200_stream_t stream);
int64_t b200_argmax_workspace_bytes(int n);

#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H_ */
