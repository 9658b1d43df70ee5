/*
 * trinity_b200 — C ABI of the sm_100a kernel backend for Trinity's fused attention-block operators
 * (Vanilla, PreNorm, QKNorm, KeyFormer, RoCo) and standalone RMSNorm.
 *
 * This is the boundary a binding (ctypes, cgo, JNI ...) talks to.  Plain pointers and sizes only; no
 * torch types.  All pointers are DEVICE pointers unless a name ends in `_host`.  Nothing here
 * allocates device memory or synchronises the stream unless its comment says so: the caller owns every
 * buffer, scratch included, exactly as the reference's generated `forward(*tensors)` writes in place
 * into caller tensors (TritonGen.py:541-714).
 *
 * Every entry point returns 0 on success and a negative TRN_E* code when validation fails (nothing is
 * launched then).  trinity_strerror() turns a code into text.  Kernels record device-side problems
 * (a bounded wait that ran out) in a status word read with trinity_last_kernel_status().
 */
#ifndef TRINITY_B200_H_
#define TRINITY_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRINITY_ABI_VERSION 3

/* element types of activations / weights / outputs */
enum { TRN_BF16 = 0, TRN_FP16 = 1 };

/* variants of the attention block (ref_rms.py:29-280) */
enum {
  TRN_VANILLA = 0,   /* ref_rms.py:45-83   */
  TRN_PRENORM = 1,   /* ref_rms.py:101-127 */
  TRN_QKNORM = 2,    /* ref_rms.py:197-231 */
  TRN_KEYFORMER = 3, /* ref_rms.py:147-179 */
  TRN_ROCO = 4       /* ref_rms.py:249-280 */
};

/* where KeyFormer's additive noise comes from */
enum {
  TRN_NOISE_NONE = 0,
  TRN_NOISE_TENSOR = 1, /* `noise` tensor, the reference's input (convert_eval_rms.py:97,201)      */
  TRN_NOISE_GUMBEL = 2  /* counter-based Gumbel(0,1) generated in the kernel from `seed`          */
};

enum {
  TRN_OK = 0,
  TRN_E_NULL = -1,      /* a required pointer is NULL                                   */
  TRN_E_SHAPE = -2,     /* a dimension is zero, negative or not supported by the kernels */
  TRN_E_ALIGN = -3,     /* a pointer or stride breaks the 16-byte rule of vector / TMA access */
  TRN_E_DTYPE = -4,     /* unknown element type                                          */
  TRN_E_VARIANT = -5,   /* unknown variant / flag combination                            */
  TRN_E_WORKSPACE = -6, /* workspace missing or too small                                */
  TRN_E_CUDA = -7,      /* a CUDA runtime / driver call failed (see trinity_last_cuda_error) */
  TRN_E_DEVICE = -8,    /* the current device is not sm_100                               */
  TRN_E_KERNEL = -9     /* a kernel reported a device-side status (timeout)               */
};

int trinity_abi_version(void);
const char* trinity_strerror(int code);
/* text of the last CUDA error seen by this library on the calling thread ("" if none) */
const char* trinity_last_cuda_error(void);
/* Device-side status word of the current device: 0 when every kernel launched so far finished its
 * waits in time.  SYNCHRONISES the device (it reads device memory); call it outside timed regions. */
int trinity_last_kernel_status(int* status_out);
/* The status word is sticky: once a wait ran out, every later kernel of the library on that device returns at
 * once and trinity_last_kernel_status() keeps reporting TRN_E_KERNEL.  This resets it to 0 (SYNCHRONISES the
 * device) after the caller has dealt with the failure. */
int trinity_clear_kernel_status(void);
/* Self-test of that failure path, no reference counterpart (the reference has no device-side failure handling;
 * its harness only catches Python exceptions, vanilla_llama_benchmark.py:329-332): launches one tiny kernel whose
 * only wait is on a barrier nothing arrives at, limited to `limit_us` microseconds (1 .. 100000).  The kernel
 * returns normally — it frees its tensor memory, does not trap and does not spin on — and leaves code 103 in
 * the status word: trinity_last_kernel_status() then returns TRN_E_KERNEL until trinity_clear_kernel_status(). */
int trinity_selftest_wait_timeout(int limit_us, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Standalone RMSNorm:  y[r, :] = x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * gamma[:]
 * Replaces the reference's X2 / X_norm IR tensors (vanilla_llama_benchmark.py:43-45) and the math of
 * ref_rms.py:102-103 (eps = 0, gamma = NULL) and ref_attn.py:348-350 (eps, weight).
 * Reduction in fp32.  `cols` must be a multiple of 8; row strides in elements, multiples of 8.
 * rstd_out (optional, fp32 [rows]) receives rsqrt(mean + eps).
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  void* y;
  const void* gamma; /* [cols] or NULL */
  float* rstd_out;   /* [rows] or NULL */
  int64_t rows, cols;
  int64_t x_row_stride, y_row_stride;
  float eps;
  int dtype;
} TrnRmsArgs;
int trinity_rmsnorm(const TrnRmsArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Addressing of a head-split activation tensor: element (b, s, h, d) lives at
 *   base + b*stride_b + s*stride_s + h*stride_h + d        (strides in elements, d contiguous)
 * which covers the reference's token-major [M, H, D] / [M, N] tensors, its head-major [H, M, D]
 * tensors and the head-major caches [H, P+M, D] (convert_eval_rms.py:62-108).
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  void* ptr;
  int64_t stride_b, stride_s, stride_h;
} TrnHeadTensor;

/* ------------------------------------------------------------------------------------------------
 * QKV projection with fused epilogues (ref_rms.py:47-56, 102-103, 217-220, 72-73):
 *   q = rowscale * (x @ wq),  k = rowscale * (x @ wk),  v = rowscale * (x @ wv)
 *   optional per-head RMS norm of q and k over head_dim (QKNorm), then
 *   q -> q_out, k/v -> rows [P, P+M) of the caches (the reference's cache append).
 * x: [B*M, N] row-major.  w*: [N, heads*D] row-major, used as x @ w (not transposed, ref_rms.py:47).
 * row_scale: fp32 [B*M] or NULL (PreNorm's rsqrt(mean x^2 + eps), applied in the epilogue).
 * With at most 32 rows (B*M) the weights are treated as CONSTANTS of the stream: the kernel starts reading them while
 * the kernel launched just before it on the same stream may still be running (programmatic dependent launch), and waits
 * for that kernel only before it touches x, row_scale and the outputs.  A caller that produces wq / wk / wv with the
 * launch immediately before this one must put any other launch (or a synchronisation) in between, or set
 * TRINITY_NO_PDL=1.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* wq;
  const void* wk;
  const void* wv;
  const float* row_scale;
  int B, M, P, N, Hq, Hkv, D;
  int dtype;
  int qk_norm;         /* 1: per-head RMS norm on q and k                 */
  float qk_eps;
  const void* gamma_q; /* [D] or NULL */
  const void* gamma_k; /* [D] or NULL */
  TrnHeadTensor q;     /* (b, s in [0,M), h in [0,Hq), d)                 */
  TrnHeadTensor k_cache; /* (b, s in [0,P+M), h in [0,Hkv), d); rows [P,P+M) written */
  TrnHeadTensor v_cache;
} TrnProjArgs;
int trinity_qkv_project(const TrnProjArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * LoRA linear layer, the neighbouring operator of the reference's lora_benchmark.py (tensor table :41-64;
 * arithmetic as its generator spells it, TritonGen.py:3092-3094):
 *   d = x @ a            [M, R]   (kept as a 16-bit tensor between the two steps, like the reference's D)
 *   o = x @ w + d @ b    [M, P]   (both products accumulated in fp32 in one accumulator)
 * x [M, N], w [N, P], a [N, R], b [R, P], all row-major and contiguous; N % 8 == 0, P % 64 == 0, R % 64 == 0.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* w;
  const void* a;
  const void* b;
  void* o;
  void* d;      /* [M, R] scratch / output of the first step */
  int M, N, P, R;
  int dtype;
} TrnLoraArgs;
int trinity_lora(const TrnLoraArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Gated MLP, the neighbouring operator of the reference's gmlp_benchmark.py (tensor table :53-74: X[M,K],
 * W1, W2 [K,N], temporaries C1, C1_exp, C2 [M,N], O[M,N]; the IR's sigmoid / exp nodes, TritonGen.py:2207, 3069-3071):
 *   c1 = x @ w1,  c2 = x @ w2   (fp32 accumulation)
 *   o  = gate(c1) * c2          gate = TRN_GATE_SILU: c1 * sigmoid(c1);  TRN_GATE_SIGMOID: sigmoid(c1)
 * One kernel: both products of an output tile meet in tensor memory and o is rounded once; c1, c2 are never
 * stored.  x [M, K], w1 / w2 [K, N], o [M, N] row-major and contiguous; K % 8 == 0, N % 64 == 0 (with at most 16
 * rows and K % 128 == 0, N % 32 == 0 suffices).
 * ---------------------------------------------------------------------------------------------- */
enum { TRN_GATE_SILU = 0, TRN_GATE_SIGMOID = 1 };
typedef struct {
  const void* x;
  const void* w1;
  const void* w2;
  void* o;
  int M, K, N;
  int dtype;
  int gate;
} TrnGmlpArgs;
int trinity_gmlp(const TrnGmlpArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Attention core (ref_rms.py:72-81): for every (b, query head h) with kv head h / (Hq/Hkv)
 *   s = scale * q k^T over keys [0, P+M);  causal: query i sees keys j <= P + i
 *   o = softmax(s) v;  lse (optional) = log-sum-exp of s in base 2:  log2(sum_j 2^(s_ij*log2 e))
 * When noise_mode != NONE the kernel computes NO output; it writes lse of the perturbed scores
 *   (s + g) / tau  instead (KeyFormer, ref_rms.py:172-174) — used by trinity_attn_colstats.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  TrnHeadTensor q;       /* s in [0,M)   */
  TrnHeadTensor k_cache; /* s in [0,P+M) */
  TrnHeadTensor v_cache;
  TrnHeadTensor o;       /* s in [0,M); ignored when noise_mode != NONE */
  float* lse;            /* fp32 [B, Hq, M] or NULL */
  int B, M, P, Hq, Hkv, D;
  int dtype;
  int causal;
  float scale;
  int noise_mode;
  float tau;
  const void* noise;     /* TRN_NOISE_TENSOR: element (b,h,i,j) at noise + b*nb + h*nh + i*ni + j */
  int64_t noise_stride_b, noise_stride_h, noise_stride_i;
  uint64_t seed;
  int single_p;          /* 0 (default): p is carried as hi + lo 16-bit parts into the P v product (~16 mantissa
                            bits of p); 1: one 16-bit part only (faster; 8 mantissa bits for bf16, 11 for fp16) */
  void* workspace;       /* optional device scratch, 256-byte aligned (NULL: none).  With it, a launch that
                            would fill less than half of the SMs divides each tile's key range among several
                            CTAs (split-KV) and merges their partial results with a second small kernel; the
                            result is the same softmax.  Contents need not be initialised.  Launches with at most
                            16 queries per head that produce an output split the key range inside thread-block
                            clusters instead and do not use it.                                              */
  size_t workspace_bytes; /* a smaller area than trinity_attention_workspace() asks for means fewer splits */
  float* lse_pert;       /* with noise_mode != NONE: when given, ONE pass computes the attention output o, lse of
                            the plain scores (if `lse` is given) and, here, lse of the perturbed scores
                            [B, Hq, M]; when NULL the call is the perturbed-lse-only pass described above    */
  float* scores;         /* optional fp32 [B, Hq, M, score_pitch]: every score the pass sees, in the base-2 log
                            domain (perturbed scores when noise_mode != NONE, else scale * s * log2 e; keys
                            a causal row must not see are -inf).  Lets small problems compute the per-key
                            statistics from memory instead of a second q k^T pass (the schedule of the
                            reference's programs that keep C_exp / C_exp_perturb in memory)               */
  int64_t score_pitch;   /* elements per (b, h, query) row of `scores`: a multiple of 32, >= P + M */
  int noise_heads;       /* TRN_NOISE_GUMBEL: the generated field is indexed by (b * noise_heads + h + noise_bh0, i, j).
                            0 means Hq.  A caller that runs a SLICE of a larger problem (a rank's batch items / heads)
                            passes the whole problem's head count and the flat index of its first (batch, head), and
                            gets exactly the noise the unsliced problem would see                              */
  int noise_bh0;
} TrnAttnArgs;
int trinity_attention(const TrnAttnArgs* a, void* cuda_stream);
/* Scratch that makes split-KV possible for this shape (0: the launch would not split).  No reference
 * counterpart: the generated Triton kernels never split the key loop (TritonGen.py:3071 walks it whole). */
size_t trinity_attention_workspace(const TrnAttnArgs* a);

/* ------------------------------------------------------------------------------------------------
 * Per-key statistics over queries (RoCo ref_rms.py:274-275, KeyFormer's C_out,
 * keyformer_llama_benchmark.py:74-79):  with p_ij = 2^(t_ij - lse_i), t = log2(e) * scores
 * (perturbed scores when noise_mode != NONE), for every (b, h, key j):
 *   sum_p[b,h,j] = sum_i p_ij        sum_p2[b,h,j] = sum_i p_ij^2   (sum_p2 optional)
 * Fixed summation order: results are bitwise reproducible run to run.
 * Outputs are fp32 when stats_fp32 != 0, else `dtype`.  Layout [B, Hq, P+M] contiguous.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  TrnHeadTensor q;
  TrnHeadTensor k_cache;
  const float* lse; /* fp32 [B, Hq, M], from trinity_attention */
  void* sum_p;
  void* sum_p2;     /* or NULL */
  int B, M, P, Hq, Hkv, D;
  int dtype;
  int stats_fp32;
  int causal;
  float scale;
  int noise_mode;
  float tau;
  const void* noise;
  int64_t noise_stride_b, noise_stride_h, noise_stride_i;
  uint64_t seed;
  const float* scores;   /* optional: the scores trinity_attention kept (TrnAttnArgs.scores, same pitch).  With them
                            the statistics are summed from memory: q, k_cache, scale, tau and the noise fields are
                            not used (noise is already in the scores; `causal` and P still say which scores
                            exist), `lse` must be the
                            log-sum-exp that belongs to those scores                                        */
  int64_t score_pitch;
  int noise_heads;       /* as in TrnAttnArgs */
  int noise_bh0;
} TrnColStatsArgs;
int trinity_attn_colstats(const TrnColStatsArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Top-k key selection per (b, h) row of an fp32 score matrix [rows, n] (n <= 8192):
 * indices of the k largest scores, sorted by descending score; equal scores keep the LOWER index
 * first.  idx_out int32 [rows, k].  No counterpart kernel exists in the reference (its harness only
 * reports scores); the rule matches torch.sort(descending=True, stable=True)[:k] on the oracle.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  const float* scores;
  int32_t* idx_out;
  int64_t rows;
  int n, k;
  int64_t score_row_stride;
} TrnTopkArgs;
int trinity_topk(const TrnTopkArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * fp32 <-> 16-bit conversion of n contiguous elements (n a multiple of 8): to_fp32 = 0 rounds fp32 `src`
 * to `dtype16` in `dst`, to_fp32 = 1 widens.  For fp32 callers (the fp32 Vanilla configuration; the
 * reference's own tensors are fp16, convert_eval_rms.py:24): the kernels compute on 16-bit operands with
 * fp32 accumulation.
 * ---------------------------------------------------------------------------------------------- */
int trinity_convert(const void* src, void* dst, int64_t n, int dtype16, int to_fp32, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Whole block, the unit the reference's generated forward() computes (TritonGen.py:590-708):
 *   [PreNorm row statistics] -> QKV projection (+QKNorm, +cache append) -> attention ->
 *   [KeyFormer / RoCo per-key statistics].
 * `workspace` (256-byte aligned base) holds, required: fp32 row scales [B*M], lse [B,Hq,M] and perturbed lse
 * [B,Hq,M]; optional, used when the caller lent them: the split-KV partials of the attention launch (shapes that
 * would fill less than half of the SMs) and, for KeyFormer / RoCo problems whose [B,Hq,M,P+M] fp32 scores fit in
 * 32 MiB, those scores (the statistics are then summed from memory instead of a second q k^T pass).
 * trinity_attn_block_workspace() returns required + optional; any size from the required part upwards is accepted.
 * skip_projection != 0: q / k_cache / v_cache are taken as given (callers that hold projected Q / K / V already,
 * as the KeyFormer and RoCo long-context configurations do).
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  int variant;
  int dtype;
  int B, M, P, N, Hq, Hkv, D;
  int skip_projection;
  const void* x;
  const void* wq;
  const void* wk;
  const void* wv;
  /* PreNorm */
  float pre_eps;
  const void* pre_gamma; /* [N] or NULL; when given, x_norm scratch [B*M, N] must be supplied */
  void* x_norm;          /* [B*M, N]: required with pre_gamma.  Given without gamma it selects the two-step
                            schedule too: X_norm is written here (rounded to the io type) and projected,
                            instead of the row scale being folded into the projection's epilogue      */
  /* QKNorm */
  float qk_eps;
  const void* gamma_q;
  const void* gamma_k;
  /* tensors */
  TrnHeadTensor q;
  TrnHeadTensor k_cache;
  TrnHeadTensor v_cache;
  TrnHeadTensor o;
  int causal;
  float scale;
  /* KeyFormer / RoCo */
  int noise_mode;
  float tau;
  const void* noise;
  int64_t noise_stride_b, noise_stride_h, noise_stride_i;
  uint64_t seed;
  void* sum_p;  /* KeyFormer C_out, RoCo C_out1: [B,Hq,P+M] */
  void* sum_p2; /* RoCo C_out2 or NULL */
  int stats_fp32;
  int single_p; /* see TrnAttnArgs */
  void* workspace;
  size_t workspace_bytes;
  int keep_scores; /* KeyFormer / RoCo: where the per-key statistics come from.  0: the library decides by size
                      (scores kept when [B,Hq,M,P+M] fp32 fit in 32 MiB); 1: keep the scores in the workspace and sum
                      the statistics from memory whenever they fit in 1 GiB — the schedule of the reference's
                      candidates that hold C_exp / C_exp_perturb in memory (TritonGen.py:1007-1042); -1: never keep
                      them, recompute q k^T in a second pass (candidates whose scores live in registers only).
                      trinity_attn_block_workspace() sizes the workspace for the same choice.  With at most 16
                      queries per head (M) and unpacked heads the statistics are summed inside the attention launch
                      in every setting — the scores never leave the chip — with bitwise the sums of setting 1. */
  int noise_heads; /* as in TrnAttnArgs: slices of a larger KeyFormer problem see the whole problem's noise */
  int noise_bh0;
} TrnBlockArgs;
size_t trinity_attn_block_workspace(const TrnBlockArgs* a);
int trinity_attn_block(const TrnBlockArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * Same block with HOST activations: copies x_host -> device staging, runs trinity_attn_block on
 * `cuda_stream`, copies o back to o_host (and the statistics when the pointers are given) and
 * synchronises the stream.  x_dev_staging / o (device) are caller buffers as above.  Weights and
 * caches stay device-resident (they are the model's state, not a per-call input).
 * With B >= 2, batch-major contiguous x / o and at least 4 MB to move, the call works through the batch in
 * up to 8 groups: group c+1 is copied in and group c-1 copied out (two internal copy streams, created on
 * the first such call on a device) while group c computes on `cuda_stream`; the outputs are bit-identical
 * to the one-pass call.  Pinned host buffers are needed for the copies to overlap.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
  TrnBlockArgs dev;        /* dev.x must point at the device staging buffer for x */
  const void* x_host;      /* [B*M, N] */
  void* o_host;            /* same layout and size as dev.o: o_bytes bytes copied */
  size_t x_bytes, o_bytes;
  void* sum_p_host;        /* optional */
  void* sum_p2_host;       /* optional */
  size_t stats_bytes;
} TrnBlockHostArgs;
int trinity_attn_block_host(const TrnBlockHostArgs* a, void* cuda_stream);

/* ------------------------------------------------------------------------------------------------
 * trinity_attn_block for callers that cannot provide (or allocate) a workspace.  It has no counterpart in
 * the reference, whose harness allocates every tensor itself with torch.
 *
 * Who needs it: code that is handed only the operator's input and output buffers by its host runtime (a
 * plugin inside an inference engine, a binding from a language with no device allocator at hand), or a
 * serving loop that bans device allocation once it is warm because cudaMalloc synchronises the whole
 * device.  For them the scratch of the block (row scales, log-sum-exp arrays) comes out of a fixed array
 * inside the library: trinity_static_scratch_capacity() bytes (8 MiB), held by every GPU that loads the
 * library until the process exits.
 *
 * Same arguments as trinity_attn_block; `workspace` / `workspace_bytes` are ignored.  x_norm (PreNorm with gamma)
 * is still the caller's.  The call performs no cudaMalloc / cudaFree and calls no allocating routine.  It runs
 * trinity_attn_block with the array as a workspace of exactly trinity_static_scratch_capacity() bytes, so its
 * results are bit-identical to that call.  Against a call whose caller lent the full
 * trinity_attn_block_workspace() they are identical when everything fits; when the optional areas (split-KV
 * partials, kept scores) fit only in part, fewer splits / the two-pass statistics are used and the results agree
 * within the rounding of a different summation order.  Limits and rules:
 *   - only the REQUIRED part of the workspace (fp32 row scales and the two log-sum-exp arrays: B*M*(1+2*Hq)
 *     values, ~2 M of them fit, e.g. the PreNorm Llama configuration B=8, M=2048, Hq=32) must fit; a problem whose
 *     required part exceeds the capacity (RoCo Falcon at B=2, M=8192, Hq=71) is refused with
 *     TRN_E_STATIC_SCRATCH and nothing is launched;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current): make that first call before any stream capture;
 *   - all calls on a device share the one array, which keeps what the previous call left there.  Nothing in
 *     it needs to be zero at entry (every value is written before it is read), but two calls that overlap
 *     on the GPU — different streams, or a graph replay racing a direct call — race on it: serialise them.
 * ---------------------------------------------------------------------------------------------- */
#define TRN_E_STATIC_SCRATCH (-10) /* problem needs more scratch than the built-in array holds */
size_t trinity_static_scratch_capacity(void);
int trinity_attn_block_static(const TrnBlockArgs* a, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* TRINITY_B200_H_ */
