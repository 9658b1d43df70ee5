// Attention core of the block (ref_rms.py:72-81): o = softmax(scale * q k^T) v per (batch, head), keys
// [0, P+M) = cached prefix + new tokens, optional causal mask (query i sees keys <= P + i), GQA/MQA by
// mapping query head h to kv head h / (Hq/Hkv).  Online softmax in fp32 (the reference's IR has no
// max-subtraction, TritonGen.py:3071; the result is the same softmax, computed stably).
//
// One CTA = 128 queries of one head, streaming 128-key blocks:
//   warp 0     TMA producer: q tile once, then k / v tiles into a ring (4-D descriptors, zero fill
//              past the last key)
//   warp 1     one lane issues tcgen05.mma: S = q k^T (fp32 in TMEM, two S buffers so the next
//              block's q k^T overlaps this block's softmax) and O += P v (fp32 in TMEM)
//   warps 2-5  one thread per query row: tcgen05.ld S, running max / sum, 2^x, P packed to 16-bit
//              into swizzled shared memory as the A operand of P v; O is rescaled in TMEM only when
//              a row's max grew by more than 2^8 since the last rescale.  By default p is split into
//              two 16-bit parts (hi + lo) and P v is issued for both, so the product carries ~16
//              mantissa bits of p instead of 8 (bf16) / 11 (fp16).
// MODE 1 (KeyFormer's second row pass, ref_rms.py:172-174) computes only the log-sum-exp of the
// perturbed scores (s + g) / tau and skips P, v and O.
//
// Algorithmic flops per launch (MODE 0): 4 * B * Hq * D * (number of visible (query, key) pairs).
#include <math.h>

#include "attn_common.cuh"

namespace trn {
namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kAttnThreads = 192;
constexpr int kTmemColsAttn = 512;    // S0 [0,128) S1 [128,256) O [256, 256+D)
constexpr float kRescaleThreshold = 8.0f;   // log2 units

struct AttnParams {
  HeadMapInfo qi, ki, vi;
  void* o;
  long long o_sb, o_ss, o_sh;
  float* lse;
  int B, M, P, L, Hq, group;
  int n_qblocks;
  int causal;
  float scale;         // MODE 1
  float scale_log2;    // MODE 0: scale * log2(e)
  float pert_log2;     // MODE 1: log2(e) / tau
  NoiseSrc noise;
  int* status;
};

template <int D, bool SPLIT>
struct AttnSmem {
  static constexpr int kStages = (D == 128) ? 2 : 4;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = 128 * 128;            // 128 rows x 64 elements
  static constexpr int kQBytes = kChunks * kChunkBytes;
  static constexpr int kKBytes = kQBytes;
  static constexpr int kVBytes = kQBytes;
  static constexpr int kPBytes = (SPLIT ? 4 : 2) * kChunkBytes;   // 128 rows x 128 keys (x2: hi and lo parts)
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = kQBytes;
  static constexpr int kPOff = kKVOff + kStages * (kKBytes + kVBytes);
  static constexpr int kBarOff = kPOff + kPBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

template <typename T, int D, int MODE, bool SPLIT>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
  using SM = AttnSmem<D, SPLIT>;
  constexpr int KS = SM::kStages;
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + SM::kBarOff;
  // barriers: q_full, k_full[KS], v_full[KS], kv_empty[KS], s_full[2], s_free[2], p_full, pv_done
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (1 + KS + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + 2 * KS + s); };
  auto s_full = [&](int b) { return bar_base + 8u * (1 + 3 * KS + b); };
  auto s_free = [&](int b) { return bar_base + 8u * (3 + 3 * KS + b); };
  const uint32_t p_full = bar_base + 8u * (5 + 3 * KS);
  const uint32_t pv_done = bar_base + 8u * (6 + 3 * KS);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + SM::kBarOff + 8 * (7 + 3 * KS));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Ctl ctl{p.status, abort_flag};

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(s_free(b), 128);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemColsAttn);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // ---- which tile: heavy (late) query blocks first so the causal tail is short
  const int nbh = p.B * p.Hq;
  const int qb = p.n_qblocks - 1 - static_cast<int>(blockIdx.x) / nbh;
  const int bh = static_cast<int>(blockIdx.x) % nbh;
  const int b = bh / p.Hq;
  const int h = bh - b * p.Hq;
  const int kvh = h / p.group;
  const int q0 = qb * BQ;
  const int q_hi = min(q0 + BQ, p.M);
  const int kv_end = p.causal ? min(p.L, p.P + q_hi) : p.L;
  const int n_blocks = (kv_end + BKV - 1) / BKV;

  const uint32_t q_s = smem_base + SM::kQOff;
  auto k_s = [&](int s) { return smem_base + SM::kKVOff + s * (SM::kKBytes + SM::kVBytes); };
  auto v_s = [&](int s) { return k_s(s) + SM::kKBytes; };
  const uint32_t p_s = smem_base + SM::kPOff;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      if (MODE == 0) tma_prefetch_desc(&tm_v);
      mbar_expect_tx(q_full, SM::kQBytes);
#pragma unroll
      for (int c = 0; c < SM::kChunks; ++c)
        tma_load_head_tile(q_s + c * SM::kChunkBytes, &tm_q, q_full, p.qi, c * 64, q0, h, b);
    }
    for (int j = 0; j < n_blocks; ++j) {
      const int st = j % KS;
      const uint32_t ph = (j / KS) & 1;
      bool ok = mbar_wait(kv_empty(st), ph ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(k_full(st), SM::kKBytes);
#pragma unroll
        for (int c = 0; c < SM::kChunks; ++c)
          tma_load_head_tile(k_s(st) + c * SM::kChunkBytes, &tm_k, k_full(st), p.ki, c * 64, j * BKV, kvh, b);
        if (MODE == 0) {
          mbar_expect_tx(v_full(st), SM::kVBytes);
#pragma unroll
          for (int c = 0; c < SM::kChunks; ++c)
            tma_load_head_tile(v_s(st) + c * SM::kChunkBytes, &tm_v, v_full(st), p.vi, c * 64, j * BKV, kvh, b);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    constexpr uint32_t idesc_qk = make_idesc_f16(Io<T>::kFmt, 0, 0, BQ, BKV);   // q, k both K-major
    constexpr uint32_t idesc_pv = make_idesc_f16(Io<T>::kFmt, 0, 1, BQ, D);     // P K-major, v MN-major
    bool ok = mbar_wait(q_full, 0, ctl, KST_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    // S[j & 1] = q k_j^T
    auto issue_qk = [&](int j) -> bool {
      const int st = j % KS;
      const uint32_t ph = (j / KS) & 1;
      bool w = mbar_wait(k_full(st), ph, ctl, KST_TIMEOUT_MMA);
      w = w && mbar_wait(s_free(j & 1), ((j >> 1) & 1) ^ 1u, ctl, KST_TIMEOUT_MMA);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t d_tmem = tmem_base + (j & 1) * BKV;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SM::kChunkBytes + (kk & 3) * 32;
          umma_ss(d_tmem, make_smem_desc(q_s + off, 0, 1024), make_smem_desc(k_s(st) + off, 0, 1024), idesc_qk,
                  kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full(j & 1));
        if (MODE == 1) umma_commit(kv_empty(st));
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_blocks && ok; ++j) {
      if (j + 1 < n_blocks) {
        ok = issue_qk(j + 1);
        if (!ok) break;
      }
      if (MODE == 0) {
        const int st = j % KS;
        const uint32_t ph = (j / KS) & 1;
        bool w = mbar_wait(v_full(st), ph, ctl, KST_TIMEOUT_MMA);
        w = w && mbar_wait(p_full, j & 1, ctl, KST_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t o_tmem = tmem_base + 2 * BKV;
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {
            const uint64_t adesc = make_smem_desc(p_s + (kk >> 2) * SM::kChunkBytes + (kk & 3) * 32, 0, 1024);
            const uint64_t bdesc = make_smem_desc(v_s(st) + kk * 2048, SM::kChunkBytes, 1024);
            umma_ss(o_tmem, adesc, bdesc, idesc_pv, (j | kk) != 0 ? 1u : 0u);
          }
          if (SPLIT) {
            // low-order part of P (p - hi), same v tile: O += P_lo v
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
              const uint64_t adesc =
                  make_smem_desc(p_s + (2 + (kk >> 2)) * SM::kChunkBytes + (kk & 3) * 32, 0, 1024);
              const uint64_t bdesc = make_smem_desc(v_s(st) + kk * 2048, SM::kChunkBytes, 1024);
              umma_ss(o_tmem, adesc, bdesc, idesc_pv, 1u);
            }
          }
          umma_commit(kv_empty(st));
          umma_commit(pv_done);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------- softmax / epilogue (warps 2..5) -------------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int q_abs = q0 + row;
    const bool row_valid = q_abs < p.M;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int limit = p.causal ? min(p.P + q_abs, p.L - 1) : p.L - 1;       // last visible key of this row
    const int limit_min = p.causal ? min(p.P + q0, p.L - 1) : p.L - 1;      // ... of the tile's first row
    uint8_t* p_gen = smem_gen + SM::kPOff;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint32_t r[32];

    for (int j = 0; j < n_blocks; ++j) {
      const int sb = j & 1;
      const int kv0 = j * BKV;
      ok = mbar_wait(s_full(sb), (j >> 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + sb * BKV + lane_addr;
      const bool masked = (kv0 + BKV - 1) > limit_min;

      if (MODE == 1) {
        // one pass, chunk-wise online log-sum-exp of the perturbed scores
        for (int c = 0; c < BKV / 32; ++c) {
          tmem_ld32(s_tmem + c * 32, r);
          tmem_wait_ld();
          float t[32];
          float cm = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = kv0 + c * 32 + i;
            float v = -INFINITY;
            if (col <= limit) {
              const float g = row_valid ? noise_at<T>(p.noise, b, h, q_abs, col) : 0.f;
              v = (__uint_as_float(r[i]) * p.scale + g) * p.pert_log2;
            }
            t[i] = v;
            cm = fmaxf(cm, v);
          }
          const float m_new = fmaxf(m_run, cm);
          if (m_new != -INFINITY) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) acc += ex2_approx(t[i] - m_new);
            l_run = l_run * ex2_approx(m_run - m_new) + acc;
            m_run = m_new;
          }
        }
        tc_fence_before();
        mbar_arrive(s_free(sb));
        continue;
      }

      // ---- pass 1: block maximum of this row
      float mb = -INFINITY;
      for (int c = 0; c < BKV / 32; ++c) {
        tmem_ld32(s_tmem + c * 32, r);
        tmem_wait_ld();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv0 + c * 32 + i <= limit) mb = fmaxf(mb, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mb = fmaxf(mb, __uint_as_float(r[i]));
        }
      }
      mb *= p.scale_log2;                         // scale > 0, so max commutes with it
      // m_run is the exponent offset in use: (row max seen at the last rescale) - kPBias.  fp16 has few
      // exponent bits, so its p values are biased up by 2^4 to keep the low-order part of p out of
      // the subnormal range; bf16 needs no bias.
      constexpr float kPBias = (Io<T>::kFmt == 0) ? 4.0f : 0.0f;
      const float m_target = mb - kPBias;
      const bool grow = (m_target - m_run) > kRescaleThreshold;   // first block: m_run = -inf -> true
      float alpha = 1.0f;
      if (grow) {
        alpha = ex2_approx(m_run - m_target);     // 0 on the first block
        m_run = m_target;
      }
      // ---- P v of the previous block must be done: it reads the P buffer and accumulates into O
      if (j > 0) {
        ok = mbar_wait(pv_done, (j - 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
          const uint32_t o_tmem = tmem_base + 2 * BKV + lane_addr;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld32(o_tmem + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(o_tmem + c * 32, r);
          }
          tmem_wait_st();
          l_run *= alpha;
        }
      }
      // ---- pass 2: p = 2^(s * c - m), row sum, P tile into swizzled shared memory
      float lsum = 0.f;
      for (int c = 0; c < BKV / 32; ++c) {
        tmem_ld32(s_tmem + c * 32, r);
        tmem_wait_ld();
        uint32_t packed[16];
        uint32_t packed_lo[SPLIT ? 16 : 1];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_run));
          float p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -m_run));
          if (masked) {
            if (kv0 + c * 32 + i > limit) p0 = 0.f;
            if (kv0 + c * 32 + i + 1 > limit) p1 = 0.f;
          }
          lsum += p0 + p1;
          const uint32_t hi = Io<T>::pack2(p0, p1);
          packed[i >> 1] = hi;
          if (SPLIT) {
            // p = hi + lo with both parts 16-bit: the P v product keeps ~16 mantissa bits of p
            const float2 hf = Io<T>::unpack2(hi);
            packed_lo[i >> 1] = Io<T>::pack2(p0 - hf.x, p1 - hf.y);
          }
        }
        uint8_t* chunk = p_gen + (c >> 1) * SM::kChunkBytes;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t unit = static_cast<uint32_t>((c & 1) * 4 + u);
          const uint32_t off = swz128(static_cast<uint32_t>(row), unit);
          *reinterpret_cast<uint4*>(chunk + off) =
              make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
          if (SPLIT)
            *reinterpret_cast<uint4*>(chunk + 2 * SM::kChunkBytes + off) =
                make_uint4(packed_lo[4 * u], packed_lo[4 * u + 1], packed_lo[4 * u + 2], packed_lo[4 * u + 3]);
        }
      }
      l_run += lsum;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(s_free(sb));
      mbar_arrive(p_full);
    }

    if (ok && MODE == 0) {
      ok = mbar_wait(pv_done, (n_blocks - 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        const uint32_t o_tmem = tmem_base + 2 * BKV + lane_addr;
        T* orow = static_cast<T*>(p.o) + static_cast<long long>(b) * p.o_sb + static_cast<long long>(q_abs) * p.o_ss +
                  static_cast<long long>(h) * p.o_sh;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld32(o_tmem + c * 32, r);
          tmem_wait_ld();
          if (row_valid) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = Io<T>::pack2(__uint_as_float(r[i]) * inv_l, __uint_as_float(r[i + 1]) * inv_l);
              v.y = Io<T>::pack2(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l);
              v.z = Io<T>::pack2(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l);
              v.w = Io<T>::pack2(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
            }
          }
        }
        tc_fence_before();
      }
    }
    if (ok && row_valid && p.lse != nullptr)
      p.lse[(static_cast<long long>(b) * p.Hq + h) * p.M + q_abs] = m_run + log2f(l_run);
  }

  // ------------------------------- teardown -------------------------------
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemColsAttn);
  }
}

template <typename T, int D, int MODE, bool SPLIT>
int launch_inst(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  using SM = AttnSmem<D, SPLIT>;
  AttnParams p{};
  const int L = a.P + a.M;
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = make_head_tmap(&tm_q, &p.qi, a.q, a.M, a.Hq, a.B, D, BQ);
  if (rc != TRN_OK) return rc;
  rc = make_head_tmap(&tm_k, &p.ki, a.k_cache, L, a.Hkv, a.B, D, BKV);
  if (rc != TRN_OK) return rc;
  if (MODE == 0) {
    rc = make_head_tmap(&tm_v, &p.vi, a.v_cache, L, a.Hkv, a.B, D, BKV);
    if (rc != TRN_OK) return rc;
  } else {
    tm_v = tm_k;
    p.vi = p.ki;
  }
  p.o = a.o.ptr;
  p.o_sb = a.o.stride_b; p.o_ss = a.o.stride_s; p.o_sh = a.o.stride_h;
  p.lse = a.lse;
  p.B = a.B; p.M = a.M; p.P = a.P; p.L = L; p.Hq = a.Hq; p.group = a.Hq / a.Hkv;
  p.n_qblocks = (a.M + BQ - 1) / BQ;
  p.causal = a.causal;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.pert_log2 = 1.4426950408889634f / a.tau;
  p.noise.mode = a.noise_mode;
  p.noise.ptr = a.noise;
  p.noise.sb = a.noise_stride_b; p.noise.sh = a.noise_stride_h; p.noise.si = a.noise_stride_i;
  p.noise.seed = a.seed;
  p.noise.M = a.M; p.noise.L = L; p.noise.Hq = a.Hq;
  p.status = ds.status;
  auto kern = attn_fwd_kernel<T, D, MODE, SPLIT>;
  rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), SM::kTotal, ds.device);
  if (rc != TRN_OK) return rc;
  const long long grid = static_cast<long long>(p.n_qblocks) * a.B * a.Hq;
  if (grid > 0x7fffffffLL) return TRN_E_SHAPE;
  kern<<<static_cast<int>(grid), kAttnThreads, SM::kTotal, st>>>(tm_q, tm_k, tm_v, p);
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}

template <typename T>
int launch_typed(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  const bool pert = a.noise_mode != TRN_NOISE_NONE;
  if (a.D == 128) {
    if (pert) return launch_inst<T, 128, 1, false>(a, st, ds);
    return a.single_p ? launch_inst<T, 128, 0, false>(a, st, ds) : launch_inst<T, 128, 0, true>(a, st, ds);
  }
  if (a.D == 64) {
    if (pert) return launch_inst<T, 64, 1, false>(a, st, ds);
    return a.single_p ? launch_inst<T, 64, 0, false>(a, st, ds) : launch_inst<T, 64, 0, true>(a, st, ds);
  }
  return TRN_E_SHAPE;
}

bool ht_ok(const TrnHeadTensor& t) {
  return t.ptr != nullptr && aligned16(t.ptr) && (t.stride_b & 7) == 0 && (t.stride_s & 7) == 0 &&
         (t.stride_h & 7) == 0;
}

}  // namespace

int launch_attention(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.B <= 0 || a.M <= 0 || a.P < 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv != 0) return TRN_E_SHAPE;
  if (a.D != 64 && a.D != 128) return TRN_E_SHAPE;
  if (!(a.scale > 0.f)) return TRN_E_SHAPE;
  const bool pert = a.noise_mode != TRN_NOISE_NONE;
  if (a.noise_mode < TRN_NOISE_NONE || a.noise_mode > TRN_NOISE_GUMBEL) return TRN_E_VARIANT;
  if (a.q.ptr == nullptr || a.k_cache.ptr == nullptr) return TRN_E_NULL;
  if (!ht_ok(a.q) || !ht_ok(a.k_cache)) return TRN_E_ALIGN;
  if (!pert) {
    if (a.v_cache.ptr == nullptr || a.o.ptr == nullptr) return TRN_E_NULL;
    if (!ht_ok(a.v_cache) || !ht_ok(a.o)) return TRN_E_ALIGN;
  } else {
    if (a.lse == nullptr) return TRN_E_NULL;
    if (!(a.tau > 0.f)) return TRN_E_SHAPE;
    if (a.noise_mode == TRN_NOISE_TENSOR && a.noise == nullptr) return TRN_E_NULL;
  }
  if (a.dtype == TRN_BF16) return launch_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
