// Per-key statistics over queries for KeyFormer and RoCo.
//   RoCo (ref_rms.py:274-275):       sum_i p_ij  and  sum_i p_ij^2  with p = softmax(scores) rows
//   KeyFormer (ref_rms.py:172-174 + the IR's C_out reduction, keyformer_llama_benchmark.py:74-79):
//                                     sum_i softmax((scores + noise) / tau)_ij
// A row's probabilities need that row's final log-sum-exp, so this is a second pass after the
// attention kernel: it recomputes the scores on the tensor cores, TRANSPOSED (keys along the TMEM
// lanes, queries along the columns), so that each thread owns one key and adds its column of
// probabilities in registers, in a fixed order — no atomics, bitwise reproducible.
//
// One CTA = 128 keys of one (batch, query head), looping over the 128-query blocks that can see them:
//   warp 0     TMA producer: k tile once, q tiles through a 4-stage ring
//   warp 1     one lane issues tcgen05.mma  S^T = k q^T  into two TMEM buffers
//   warps 2-5  thread = key: p = 2^(t - lse_query), accumulate sum p and sum p^2
#include <math.h>

#include "attn_common.cuh"

namespace trn {
namespace {

constexpr int BKEY = 128;
constexpr int BQRY = 128;
constexpr int kCsThreads = 192;
constexpr int kCsStages = 4;
constexpr int kCsTmemCols = 256;

struct CsParams {
  HeadMapInfo qi, ki;
  const float* lse;
  void* sum_p;
  void* sum_p2;
  int B, M, P, L, Hq, group;
  int n_kblocks, n_qblocks;
  int causal;
  int stats_fp32;
  float scale, scale_log2, pert_log2;
  NoiseSrc noise;
  int* status;
};

template <int D>
struct CsSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = 128 * 128;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kKOff = 0;
  static constexpr int kQOff = kTileBytes;
  static constexpr int kLseOff = kQOff + kCsStages * kTileBytes;    // 4 warps x 2 buffers x 128 floats
  static constexpr int kBarOff = kLseOff + 4 * 2 * 128 * 4;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

template <typename T, int D, bool PERT>
__global__ void __launch_bounds__(kCsThreads, 1)
attn_colstats_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CsParams p) {
  using SM = CsSmem<D>;
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + SM::kBarOff;
  const uint32_t k_full = bar_base;
  auto q_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bar_base + 8u * (1 + kCsStages + s); };
  auto s_full = [&](int b) { return bar_base + 8u * (1 + 2 * kCsStages + b); };
  auto s_free = [&](int b) { return bar_base + 8u * (3 + 2 * kCsStages + b); };
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_gen + SM::kBarOff + 8 * (5 + 2 * kCsStages));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  float* lse_s = reinterpret_cast<float*>(smem_gen + SM::kLseOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Ctl ctl{p.status, abort_flag};

  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    for (int s = 0; s < kCsStages; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(s_free(b), 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kCsTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // ---- which tile: early key blocks (seen by the most queries under a causal mask) first
  const int nbh = p.B * p.Hq;
  const int kb = static_cast<int>(blockIdx.x) / nbh;
  const int bh = static_cast<int>(blockIdx.x) % nbh;
  const int b = bh / p.Hq;
  const int h = bh - b * p.Hq;
  const int kvh = h / p.group;
  const int k0 = kb * BKEY;
  // first query block that can see any key of this tile: query q sees key k iff k <= P + q
  const int i_start = p.causal ? max(0, k0 - p.P) / BQRY : 0;
  const int n_iter = p.n_qblocks - i_start;

  const uint32_t k_s = smem_base + SM::kKOff;
  auto q_s = [&](int s) { return smem_base + SM::kQOff + s * SM::kTileBytes; };

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      mbar_expect_tx(k_full, SM::kTileBytes);
#pragma unroll
      for (int c = 0; c < SM::kChunks; ++c)
        tma_load_head_tile(k_s + c * SM::kChunkBytes, &tm_k, k_full, p.ki, c * 64, k0, kvh, b);
    }
    for (int it = 0; it < n_iter; ++it) {
      const int st = it % kCsStages;
      const uint32_t ph = (it / kCsStages) & 1;
      bool ok = mbar_wait(q_empty(st), ph ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(q_full(st), SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < SM::kChunks; ++c)
          tma_load_head_tile(q_s(st) + c * SM::kChunkBytes, &tm_q, q_full(st), p.qi, c * 64, (i_start + it) * BQRY,
                             h, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_f16(Io<T>::kFmt, 0, 0, BKEY, BQRY);
    bool ok = mbar_wait(k_full, 0, ctl, KST_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it % kCsStages;
      const uint32_t ph = (it / kCsStages) & 1;
      bool w = mbar_wait(q_full(st), ph, ctl, KST_TIMEOUT_MMA);
      w = w && mbar_wait(s_free(it & 1), ((it >> 1) & 1) ^ 1u, ctl, KST_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t d_tmem = tmem_base + (it & 1) * BQRY;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SM::kChunkBytes + (kk & 3) * 32;
          umma_ss(d_tmem, make_smem_desc(k_s + off, 0, 1024), make_smem_desc(q_s(st) + off, 0, 1024), idesc,
                  kk != 0 ? 1u : 0u);
        }
        umma_commit(q_empty(st));
        umma_commit(s_full(it & 1));
      }
      __syncwarp();
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;            // key within the tile
    const int key = k0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    float acc1 = 0.f, acc2 = 0.f;
    bool ok = true;
    uint32_t r[32];
    for (int it = 0; it < n_iter; ++it) {
      const int sb = it & 1;
      const int q0 = (i_start + it) * BQRY;
      {
        // each warp stages its own copy of this block's per-query log-sum-exp (no cross-warp barrier);
        // +inf for queries past M makes their p = 0
        float* dst = lse_s + (quad * 2 + sb) * 128;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int q = q0 + u * 32 + lane;
          float v = INFINITY;
          if (q < p.M) v = __ldg(p.lse + (static_cast<long long>(b) * p.Hq + h) * p.M + q);
          dst[u * 32 + lane] = v;
        }
        __syncwarp();
      }
      ok = mbar_wait(s_full(sb), (it >> 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + sb * BQRY + lane_addr;
      // causal: this key is visible to query q0 + col iff col >= key - P - q0
      const int cmin = p.causal ? (key - p.P - q0) : 0;
      const bool masked = p.causal && (k0 + BKEY - 1 - p.P > q0);
      const float* lrow = lse_s + (quad * 2 + sb) * 128;
      for (int c = 0; c < BQRY / 32; ++c) {
        tmem_ld32(s_tmem + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = c * 32 + i;
          float t;
          if (PERT) {
            const int q = q0 + col;
            const float g = (q < p.M && key < p.L) ? noise_at<T>(p.noise, b, h, q, key) : 0.f;
            t = (__uint_as_float(r[i]) * p.scale + g) * p.pert_log2;
          } else {
            t = __uint_as_float(r[i]) * p.scale_log2;
          }
          float pr = ex2_approx(t - lrow[col]);
          if (masked && col < cmin) pr = 0.f;
          acc1 += pr;
          acc2 = fmaf(pr, pr, acc2);
        }
      }
      tc_fence_before();
      mbar_arrive(s_free(sb));
    }
    if (ok && key < p.L) {
      const long long o = (static_cast<long long>(b) * p.Hq + h) * p.L + key;
      if (p.stats_fp32) {
        static_cast<float*>(p.sum_p)[o] = acc1;
        if (p.sum_p2 != nullptr) static_cast<float*>(p.sum_p2)[o] = acc2;
      } else {
        static_cast<T*>(p.sum_p)[o] = Io<T>::from_f(acc1);
        if (p.sum_p2 != nullptr) static_cast<T*>(p.sum_p2)[o] = Io<T>::from_f(acc2);
      }
    }
  }

  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kCsTmemCols);
  }
}

template <typename T, int D, bool PERT>
int launch_inst(const TrnColStatsArgs& a, cudaStream_t st, const DeviceState& ds) {
  using SM = CsSmem<D>;
  CsParams p{};
  const int L = a.P + a.M;
  CUtensorMap tm_q, tm_k;
  int rc = make_head_tmap(&tm_q, &p.qi, a.q, a.M, a.Hq, a.B, D, BQRY);
  if (rc != TRN_OK) return rc;
  rc = make_head_tmap(&tm_k, &p.ki, a.k_cache, L, a.Hkv, a.B, D, BKEY);
  if (rc != TRN_OK) return rc;
  p.lse = a.lse;
  p.sum_p = a.sum_p;
  p.sum_p2 = a.sum_p2;
  p.B = a.B; p.M = a.M; p.P = a.P; p.L = L; p.Hq = a.Hq; p.group = a.Hq / a.Hkv;
  p.n_kblocks = (L + BKEY - 1) / BKEY;
  p.n_qblocks = (a.M + BQRY - 1) / BQRY;
  p.causal = a.causal;
  p.stats_fp32 = a.stats_fp32;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.pert_log2 = 1.4426950408889634f / a.tau;
  p.noise.mode = a.noise_mode;
  p.noise.ptr = a.noise;
  p.noise.sb = a.noise_stride_b; p.noise.sh = a.noise_stride_h; p.noise.si = a.noise_stride_i;
  p.noise.seed = a.seed;
  p.noise.M = a.M; p.noise.L = L; p.noise.Hq = a.Hq;
  p.status = ds.status;
  auto kern = attn_colstats_kernel<T, D, PERT>;
  rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), SM::kTotal, ds.device);
  if (rc != TRN_OK) return rc;
  const long long grid = static_cast<long long>(p.n_kblocks) * a.B * a.Hq;
  if (grid > 0x7fffffffLL) return TRN_E_SHAPE;
  kern<<<static_cast<int>(grid), kCsThreads, SM::kTotal, st>>>(tm_q, tm_k, p);
  TRN_CUDA_TRY(cudaGetLastError());
  return TRN_OK;
}

template <typename T>
int launch_typed(const TrnColStatsArgs& a, cudaStream_t st, const DeviceState& ds) {
  const bool pert = a.noise_mode != TRN_NOISE_NONE;
  if (a.D == 128) return pert ? launch_inst<T, 128, true>(a, st, ds) : launch_inst<T, 128, false>(a, st, ds);
  if (a.D == 64) return pert ? launch_inst<T, 64, true>(a, st, ds) : launch_inst<T, 64, false>(a, st, ds);
  return TRN_E_SHAPE;
}

bool ht_ok(const TrnHeadTensor& t) {
  return t.ptr != nullptr && aligned16(t.ptr) && (t.stride_b & 7) == 0 && (t.stride_s & 7) == 0 &&
         (t.stride_h & 7) == 0;
}

}  // namespace

int launch_colstats(const TrnColStatsArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.B <= 0 || a.M <= 0 || a.P < 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv != 0) return TRN_E_SHAPE;
  if (a.D != 64 && a.D != 128) return TRN_E_SHAPE;
  if (!(a.scale > 0.f)) return TRN_E_SHAPE;
  if (a.noise_mode < TRN_NOISE_NONE || a.noise_mode > TRN_NOISE_GUMBEL) return TRN_E_VARIANT;
  if (a.noise_mode != TRN_NOISE_NONE && !(a.tau > 0.f)) return TRN_E_SHAPE;
  if (a.noise_mode == TRN_NOISE_TENSOR && a.noise == nullptr) return TRN_E_NULL;
  if (a.lse == nullptr || a.sum_p == nullptr) return TRN_E_NULL;
  if (!ht_ok(a.q) || !ht_ok(a.k_cache)) return a.q.ptr == nullptr || a.k_cache.ptr == nullptr ? TRN_E_NULL : TRN_E_ALIGN;
  if (a.dtype == TRN_BF16) return launch_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
