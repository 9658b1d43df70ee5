// Per-key statistics over queries for KeyFormer and RoCo.
//   RoCo (ref_rms.py:274-275):       sum_i p_ij  and  sum_i p_ij^2  with p = softmax(scores) rows
//   KeyFormer (ref_rms.py:172-174 + the IR's C_out reduction, keyformer_llama_benchmark.py:74-79):
//                                     sum_i softmax((scores + noise) / tau)_ij
// A row's probabilities need that row's final log-sum-exp, so this is a second pass after the
// attention kernel: it recomputes the scores on the tensor cores, TRANSPOSED (keys along the TMEM
// lanes, queries along the columns), so that each thread owns one key and adds its column of
// probabilities in registers, in a fixed order — no atomics, bitwise reproducible.
//
// One CTA owns TWO 128-key tiles and loops over the 128-query blocks that can see them:
//   * GQA / MQA: the same keys for two query heads of one kv group (k tile shared through L2, q differs);
//   * MHA: two consecutive key blocks of one head.
//   warp 0      TMA producer: both k tiles once, then both tiles' q blocks through a ring
//   warp 1      one lane issues tcgen05.mma  S^T_t = k_t q_t^T  into two TMEM buffers per tile
//   warps 2-17  four statistics warpgroups, two per tile; thread = key, and the two warpgroups of a tile
//               split every query block's columns in halves (64 queries each): 16 arithmetic warps per SM
//               instead of 8 keep the issue slots and the XU pipe busy while others wait on a result.
//               p = 2^(t - lse_query), accumulate sum p and sum p^2 (packed fp32x2 arithmetic); the second
//               half's sums are added to the first's through shared memory at the end (fixed order)
#include <math.h>

#include <type_traits>

#include "attn_common.cuh"

namespace trn {
namespace {

constexpr int BKEY = 128;
constexpr int BQRY = 128;
constexpr int kCsHalves = 2;           // statistics warpgroups per key tile
constexpr int kCsThreads = 64 + 2 * kCsHalves * 128;
constexpr int kCsTmemCols = 512;      // tile t, buffer u: columns [(2t+u)*128, +128)

struct CsParams {
  HeadMapInfo qi, ki;
  const float* lse;
  void* sum_p;
  void* sum_p2;
  int B, M, P, L, Hq, Hkv, group;
  int n_kblocks, n_qblocks;
  int pair_heads, units;
  int causal;
  int stats_fp32;
  float scale, scale_log2, pert_log2;
  NoiseSrc noise;
  int* status;
};

template <int D>
struct CsSmem {
  static constexpr int kStages = (D == 128) ? 2 : 4;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = 128 * 128;
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kKOff = 0;                                     // two k tiles
  static constexpr int kQOff = 2 * kTileBytes;                        // ring of (q tile 0, q tile 1)
  static constexpr int kLseOff = kQOff + kStages * 2 * kTileBytes;    // 16 warps x 2 buffers x 64 floats
  static constexpr int kHashOff = kLseOff + 16 * 2 * 64 * 4;          // same shape: per-query noise row hashes
  static constexpr int kPartOff = kHashOff + 16 * 2 * 64 * 4;         // second half's sums: 2 tiles x 128 keys x 2
  static constexpr int kBarOff = kPartOff + 2 * 128 * 2 * 4;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

struct CsTile {
  int h, kvh, k0, present;
};

template <typename T, int D, bool PERT>
__global__ void __launch_bounds__(kCsThreads, 1)
attn_colstats_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CsParams p) {
  using SM = CsSmem<D>;
  constexpr int KS = SM::kStages;
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + SM::kBarOff;
  // barriers: k_full, q_full[KS], q_empty[KS], s_full[2 tiles][2 buffers], s_free[2][2]
  const uint32_t k_full = bar_base;
  auto q_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto q_empty = [&](int s) { return bar_base + 8u * (1 + KS + s); };
  auto s_full = [&](int t, int u) { return bar_base + 8u * (1 + 2 * KS + 2 * t + u); };
  auto s_free = [&](int t, int u) { return bar_base + 8u * (5 + 2 * KS + 2 * t + u); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + SM::kBarOff + 8 * (9 + 2 * KS));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  float* lse_s = reinterpret_cast<float*>(smem_gen + SM::kLseOff);
  uint32_t* hash_s = reinterpret_cast<uint32_t*>(smem_gen + SM::kHashOff);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Ctl ctl{p.status, abort_flag};

  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    for (int s = 0; s < KS; ++s) {
      mbar_init(q_full(s), 1);
      mbar_init(q_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t)
      for (int u = 0; u < 2; ++u) {
        mbar_init(s_full(t, u), 1);
        mbar_init(s_free(t, u), 128 * kCsHalves);
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
  griddep_wait();          // the attention pass's log-sum-exp values are read from here on
  griddep_launch();

  // ---- which two tiles: early key blocks (seen by the most queries under a causal mask) first
  const int row_blk = static_cast<int>(blockIdx.x) / p.units;
  const int unit = static_cast<int>(blockIdx.x) % p.units;
  int b;
  CsTile tile[2];
  if (p.pair_heads) {
    const int pairs_per_group = (p.group + 1) >> 1;
    const int pi = unit % pairs_per_group;
    const int bk = unit / pairs_per_group;
    const int kvh = bk % p.Hkv;
    b = bk / p.Hkv;
    tile[0] = CsTile{kvh * p.group + 2 * pi, kvh, row_blk * BKEY, 1};
    tile[1] = CsTile{kvh * p.group + 2 * pi + 1, kvh, row_blk * BKEY, (2 * pi + 1 < p.group) ? 1 : 0};
  } else {
    b = unit / p.Hq;
    const int h = unit - b * p.Hq;
    const int kvh = h / p.group;
    tile[0] = CsTile{h, kvh, row_blk * 2 * BKEY, 1};
    tile[1] = CsTile{h, kvh, row_blk * 2 * BKEY + BKEY, (row_blk * 2 * BKEY + BKEY < p.L) ? 1 : 0};
  }
  // first query block that can see any key of tile 0 (tile 1 starts at or after it): query q sees key k
  // iff k <= P + q
  const int i_start = p.causal ? max(0, tile[0].k0 - p.P) / BQRY : 0;
  const int n_iter = p.n_qblocks - i_start;

  auto k_s = [&](int t) { return smem_base + SM::kKOff + t * SM::kTileBytes; };
  auto q_s = [&](int s, int t) { return smem_base + SM::kQOff + (s * 2 + t) * SM::kTileBytes; };

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      const int n_tiles = tile[0].present + tile[1].present;
      mbar_expect_tx(k_full, n_tiles * SM::kTileBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (tile[t].present) {
#pragma unroll
          for (int c = 0; c < SM::kChunks; ++c)
            tma_load_head_tile(k_s(t) + c * SM::kChunkBytes, &tm_k, k_full, p.ki, c * 64, tile[t].k0, tile[t].kvh, b);
        }
    }
    for (int it = 0; it < n_iter; ++it) {
      const int st = it % KS;
      const uint32_t ph = (it / KS) & 1;
      bool ok = mbar_wait(q_empty(st), ph ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        const int n_tiles = tile[0].present + tile[1].present;
        mbar_expect_tx(q_full(st), n_tiles * SM::kTileBytes);
#pragma unroll
        for (int t = 0; t < 2; ++t)
          if (tile[t].present) {
#pragma unroll
            for (int c = 0; c < SM::kChunks; ++c)
              tma_load_head_tile(q_s(st, t) + c * SM::kChunkBytes, &tm_q, q_full(st), p.qi, c * 64,
                                 (i_start + it) * BQRY, tile[t].h, b);
          }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc_f16(Io<T>::kFmt, 0, 0, BKEY, BQRY);
    bool ok = mbar_wait(k_full, 0, ctl, KST_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it % KS;
      const uint32_t ph = (it / KS) & 1;
      const int u = it & 1;
      ok = mbar_wait(q_full(st), ph, ctl, KST_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      for (int t = 0; t < 2 && ok; ++t) {
        if (!tile[t].present) continue;
        ok = mbar_wait(s_free(t, u), ((it >> 1) & 1) ^ 1u, ctl, KST_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t d_tmem = tmem_base + (2 * t + u) * BQRY;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * SM::kChunkBytes + (kk & 3) * 32;
            umma_ss(d_tmem, make_smem_desc(k_s(t) + off, 0, 1024), make_smem_desc(q_s(st, t) + off, 0, 1024), idesc,
                    kk != 0 ? 1u : 0u);
          }
          umma_commit(s_full(t, u));
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) umma_commit(q_empty(st));
      __syncwarp();
    }
  } else {
    const int t = ((warp - 2) >> 2) & 1;
    const int hf = (warp - 2) >> 3;              // which half of a query block's columns
    const int quad = warp & 3;
    const int row = quad * 32 + lane;            // key within the tile
    const int key = tile[t].k0 + row;
    const int h = tile[t].h;
    const bool present = tile[t].present != 0;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    float* my_lse = lse_s + ((warp - 2) * 2) * 64;
    uint32_t* my_hash = hash_s + ((warp - 2) * 2) * 64;
    float2* part = reinterpret_cast<float2*>(smem_gen + SM::kPartOff) + t * 128 + row;
    const uint32_t headkey = PERT ? noise_headkey(p.noise.seed, static_cast<uint32_t>(b * p.noise.Hq + h + p.noise.bh0)) : 0u;
    float2 acc1 = make_float2(0.f, 0.f), acc2 = make_float2(0.f, 0.f);
    bool ok = true;
    uint32_t r[32];
    const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
    for (int it = 0; it < n_iter && present; ++it) {
      const int u = it & 1;
      const int q0 = (i_start + it) * BQRY;
      // staged values are indexed by the block's column: this warp holds columns [64 hf, 64 hf + 64)
      float* nl = my_lse + u * 64 - hf * 64;
      const uint32_t* hrow = my_hash + u * 64 - hf * 64;
      {
        // each warp stages its own copy of its columns' per-query NEGATED log-sum-exp (no cross-warp
        // barrier); -inf for queries past M makes their p = 0
#pragma unroll
        for (int v = 2 * hf; v < 2 * hf + 2; ++v) {
          const int q = q0 + v * 32 + lane;
          float val = -INFINITY;
          if (q < p.M) val = -__ldg(p.lse + (static_cast<long long>(b) * p.Hq + h) * p.M + q);
          nl[v * 32 + lane] = val;
          if (PERT) my_hash[u * 64 - hf * 64 + v * 32 + lane] = noise_rowhash(headkey, static_cast<uint32_t>(q));
        }
        __syncwarp();
      }
      ok = mbar_wait(s_full(t, u), (it >> 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + (2 * t + u) * BQRY + lane_addr;
      // 32-query chunks that hold at least one query (M = 16 new tokens: one chunk instead of four)
      const int c_begin = 2 * hf;
      const int n_chunks = min(2 * hf + 2, (p.M - q0 + 31) / 32);          // one past this warp's last chunk
      // causal: this key is visible to query q0 + col iff col >= key - P - q0
      const int cmin = p.causal ? (key - p.P - q0) : 0;
      const bool masked = p.causal && (tile[t].k0 + BKEY - 1 - p.P > q0);
      if (PERT && p.noise.mode == TRN_NOISE_GUMBEL) {   // warp-uniform: rows past L just compute unused values
        // generated noise: the per-key part of the hash is a thread constant, the per-query part comes from
        // shared memory four at a time.  Queries past M have -lse = -inf and give p = 0; compiled twice so
        // that only the block on the causal diagonal carries the per-element compare
        const uint32_t jc = static_cast<uint32_t>(key) * 0x85ebca6bu;
        const float c_s = p.scale * p.pert_log2;
        const float c_g = -0.6931471805599453f * p.pert_log2;
        auto gumbel_block = [&](auto masked_tag) {
          constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll 1
          for (int c = c_begin; c < n_chunks; ++c) {
            tmem_ld32(s_tmem + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const uint4 h4 = *reinterpret_cast<const uint4*>(hrow + c * 32 + i);
              const float4 n4 = *reinterpret_cast<const float4*>(nl + c * 32 + i);
              const uint32_t hh[4] = {h4.x, h4.y, h4.z, h4.w};
              const float nn[4] = {n4.x, n4.y, n4.z, n4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint32_t x = hh[e] ^ jc;
                x ^= x >> 16; x *= 0x7feb352du;
                x ^= x >> 15;
                const float tt = fmaf(gumbel_log2e_from_bits(x), c_g, fmaf(__uint_as_float(r[i + e]), c_s, nn[e]));
                float pr = ex2_approx(tt);
                if (kMasked && c * 32 + i + e < cmin) pr = 0.f;
                if (e & 1) acc1.y += pr; else acc1.x += pr;
              }
            }
          }
        };
        if (masked) gumbel_block(std::true_type{});
        else gumbel_block(std::false_type{});
      } else if (PERT) {
        for (int c = c_begin; c < n_chunks; ++c) {
          tmem_ld32(s_tmem + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            float tt;
            if (PERT) {
              const int q = q0 + col;
              const float g = (q < p.M && key < p.L) ? noise_at<T>(p.noise, hrow[col], b, h, q, key) : 0.f;
              tt = (__uint_as_float(r[i]) * p.scale + g) * p.pert_log2;
            } else {
              tt = __uint_as_float(r[i]) * p.scale_log2;
            }
            float pr = ex2_approx(tt + nl[col]);
            if (masked && col < cmin) pr = 0.f;
            acc1.x += pr;
            acc2.x = fmaf(pr, pr, acc2.x);
          }
        }
      } else {
        auto plain_block = [&](auto masked_tag) {
          constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll 1
          for (int c = c_begin; c < n_chunks; ++c) {
            tmem_ld32(s_tmem + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 n4 = *reinterpret_cast<const float4*>(nl + c * 32 + i);
              const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), c2,
                                           make_float2(n4.x, n4.y));
              const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])), c2,
                                           make_float2(n4.z, n4.w));
              float2 p0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y));
              float2 p1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
              if constexpr (kMasked) {
                const int col = c * 32 + i;
                if (col < cmin) p0.x = 0.f;
                if (col + 1 < cmin) p0.y = 0.f;
                if (col + 2 < cmin) p1.x = 0.f;
                if (col + 3 < cmin) p1.y = 0.f;
              }
              acc1 = __fadd2_rn(acc1, p0);
              acc2 = __ffma2_rn(p0, p0, acc2);
              acc1 = __fadd2_rn(acc1, p1);
              acc2 = __ffma2_rn(p1, p1, acc2);
            }
          }
        };
        if (masked) plain_block(std::true_type{});
        else plain_block(std::false_type{});
      }
      tc_fence_before();
      mbar_arrive(s_free(t, u));
    }
    // the second half hands its sums to the first, which owns the key's output
    if (hf == 1) *part = make_float2(acc1.x + acc1.y, acc2.x + acc2.y);
    asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "n"(128 * kCsHalves) : "memory");
    if (hf == 0 && ok && present && key < p.L) {
      const float2 other = *part;
      const float a1 = (acc1.x + acc1.y) + other.x, a2 = (acc2.x + acc2.y) + other.y;
      const long long o = (static_cast<long long>(b) * p.Hq + h) * p.L + key;
      if (p.stats_fp32) {
        static_cast<float*>(p.sum_p)[o] = a1;
        if (p.sum_p2 != nullptr) static_cast<float*>(p.sum_p2)[o] = a2;
      } else {
        static_cast<T*>(p.sum_p)[o] = Io<T>::from_f(a1);
        if (p.sum_p2 != nullptr) static_cast<T*>(p.sum_p2)[o] = Io<T>::from_f(a2);
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

// Per-key statistics from scores kept in memory by the attention pass (small problems): thread = key,
//   sum_p[key] = sum_i 2^(t[i][key] - lse[i]),  sum_p2 likewise with squares, i over the M queries in order.
// No q, k, tensor cores or noise here: t already holds the (perturbed) scores in the log2 domain.
template <typename T>
__global__ void __launch_bounds__(256)
colstats_from_scores_kernel(const float* __restrict__ scores, long long pitch, const float* __restrict__ lse,
                            void* __restrict__ sum_p, void* __restrict__ sum_p2, int M, int L, int first_query_off,
                            int stats_fp32, const int* __restrict__ status) {
  griddep_wait();
  griddep_launch();
  if (*reinterpret_cast<const volatile int*>(status) != 0) return;
  const int key = blockIdx.x * blockDim.x + threadIdx.x;
  const long long bh = blockIdx.y;
  if (key >= L) return;
  const float* t = scores + bh * M * pitch + key;
  const float* l = lse + bh * M;
  float a1 = 0.f, a2 = 0.f;
  // causal: query i sees this key iff i >= key - P; the attention pass never wrote the scores of the others
  int i = max(0, key - first_query_off);
  for (; i + 4 <= M; i += 4) {           // four independent loads in flight
    const float t0 = __ldg(t + (i + 0) * pitch), t1 = __ldg(t + (i + 1) * pitch);
    const float t2 = __ldg(t + (i + 2) * pitch), t3 = __ldg(t + (i + 3) * pitch);
    const float p0 = ex2_approx(t0 - __ldg(l + i)), p1 = ex2_approx(t1 - __ldg(l + i + 1));
    const float p2 = ex2_approx(t2 - __ldg(l + i + 2)), p3 = ex2_approx(t3 - __ldg(l + i + 3));
    a1 += p0; a2 = fmaf(p0, p0, a2);
    a1 += p1; a2 = fmaf(p1, p1, a2);
    a1 += p2; a2 = fmaf(p2, p2, a2);
    a1 += p3; a2 = fmaf(p3, p3, a2);
  }
  for (; i < M; ++i) {
    const float pr = ex2_approx(__ldg(t + i * pitch) - __ldg(l + i));
    a1 += pr;
    a2 = fmaf(pr, pr, a2);
  }
  const long long o = bh * L + key;
  if (stats_fp32) {
    static_cast<float*>(sum_p)[o] = a1;
    if (sum_p2 != nullptr) static_cast<float*>(sum_p2)[o] = a2;
  } else {
    static_cast<T*>(sum_p)[o] = Io<T>::from_f(a1);
    if (sum_p2 != nullptr) static_cast<T*>(sum_p2)[o] = Io<T>::from_f(a2);
  }
}

template <typename T>
int launch_from_scores(const TrnColStatsArgs& a, cudaStream_t st, const DeviceState& ds) {
  const int L = a.P + a.M;
  const long long bh = static_cast<long long>(a.B) * a.Hq;
  if (bh > 65535) return TRN_E_SHAPE;
  dim3 grid(static_cast<unsigned>((L + 255) / 256), static_cast<unsigned>(bh));
  // non-causal: every query sees every key (offset = L makes key - offset negative for all keys)
  TRN_CUDA_TRY(launch_pdl(colstats_from_scores_kernel<T>, grid, dim3(256), 0, st, a.scores,
                          static_cast<long long>(a.score_pitch), a.lse, a.sum_p, a.sum_p2, a.M, L, a.causal ? a.P : L,
                          a.stats_fp32, static_cast<const int*>(ds.status)));
  return TRN_OK;
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
  p.B = a.B; p.M = a.M; p.P = a.P; p.L = L; p.Hq = a.Hq; p.Hkv = a.Hkv; p.group = a.Hq / a.Hkv;
  p.n_kblocks = (L + BKEY - 1) / BKEY;
  p.n_qblocks = (a.M + BQRY - 1) / BQRY;
  p.pair_heads = p.group >= 2 ? 1 : 0;
  long long rows_of_ctas;
  if (p.pair_heads) {
    p.units = a.B * a.Hkv * ((p.group + 1) / 2);
    rows_of_ctas = p.n_kblocks;
  } else {
    p.units = a.B * a.Hq;
    rows_of_ctas = (p.n_kblocks + 1) / 2;
  }
  p.causal = a.causal;
  p.stats_fp32 = a.stats_fp32;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.pert_log2 = 1.4426950408889634f / a.tau;
  p.noise.mode = a.noise_mode;
  p.noise.ptr = a.noise;
  p.noise.sb = a.noise_stride_b; p.noise.sh = a.noise_stride_h; p.noise.si = a.noise_stride_i;
  p.noise.seed = a.seed;
  p.noise.M = a.M; p.noise.L = L;
  p.noise.Hq = a.noise_heads > 0 ? a.noise_heads : a.Hq;
  p.noise.bh0 = a.noise_bh0;
  p.status = ds.status;
  auto kern = attn_colstats_kernel<T, D, PERT>;
  rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), SM::kTotal, ds.device);
  if (rc != TRN_OK) return rc;
  const long long grid = rows_of_ctas * p.units;
  if (grid > 0x7fffffffLL) return TRN_E_SHAPE;
  TRN_CUDA_TRY(launch_pdl(kern, dim3(static_cast<unsigned>(grid)), dim3(kCsThreads), SM::kTotal, st, tm_q, tm_k, p));
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
  if (a.scores != nullptr) {
    // scores kept by the attention pass: no second q k^T
    if (a.score_pitch < a.P + a.M) return TRN_E_SHAPE;
    if (a.dtype == TRN_BF16) return launch_from_scores<__nv_bfloat16>(a, st, ds);
    if (a.dtype == TRN_FP16) return launch_from_scores<__half>(a, st, ds);
    return TRN_E_DTYPE;
  }
  if (!ht_ok(a.q) || !ht_ok(a.k_cache)) return a.q.ptr == nullptr || a.k_cache.ptr == nullptr ? TRN_E_NULL : TRN_E_ALIGN;
  if (a.dtype == TRN_BF16) return launch_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
