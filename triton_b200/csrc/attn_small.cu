// Attention core for at most 16 queries per (batch, head) — decode, chunked prefill, the reference's own M = 16,
// P = 1024 shapes (ref_rms.py:72-81: o = softmax(scale * q k^T) v over the cached prefix plus the new keys).
//
// With 16 query rows a 128-row tensor-memory tile is 7/8 padding and the launch is a latency chain (tensor-memory
// allocation, descriptors, a second launch to merge split-KV partials).  Here a CTA of four warps owns one (batch, head)
// and 1 / n_splits of its keys; each warp walks its own quarter of that range in chunks of 32 keys through a private
// two-stage cp.async ring, with warp-level mma.m16n8k16 for s = q k^T (q fragments stay in registers) and o += p v (p is
// re-used from the score accumulators as the A operand, as hi + lo 16-bit parts), and an online softmax on the
// accumulator registers.  The four warps' partial (max, sum, o) meet in shared memory, the CTAs of a head — a thread-
// block cluster — meet in rank 0's shared memory (st.shared::cluster between two cluster barriers), always in the same
// order: one launch, no scratch, bitwise reproducible.
//
// MODE 2 (KeyFormer, ref_rms.py:172-174) carries a second online log-sum-exp, of the perturbed scores
// (s * scale + g) / tau, beside the attention; MODE 2 / 3 can write every score they see (perturbed / plain, base-2 log
// domain, -inf where a causal row must not look) for the per-key statistics kernel to sum from memory.
//
// Algorithmic work per launch: 4 * B * Hq * D * M * (visible keys) flop; bytes: q, o and every visible k / v row once.
#include <math.h>

#include "attn_common.cuh"
#include "small_mma.cuh"

namespace trn {
namespace {

// Four warps, 32-key chunks, two stages.  Eight warps with 16-key chunks (two or three stages), eight warps with 32-key
// chunks and four warps with 16-key chunks in a four-deep ring were A/B'd in one process and came out within the timer's
// resolution of this layout on every shape tried (Llama M16 / P1024 11.3-12.1 us warm, 18.5 us L2-flushed for all): the
// key loop is bound by the warp-level MMA rate of the SM (96 mma.m16n8k16 per 32-key chunk with the two-part p), not by
// how the chunks are dealt out.
constexpr int kAsWarps = 4;
constexpr int kAsThreads = 32 * kAsWarps;
constexpr int kAsKeys = 32;                   // keys per chunk: 16 or 32
constexpr int kAsStages = 2;
constexpr int kAsKeepChunks = 5;              // chunks of scores a warp can keep for the fused statistics
constexpr int kAsKeepPitch = kAsKeepChunks * kAsKeys + 8;   // +8 floats: rows g = 0..7 of a float2 store spread over the banks
constexpr int kAsNB = kAsKeys / 8;            // 8-key score blocks per chunk
constexpr int kAsTPR = kAsThreads / 16;       // threads per row in the merges
constexpr int kAsMaxSplits = 8;

template <int D>
struct AsSmem {
  static constexpr int kPitch = D * 2 + 16;                    // bytes per staged key row: conflict-free ldmatrix
  static constexpr int kPanel = kAsKeys * kPitch;              // one [32 x D] panel of k or v
  static constexpr int kWarpRing = kAsStages * 2 * kPanel;
  static constexpr int kRingBytes = kAsWarps * kWarpRing;
  // after the key loop the ring is dead: the warps' partials [warps][16][kRow] fp32, then rank 0's exchange area for
  // the cluster [8][16][kRow]
  static constexpr int kRow = D + 4;                           // o | max, sum | the perturbed scores' max, sum
  static constexpr int kPart = 0;
  static constexpr int kXchg = kPart + kAsWarps * 16 * kRow * 4;
  static constexpr int kEpilogue = kXchg + kAsMaxSplits * 16 * kRow * 4;
  static constexpr int kTotal = kRingBytes > kEpilogue ? kRingBytes : kEpilogue;
  // launches that also sum the per-key statistics keep every score of the CTA until the rows' log-sum-exp is known:
  // [warp][16 rows][kKeepPitch] fp32 behind everything else, then the 16 log-sum-exps rank 0 hands to every rank
  static constexpr int kKeep = (kTotal + 127) & ~127;
  static constexpr int kLseBcast = kKeep + kAsWarps * 16 * kAsKeepPitch * 4;
  static constexpr int kTotalStats = kLseBcast + 16 * 4;
};

struct AsParams {
  const void* q; const void* k; const void* v; void* o;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh;
  float* lse;
  int B, M, P, L, Hq, group;
  int pack;      // query heads of one kv head that share a CTA's 16 rows (pack * M <= 16): row r = (head r / M, query r % M)
  int causal;
  float scale_log2;
  int n_splits;
  // MODE 2 / 3
  float scale, pert_log2;      // perturbed score in the log2 domain: (s * scale + g) * pert_log2, pert_log2 = log2(e) / tau
  NoiseSrc noise;
  int noise_pair_ok;           // noise tensor: two neighbouring keys of a row can be fetched as one 32-bit load
  float* lse_pert;             // MODE 2: [B, Hq, M]
  float* scores;               // optional [B, Hq, M, score_pitch]
  long long score_pitch;
  // MODE 2 / 3, optional: per-key sums over the queries of p = 2^(t - lse) (and of p^2) in the same launch, t = the
  // perturbed (MODE 2) or plain (MODE 3) scores, [B, Hq, L] fp32 or T (the statistics of trinity_attn_colstats)
  void* sum_p;
  void* sum_p2;
  int stats_fp32;
};

// HILO: p enters p v as two 16-bit parts (hi + lo, the library's default accuracy); false: one part (single_p callers)
// MODE 0: attention; 2: attention + log-sum-exp of the perturbed scores (+ those scores kept); 3: attention + plain
// scores kept
template <typename T, int D, bool HILO, int MODE>
__global__ void __launch_bounds__(kAsThreads)
attn_small_kernel(const AsParams p) {
  constexpr bool kPert = (MODE == 2);
  using SM = AsSmem<D>;
  constexpr int KS = D / 16;           // k steps of q k^T
  constexpr int NB = D / 8;            // 8-column blocks of o
  extern __shared__ __align__(16) uint8_t as_smem[];
  const uint32_t smem_base = smem_u32(as_smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t rank = cluster_ctarank();
  const int unit = static_cast<int>(blockIdx.x) / p.n_splits, units_per_batch = p.Hq / p.pack;
  const int b = unit / units_per_batch, h0 = (unit - b * units_per_batch) * p.pack, kvh = h0 / p.group;
  const int n_rows = p.pack * p.M;
  griddep_wait();                      // q / k / v come from the projection launched before
  griddep_launch();

  // ---- q fragments: rows g and g + 8 of the (at most 16) queries, all of head_dim
  const T* qb = static_cast<const T*>(p.q) + b * p.q_sb;
  const bool row_lo = g < n_rows, row_hi = g + 8 < n_rows;
  const int hd_lo = row_lo ? g / p.M : 0, hd_hi = row_hi ? (g + 8) / p.M : 0;          // head within the pack
  const int i_lo = row_lo ? g - hd_lo * p.M : 0, i_hi = row_hi ? g + 8 - hd_hi * p.M : 0;   // query within the head
  const T* q_lo = qb + (h0 + hd_lo) * p.q_sh + static_cast<long long>(i_lo) * p.q_ss;
  const T* q_hi = qb + (h0 + hd_hi) * p.q_sh + static_cast<long long>(i_hi) * p.q_ss;
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const uint32_t* lo = reinterpret_cast<const uint32_t*>(q_lo + ks * 16);
    const uint32_t* hi = reinterpret_cast<const uint32_t*>(q_hi + ks * 16);
    qa[ks][0] = row_lo ? __ldg(lo + t) : 0u;
    qa[ks][1] = row_hi ? __ldg(hi + t) : 0u;
    qa[ks][2] = row_lo ? __ldg(lo + 4 + t) : 0u;
    qa[ks][3] = row_hi ? __ldg(hi + 4 + t) : 0u;
  }

  // ---- this warp's chunks of the key range (chunks of kAsKeys keys dealt out evenly to the kAsWarps * n_splits warps of the cluster)
  const int kv_end = p.causal ? min(p.L, p.P + p.M) : p.L;       // keys any of the queries can see
  const int total_chunks = (kv_end + kAsKeys - 1) / kAsKeys;
  const int n_warps = kAsWarps * p.n_splits, wi = static_cast<int>(rank) * kAsWarps + warp;
  const int chunk_lo = total_chunks * wi / n_warps, chunk_hi = total_chunks * (wi + 1) / n_warps;
  const int n_chunks = chunk_hi - chunk_lo;
  const T* kb = static_cast<const T*>(p.k) + b * p.k_sb + kvh * p.k_sh;
  const T* vb = static_cast<const T*>(p.v) + b * p.v_sb + kvh * p.v_sh;
  const uint32_t ring = smem_base + warp * SM::kWarpRing;
  auto k_stage = [&](int s) { return ring + s * 2 * SM::kPanel; };
  auto v_stage = [&](int s) { return k_stage(s) + SM::kPanel; };
  auto load_stage = [&](int chunk) {
    const int s = chunk % kAsStages;
    const int key0 = (chunk_lo + chunk) * kAsKeys;
    constexpr int kSeg = D / 8;                                  // 16-byte segments per key row
#pragma unroll
    for (int i = 0; i < kAsKeys * kSeg / 32; ++i) {
      const int c = i * 32 + lane, row = c / kSeg, seg = c % kSeg;
      const int key = min(key0 + row, p.L - 1);                  // rows past the last key repeat it (masked below)
      cp_async16(k_stage(s) + row * SM::kPitch + seg * 16, kb + static_cast<long long>(key) * p.k_ss + seg * 8);
      cp_async16(v_stage(s) + row * SM::kPitch + seg * 16, vb + static_cast<long long>(key) * p.v_ss + seg * 8);
    }
  };

  float oacc[NB][4];
#pragma unroll
  for (int i = 0; i < NB; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) oacc[i][j] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;     // rows g and g + 8
  const int lim_lo = p.causal ? min(p.P + i_lo, p.L - 1) : p.L - 1;     // last visible key of each row
  const int lim_hi = p.causal ? min(p.P + i_hi, p.L - 1) : p.L - 1;

  // MODE 2 / 3: the rows' noise and score addresses, state of the perturbed log-sum-exp
  float m2_lo = -INFINITY, m2_hi = -INFINITY, l2_lo = 0.f, l2_hi = 0.f;
  const int hq_lo = h0 + hd_lo, hq_hi = h0 + hd_hi;
  uint32_t rh_lo = 0u, rh_hi = 0u;
  const T* nz_lo = nullptr;
  const T* nz_hi = nullptr;
  float* sc_lo = nullptr;
  float* sc_hi = nullptr;
  if constexpr (kPert) {
    rh_lo = noise_rowhash(noise_headkey(p.noise.seed, static_cast<uint32_t>(b * p.noise.Hq + hq_lo + p.noise.bh0)), static_cast<uint32_t>(i_lo));
    rh_hi = noise_rowhash(noise_headkey(p.noise.seed, static_cast<uint32_t>(b * p.noise.Hq + hq_hi + p.noise.bh0)), static_cast<uint32_t>(i_hi));
    if (p.noise.mode == TRN_NOISE_TENSOR) {
      nz_lo = static_cast<const T*>(p.noise.ptr) + b * p.noise.sb + hq_lo * p.noise.sh + i_lo * p.noise.si;
      nz_hi = static_cast<const T*>(p.noise.ptr) + b * p.noise.sb + hq_hi * p.noise.sh + i_hi * p.noise.si;
    }
  }
  const bool fuse_stats = MODE != 0 && p.sum_p != nullptr;
  float* keep = reinterpret_cast<float*>(as_smem + SM::kKeep) + warp * 16 * kAsKeepPitch;
  if constexpr (MODE != 0) {
    if (p.scores != nullptr) {
      if (row_lo) sc_lo = p.scores + ((static_cast<long long>(b) * p.Hq + hq_lo) * p.M + i_lo) * p.score_pitch;
      if (row_hi) sc_hi = p.scores + ((static_cast<long long>(b) * p.Hq + hq_hi) * p.M + i_hi) * p.score_pitch;
    }
  }

#pragma unroll
  for (int c = 0; c < kAsStages - 1; ++c) {
    if (c < n_chunks) load_stage(c);
    cp_async_commit();
  }
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    if (chunk + kAsStages - 1 < n_chunks) load_stage(chunk + kAsStages - 1);
    cp_async_commit();
    const int s = chunk % kAsStages;
    const int key0 = (chunk_lo + chunk) * kAsKeys;
    // noise of this thread's 16 scores, requested before the wait for the chunk's k / v
    float gz[kAsNB][4];
    if constexpr (kPert) {
#pragma unroll
      for (int nb = 0; nb < kAsNB; ++nb) {
        const int key = key0 + nb * 8 + 2 * t;
        if (p.noise.mode == TRN_NOISE_TENSOR && p.noise_pair_ok && key + 1 < p.L) {
          const float2 a = Io<T>::unpack2(__ldg(reinterpret_cast<const uint32_t*>(nz_lo + key)));
          const float2 c = Io<T>::unpack2(__ldg(reinterpret_cast<const uint32_t*>(nz_hi + key)));
          gz[nb][0] = a.x; gz[nb][1] = a.y; gz[nb][2] = c.x; gz[nb][3] = c.y;
        } else {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kk = min(key + e, p.L - 1);
            gz[nb][e] = noise_at<T>(p.noise, rh_lo, b, hq_lo, i_lo, kk);
            gz[nb][2 + e] = noise_at<T>(p.noise, rh_hi, b, hq_hi, i_hi, kk);
          }
        }
      }
    }
    cp_async_wait<kAsStages - 1>();
    __syncwarp();
    // ---- s = q k^T for 32 keys: four 8-key blocks
    float sacc[kAsNB][4];
#pragma unroll
    for (int i = 0; i < kAsNB; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sacc[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < kAsNB / 2; ++n2) {
        // matrices: (keys n2*16 .. +7, d ks*16 .. +7), (same keys, d + 8), (keys + 8, d), (keys + 8, d + 8)
        const int key = n2 * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
        const int dd = ks * 16 + ((lane >> 3) & 1) * 8;
        uint32_t b0, b1, b2, b3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                     : "r"(k_stage(s) + key * SM::kPitch + dd * 2));
        mma16816<T>(sacc[2 * n2], qa[ks], b0, b1);
        mma16816<T>(sacc[2 * n2 + 1], qa[ks], b2, b3);
      }
    }
    if constexpr (kPert) {
      // ---- perturbed scores: online log-sum-exp, optional write-out
      float tl[kAsNB][2], th[kAsNB][2];
      float c_lo = -INFINITY, c_hi = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < kAsNB; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + nb * 8 + 2 * t + e;
          tl[nb][e] = (key <= lim_lo) ? (sacc[nb][e] * p.scale + gz[nb][e]) * p.pert_log2 : -INFINITY;
          th[nb][e] = (key <= lim_hi) ? (sacc[nb][2 + e] * p.scale + gz[nb][2 + e]) * p.pert_log2 : -INFINITY;
          c_lo = fmaxf(c_lo, tl[nb][e]);
          c_hi = fmaxf(c_hi, th[nb][e]);
        }
        if (sc_lo != nullptr) *reinterpret_cast<float2*>(sc_lo + key0 + nb * 8 + 2 * t) = make_float2(tl[nb][0], tl[nb][1]);
        if (sc_hi != nullptr) *reinterpret_cast<float2*>(sc_hi + key0 + nb * 8 + 2 * t) = make_float2(th[nb][0], th[nb][1]);
        if (fuse_stats) {
          *reinterpret_cast<float2*>(keep + g * kAsKeepPitch + chunk * kAsKeys + nb * 8 + 2 * t) = make_float2(tl[nb][0], tl[nb][1]);
          *reinterpret_cast<float2*>(keep + (g + 8) * kAsKeepPitch + chunk * kAsKeys + nb * 8 + 2 * t) = make_float2(th[nb][0], th[nb][1]);
        }
      }
      c_lo = fmaxf(c_lo, __shfl_xor_sync(0xffffffffu, c_lo, 1)); c_lo = fmaxf(c_lo, __shfl_xor_sync(0xffffffffu, c_lo, 2));
      c_hi = fmaxf(c_hi, __shfl_xor_sync(0xffffffffu, c_hi, 1)); c_hi = fmaxf(c_hi, __shfl_xor_sync(0xffffffffu, c_hi, 2));
      const float n_lo = fmaxf(m2_lo, c_lo), n_hi = fmaxf(m2_hi, c_hi);
      const float u_lo = (n_lo == -INFINITY) ? 0.f : n_lo, u_hi = (n_hi == -INFINITY) ? 0.f : n_hi;
      float a_lo = 0.f, a_hi = 0.f;
#pragma unroll
      for (int nb = 0; nb < kAsNB; ++nb) {
        a_lo += ex2_approx(tl[nb][0] - u_lo) + ex2_approx(tl[nb][1] - u_lo);
        a_hi += ex2_approx(th[nb][0] - u_hi) + ex2_approx(th[nb][1] - u_hi);
      }
      l2_lo = l2_lo * ex2_approx(m2_lo - u_lo) + a_lo;
      l2_hi = l2_hi * ex2_approx(m2_hi - u_hi) + a_hi;
      m2_lo = n_lo; m2_hi = n_hi;
    }
    // ---- online softmax on the accumulators (log2 domain); invisible keys -> -inf
    float mb_lo = -INFINITY, mb_hi = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < kAsNB; ++nb) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + nb * 8 + 2 * t + e;
        sacc[nb][e] = (key <= lim_lo) ? sacc[nb][e] * p.scale_log2 : -INFINITY;
        sacc[nb][2 + e] = (key <= lim_hi) ? sacc[nb][2 + e] * p.scale_log2 : -INFINITY;
        mb_lo = fmaxf(mb_lo, sacc[nb][e]);
        mb_hi = fmaxf(mb_hi, sacc[nb][2 + e]);
      }
      if constexpr (MODE == 3) {
        if (sc_lo != nullptr) *reinterpret_cast<float2*>(sc_lo + key0 + nb * 8 + 2 * t) = make_float2(sacc[nb][0], sacc[nb][1]);
        if (sc_hi != nullptr) *reinterpret_cast<float2*>(sc_hi + key0 + nb * 8 + 2 * t) = make_float2(sacc[nb][2], sacc[nb][3]);
        if (fuse_stats) {
          *reinterpret_cast<float2*>(keep + g * kAsKeepPitch + chunk * kAsKeys + nb * 8 + 2 * t) = make_float2(sacc[nb][0], sacc[nb][1]);
          *reinterpret_cast<float2*>(keep + (g + 8) * kAsKeepPitch + chunk * kAsKeys + nb * 8 + 2 * t) = make_float2(sacc[nb][2], sacc[nb][3]);
        }
      }
    }
    mb_lo = fmaxf(mb_lo, __shfl_xor_sync(0xffffffffu, mb_lo, 1)); mb_lo = fmaxf(mb_lo, __shfl_xor_sync(0xffffffffu, mb_lo, 2));
    mb_hi = fmaxf(mb_hi, __shfl_xor_sync(0xffffffffu, mb_hi, 1)); mb_hi = fmaxf(mb_hi, __shfl_xor_sync(0xffffffffu, mb_hi, 2));
    const float mn_lo = fmaxf(m_lo, mb_lo), mn_hi = fmaxf(m_hi, mb_hi);
    const float use_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, use_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    const float al_lo = ex2_approx(m_lo - use_lo), al_hi = ex2_approx(m_hi - use_hi);     // 0 while m = -inf
    m_lo = mn_lo; m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    uint32_t p_hi[kAsNB][2], p_lo[kAsNB][2];                 // per 8-key block: rows g / g + 8, as packed pairs (hi and lo parts)
#pragma unroll
    for (int nb = 0; nb < kAsNB; ++nb) {
      const float a0 = ex2_approx(sacc[nb][0] - use_lo), a1 = ex2_approx(sacc[nb][1] - use_lo);
      const float c0 = ex2_approx(sacc[nb][2] - use_hi), c1 = ex2_approx(sacc[nb][3] - use_hi);
      sum_lo += a0 + a1;
      sum_hi += c0 + c1;
      p_hi[nb][0] = Io<T>::pack2(a0, a1);
      p_hi[nb][1] = Io<T>::pack2(c0, c1);
      if constexpr (HILO) {
        const float2 ra = Io<T>::unpack2(p_hi[nb][0]), rc = Io<T>::unpack2(p_hi[nb][1]);
        p_lo[nb][0] = Io<T>::pack2(a0 - ra.x, a1 - ra.y);
        p_lo[nb][1] = Io<T>::pack2(c0 - rc.x, c1 - rc.y);
      }
    }
    l_lo = l_lo * al_lo + sum_lo;       // this thread's share of the row sums (its 8 of the chunk's 32 keys)
    l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < NB; ++i) {
      oacc[i][0] *= al_lo; oacc[i][1] *= al_lo;
      oacc[i][2] *= al_hi; oacc[i][3] *= al_hi;
    }
    // ---- o += p v: two k steps of 16 keys; p's accumulator layout is the A fragment's
#pragma unroll
    for (int kk = 0; kk < kAsKeys / 16; ++kk) {
      const uint32_t ah[4] = {p_hi[2 * kk][0], p_hi[2 * kk][1], p_hi[2 * kk + 1][0], p_hi[2 * kk + 1][1]};
      const uint32_t al[4] = {p_lo[2 * kk][0], p_lo[2 * kk][1], p_lo[2 * kk + 1][0], p_lo[2 * kk + 1][1]};
#pragma unroll
      for (int n2 = 0; n2 < NB / 2; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(v_stage(s) + (kk * 16 + (lane & 15)) * SM::kPitch + (n2 * 16 + (lane >> 4) * 8) * 2, b0, b1, b2, b3);
        mma16816<T>(oacc[2 * n2], ah, b0, b1);
        mma16816<T>(oacc[2 * n2 + 1], ah, b2, b3);
        if constexpr (HILO) {
          mma16816<T>(oacc[2 * n2], al, b0, b1);
          mma16816<T>(oacc[2 * n2 + 1], al, b2, b3);
        }
      }
    }
    __syncwarp();                      // every lane is done with stage s before it is refilled
  }
  cp_async_wait<0>();
  // row sums: the four lanes of a group hold different keys of the same rows
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if constexpr (kPert) {
    l2_lo += __shfl_xor_sync(0xffffffffu, l2_lo, 1); l2_lo += __shfl_xor_sync(0xffffffffu, l2_lo, 2);
    l2_hi += __shfl_xor_sync(0xffffffffu, l2_hi, 1); l2_hi += __shfl_xor_sync(0xffffffffu, l2_hi, 2);
  }
  __syncthreads();                     // every warp is done with its ring: the partials take its place

  // ---- the four warps' partials -> shared memory [warp][row][D | max | sum]
  float* part = reinterpret_cast<float*>(as_smem + SM::kPart);
#pragma unroll
  for (int n = 0; n < NB; ++n) {
    *reinterpret_cast<float2*>(part + (warp * 16 + g) * SM::kRow + n * 8 + 2 * t) = make_float2(oacc[n][0], oacc[n][1]);
    *reinterpret_cast<float2*>(part + (warp * 16 + g + 8) * SM::kRow + n * 8 + 2 * t) = make_float2(oacc[n][2], oacc[n][3]);
  }
  if (t == 0) {
    *reinterpret_cast<float2*>(part + (warp * 16 + g) * SM::kRow + D) = make_float2(m_lo, l_lo);
    *reinterpret_cast<float2*>(part + (warp * 16 + g + 8) * SM::kRow + D) = make_float2(m_hi, l_hi);
    if constexpr (kPert) {
      *reinterpret_cast<float2*>(part + (warp * 16 + g) * SM::kRow + D + 2) = make_float2(m2_lo, l2_lo);
      *reinterpret_cast<float2*>(part + (warp * 16 + g + 8) * SM::kRow + D + 2) = make_float2(m2_hi, l2_hi);
    }
  }
  __syncthreads();
  // thread = (row, D / 8 columns): merge `n` partials laid out [n][16][kRow] in fixed order -> (o, max, sum) of the row
  constexpr int CW = D / kAsTPR;
  const int row = threadIdx.x / kAsTPR, c0 = (threadIdx.x % kAsTPR) * CW;
  float acc[CW], mx, tot, mx2 = -INFINITY, tot2 = 0.f;
  auto merge = [&](const float* src, int n) {
    if constexpr (kPert) {
      mx2 = -INFINITY;
      for (int i = 0; i < n; ++i) mx2 = fmaxf(mx2, src[(i * 16 + row) * SM::kRow + D + 2]);
      tot2 = 0.f;
      for (int i = 0; i < n; ++i) {
        const float mi = src[(i * 16 + row) * SM::kRow + D + 2];
        if (mi != -INFINITY) tot2 = fmaf(ex2_approx(mi - mx2), src[(i * 16 + row) * SM::kRow + D + 3], tot2);
      }
    }
    mx = -INFINITY;
    for (int i = 0; i < n; ++i) mx = fmaxf(mx, src[(i * 16 + row) * SM::kRow + D]);
    tot = 0.f;
#pragma unroll
    for (int c = 0; c < CW; ++c) acc[c] = 0.f;
    for (int i = 0; i < n; ++i) {
      const float mi = src[(i * 16 + row) * SM::kRow + D];
      if (mi == -INFINITY) continue;                 // this part saw no visible key of the row
      const float w = ex2_approx(mi - mx);
      tot = fmaf(w, src[(i * 16 + row) * SM::kRow + D + 1], tot);
#pragma unroll
      for (int c = 0; c < CW; ++c) acc[c] = fmaf(w, src[(i * 16 + row) * SM::kRow + c0 + c], acc[c]);
    }
  };
  merge(part, kAsWarps);
  if (p.n_splits > 1) {
    cluster_sync_all_relaxed();        // every CTA of the cluster is past its ring: rank 0's exchange area may be written
    const uint32_t slot = map_to_rank(smem_base + SM::kXchg, 0) + rank * (16 * SM::kRow * 4);
#pragma unroll
    for (int c = 0; c < CW; c += 2) st_cluster_f2(slot + (row * SM::kRow + c0 + c) * 4, acc[c], acc[c + 1]);
    if ((threadIdx.x % kAsTPR) == 0) {
      st_cluster_f2(slot + (row * SM::kRow + D) * 4, mx, tot);
      if constexpr (kPert) st_cluster_f2(slot + (row * SM::kRow + D + 2) * 4, mx2, tot2);
    }
    cluster_sync_all();                // the parts of every rank have landed in rank 0
    if (rank != 0 && !fuse_stats) return;
    if (rank == 0) merge(reinterpret_cast<const float*>(as_smem + SM::kXchg), p.n_splits);
  }
  if (rank == 0 && fuse_stats && (threadIdx.x % kAsTPR) == 0) {
    // the log-sum-exp the statistics are taken against (perturbed scores' in MODE 2), to every rank of the cluster
    const float l = kPert ? mx2 + log2f(tot2) : mx + log2f(tot);
    for (int r = 0; r < p.n_splits; ++r)
      st_cluster_u32((p.n_splits > 1 ? map_to_rank(smem_base + SM::kLseBcast, r) : smem_base + SM::kLseBcast) + row * 4,
                     __float_as_uint(l));
  }
  if (rank == 0 && row < n_rows) {
    const int hd = row / p.M, i = row - hd * p.M, h = h0 + hd;
    const float inv = tot > 0.f ? 1.0f / tot : 0.f;
    T* dst = static_cast<T*>(p.o) + b * p.o_sb + static_cast<long long>(i) * p.o_ss + h * p.o_sh + c0;
    if constexpr (CW % 8 == 0) {
#pragma unroll
      for (int c = 0; c < CW; c += 8) {
        uint4 v;
        v.x = Io<T>::pack2(acc[c] * inv, acc[c + 1] * inv); v.y = Io<T>::pack2(acc[c + 2] * inv, acc[c + 3] * inv);
        v.z = Io<T>::pack2(acc[c + 4] * inv, acc[c + 5] * inv); v.w = Io<T>::pack2(acc[c + 6] * inv, acc[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = v;
      }
    } else {
#pragma unroll
      for (int c = 0; c < CW; c += 4) {
        uint2 v;
        v.x = Io<T>::pack2(acc[c] * inv, acc[c + 1] * inv); v.y = Io<T>::pack2(acc[c + 2] * inv, acc[c + 3] * inv);
        *reinterpret_cast<uint2*>(dst + c) = v;
      }
    }
    if (p.lse != nullptr && (threadIdx.x % kAsTPR) == 0)
      p.lse[(static_cast<long long>(b) * p.Hq + h) * p.M + i] = mx + log2f(tot);
    if constexpr (kPert) {
      if ((threadIdx.x % kAsTPR) == 0) p.lse_pert[(static_cast<long long>(b) * p.Hq + h) * p.M + i] = mx2 + log2f(tot2);
    }
  }
  if constexpr (MODE != 0) {
    if (fuse_stats) {
      // ---- per-key statistics of this warp's keys (the launcher fuses only unpacked heads: row = query, h0 = head):
      // thread = key, queries in ascending order, the arithmetic of colstats_from_scores_kernel on the same numbers
      if (p.n_splits > 1) cluster_sync_all(); else __syncthreads();
      const float* lse_row = reinterpret_cast<const float*>(as_smem + SM::kLseBcast);
      const long long out0 = (static_cast<long long>(b) * p.Hq + h0) * p.L;
      const int first_query_off = p.causal ? p.P : p.L;
      for (int kk = lane; kk < n_chunks * kAsKeys; kk += 32) {
        const int key = chunk_lo * kAsKeys + kk;
        if (key >= p.L) break;
        float a1 = 0.f, a2 = 0.f;
        for (int i = max(0, key - first_query_off); i < p.M; ++i) {
          const float pr = ex2_approx(keep[i * kAsKeepPitch + kk] - lse_row[i]);
          a1 += pr;
          a2 = fmaf(pr, pr, a2);
        }
        if (p.stats_fp32) {
          static_cast<float*>(p.sum_p)[out0 + key] = a1;
          if (p.sum_p2 != nullptr) static_cast<float*>(p.sum_p2)[out0 + key] = a2;
        } else {
          static_cast<T*>(p.sum_p)[out0 + key] = Io<T>::from_f(a1);
          if (p.sum_p2 != nullptr) static_cast<T*>(p.sum_p2)[out0 + key] = Io<T>::from_f(a2);
        }
      }
    }
  }
}

// grouped-query heads of one kv head share the CTA's 16 rows while they fit (decode: M = 1 packs 16 heads)
int pack_of(const TrnAttnArgs& a) {
  const int group = a.Hq / a.Hkv;
  for (int c = group; c >= 1; --c)
    if (group % c == 0 && c * a.M <= 16) return c;
  return 1;
}
// CTAs per unit (= cluster size): fill the SMs once, keep every warp at least two chunks of keys
int splits_of(const TrnAttnArgs& a, int pack, int sm_count) {
  const long long units = static_cast<long long>(a.B) * (a.Hq / pack);
  const int chunks = (a.P + a.M + kAsKeys - 1) / kAsKeys;
  int ns = kAsMaxSplits;
  while (ns > 1 && (units * ns > sm_count || chunks < 2 * kAsWarps * ns)) ns >>= 1;
  return ns;
}

template <typename T, int D, bool HILO, int MODE>
int launch_inst(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds, const AttnFusedStats* fs = nullptr) {
  using SM = AsSmem<D>;
  auto kern = attn_small_kernel<T, D, HILO, MODE>;
  const int smem = (fs != nullptr && MODE != 0) ? SM::kTotalStats : SM::kTotal;
  const int rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), SM::kTotalStats, ds.device);
  if (rc != TRN_OK) return rc;
  AsParams p{};
  if (fs != nullptr && MODE != 0) {
    p.sum_p = fs->sum_p;
    p.sum_p2 = fs->sum_p2;
    p.stats_fp32 = fs->stats_fp32;
  }
  p.q = a.q.ptr; p.k = a.k_cache.ptr; p.v = a.v_cache.ptr; p.o = a.o.ptr;
  p.q_sb = a.q.stride_b; p.q_ss = a.q.stride_s; p.q_sh = a.q.stride_h;
  p.k_sb = a.k_cache.stride_b; p.k_ss = a.k_cache.stride_s; p.k_sh = a.k_cache.stride_h;
  p.v_sb = a.v_cache.stride_b; p.v_ss = a.v_cache.stride_s; p.v_sh = a.v_cache.stride_h;
  p.o_sb = a.o.stride_b; p.o_ss = a.o.stride_s; p.o_sh = a.o.stride_h;
  p.lse = a.lse;
  p.B = a.B; p.M = a.M; p.P = a.P; p.L = a.P + a.M; p.Hq = a.Hq; p.group = a.Hq / a.Hkv;
  p.causal = a.causal;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.scale = a.scale;
  p.pert_log2 = 1.4426950408889634f / a.tau;
  p.noise.mode = a.noise_mode;
  p.noise.ptr = a.noise;
  p.noise.sb = a.noise_stride_b; p.noise.sh = a.noise_stride_h; p.noise.si = a.noise_stride_i;
  p.noise.seed = a.seed;
  p.noise.M = a.M; p.noise.L = p.L;
  p.noise.Hq = a.noise_heads > 0 ? a.noise_heads : a.Hq;
  p.noise.bh0 = a.noise_bh0;
  p.noise_pair_ok = (a.noise != nullptr && (reinterpret_cast<uintptr_t>(a.noise) & 3u) == 0 && (a.noise_stride_b & 1) == 0 &&
                     (a.noise_stride_h & 1) == 0 && (a.noise_stride_i & 1) == 0) ? 1 : 0;
  p.lse_pert = a.lse_pert;
  p.scores = a.scores;
  p.score_pitch = a.score_pitch;
  p.pack = pack_of(a);
  const long long heads = static_cast<long long>(a.B) * (a.Hq / p.pack);
  const int ns = splits_of(a, p.pack, ds.sm_count);
  p.n_splits = ns;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(heads * ns), 1, 1);
  cfg.blockDim = dim3(kAsThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(ns);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  TRN_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, p));
  return TRN_OK;
}

template <typename T, int D>
int launch_mode(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds, const AttnFusedStats* fs) {
  if (a.noise_mode != TRN_NOISE_NONE) return launch_inst<T, D, true, 2>(a, st, ds, fs);
  if (a.scores != nullptr || fs != nullptr) return launch_inst<T, D, true, 3>(a, st, ds, fs);
  return a.single_p == 0 ? launch_inst<T, D, true, 0>(a, st, ds) : launch_inst<T, D, false, 0>(a, st, ds);
}

}  // namespace

// at most 16 queries per head: plain attention (scores kept or not), or attention fused with the perturbed scores'
// log-sum-exp; the perturbed-lse-only pass (no output) stays with the tensor-memory kernel
bool attn_small_applies(const TrnAttnArgs& a) {
  if (a.noise_mode != TRN_NOISE_NONE && a.lse_pert == nullptr) return false;
  return a.M <= 16 && (a.D == 64 || a.D == 128) && static_cast<long long>(a.B) * a.Hq <= 0x3fffffffLL;
}

// the statistics can ride along when a row is a query of ONE head (no packed heads) and every warp's share of the keys
// fits its score area
bool attn_small_stats_applies(const TrnAttnArgs& a, int sm_count) {
  if (!attn_small_applies(a)) return false;
  const int pack = pack_of(a);
  if (pack != 1) return false;
  const int ns = splits_of(a, pack, sm_count);
  const int chunks = (a.P + a.M + kAsKeys - 1) / kAsKeys, warps = kAsWarps * ns;
  return (chunks + warps - 1) / warps <= kAsKeepChunks;
}

int launch_attn_small(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds, const AttnFusedStats* fs) {
  if (a.dtype == TRN_BF16)
    return a.D == 128 ? launch_mode<__nv_bfloat16, 128>(a, st, ds, fs) : launch_mode<__nv_bfloat16, 64>(a, st, ds, fs);
  if (a.dtype == TRN_FP16) return a.D == 128 ? launch_mode<__half, 128>(a, st, ds, fs) : launch_mode<__half, 64>(a, st, ds, fs);
  return TRN_E_DTYPE;
}

}  // namespace trn
