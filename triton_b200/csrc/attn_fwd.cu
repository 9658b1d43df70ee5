// Attention core of the block (ref_rms.py:72-81): o = softmax(scale * q k^T) v per (batch, head), keys
// [0, P+M) = cached prefix + new tokens, optional causal mask (query i sees keys <= P + i), GQA/MQA by
// mapping query head h to kv head h / (Hq/Hkv).  Online softmax in fp32 (the reference's IR has no
// max-subtraction, TritonGen.py:3071; the result is the same softmax, computed stably).
//
// One CTA works on TWO 128-query tiles that read the same k / v stream, so that each SM sub-partition
// hosts two softmax warps and the tensor pipe always has the other tile's MMAs to run:
//   * GQA / MQA (Hq/Hkv >= 2): the tiles are the same 128 queries of two query heads of one kv group
//     (identical causal structure: perfectly balanced);
//   * MHA: the tiles are two consecutive 128-query blocks of one head.
//   warp 0      TMA producer: both q tiles once, then k / v tiles into a ring (4-D descriptors, zero
//               fill past the last key)
//   warp 1      one lane issues tcgen05.mma: S_t = q_t k^T (fp32 in TMEM) and O_t += P_t v, where P_t is
//               read from TENSOR MEMORY as the A operand (it overwrites S_t in place, no shared-memory
//               round trip)
//   warps 2-5   softmax warpgroup of tile 0, warps 6-9 of tile 1: one thread per query row; tcgen05.ld S,
//               running max / sum, 2^x, p packed to 16 bits and written back over S with tcgen05.st.
//               By default p is split into two 16-bit parts (hi + lo) and P v is issued for both, so the
//               product carries ~16 mantissa bits of p.  O is rescaled in TMEM only when a row's max
//               grew by more than 2^8 since the last rescale.
// MODE 1 (KeyFormer's second row pass, ref_rms.py:172-174) computes only the log-sum-exp of the
// perturbed scores (s + g) / tau and skips P, v and O.  MODE 2 does both in one pass over the scores: the
// attention output and, from the same S tile while it is in registers, the perturbed log-sum-exp.
// Optionally every (perturbed) score is also written out in the log2 domain, so that for small problems the
// per-key statistics need no second q k^T pass.
//
// Algorithmic flops per launch (MODE 0): 4 * B * Hq * D * (number of visible (query, key) pairs).
#include <math.h>

#include <type_traits>

#include "attn_common.cuh"

namespace trn {
namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int kAttnThreads = 320;
constexpr int kTmemColsAttn = 512;    // S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D)
constexpr float kRescaleThreshold = 8.0f;   // log2 units


struct AttnParams {
  HeadMapInfo qi, ki, vi;
  void* o;
  long long o_sb, o_ss, o_sh;
  float* lse;
  float* lse_pert;     // MODE 2: log-sum-exp of the perturbed scores (MODE 1 writes it to `lse`)
  float* scores;       // optional [B, Hq, M, score_pitch] fp32: every score in the log2 domain (perturbed in MODE 1 / 2)
  int score_pitch;     // multiple of 32
  int B, M, P, L, Hq, Hkv, group;
  int n_qblocks;       // 128-row query blocks
  int pair_heads;      // 1: tiles = two heads of a kv group; 0: tiles = two consecutive query blocks
  int units;           // CTAs per query-block row (pairs, or batch*heads)
  int causal;
  float scale;         // MODE 1
  float scale_log2;    // MODE 0: scale * log2(e)
  float pert_log2;     // MODE 1: log2(e) / tau
  NoiseSrc noise;
  int noise_vec_ok;    // noise tensor base and strides allow 128-bit row loads
  // split-KV: the key blocks of a CTA's tiles are divided among n_splits CTAs, each of which writes a
  // normalised fp32 partial output and the base-2 log-sum-exp of its key range; a second kernel merges
  int n_splits;
  int ctas_per_split;
  float* part_o;       // [n_splits, B, Hq, M, D]
  float* part_lse;     // [n_splits, B, Hq, M]
  float* part_lse2;    // MODE 2: the same for the perturbed scores
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int kStages = (D == 128) ? 2 : 4;
  static constexpr int kChunks = D / 64;
  static constexpr int kChunkBytes = 128 * 128;            // 128 rows x 64 elements
  static constexpr int kTileBytes = kChunks * kChunkBytes;
  static constexpr int kQOff = 0;                          // two q tiles
  static constexpr int kKVOff = 2 * kTileBytes;
  static constexpr int kBarOff = kKVOff + kStages * 2 * kTileBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

struct TileInfo {
  int h;          // query head
  int q0;         // first query row
  int n_blocks;   // key blocks this CTA visits for the tile
  bool present;   // the tile exists (it has query rows)
};

// DUP (at most 32 queries per head: decode, chunked prefill, the reference's M = 16): the queries are loaded
// four times into the 128 tile rows, so that S has four identical 32-row replicas, and replica r (= warp r of
// the tile's softmax warpgroup) works only on score columns [32 r, 32 r + 32) of every key block.  Its rows of P
// are zero elsewhere, so each replica accumulates an independent partial (o, lse) over a quarter of the keys;
// the four are merged inside the CTA through shared memory before anything is written.  The per-row work of
// a thread drops four-fold.
constexpr int kDupRows = 32;
constexpr int kDup = BQ / kDupRows;

template <typename T, int D, int MODE, int PF, bool DUP>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
  using SM = AttnSmem<D>;
  constexpr int KS = SM::kStages;
  // PF: how p enters the P v product.  0: two 16-bit parts hi + lo of the io type (~16 mantissa bits of p);
  // 1: one part of the io type (8 bits for bf16, 11 for fp16).  p and v must have the same 16-bit type: a
  // kind::f16 product of an fp16 A with a bf16 B is refused by the tensor core (illegal instruction on B200).
  constexpr bool SPLIT = (PF == 0);
  using PT = T;
  // MODE 0: attention; 1: perturbed log-sum-exp only; 2: both in one pass; 3: attention that also keeps its scores;
  // 4: MODE 2 for generated Gumbel noise at tau = 1, where exp(s + g) = exp(s) / E with E = -ln u: the perturbed
  //    weight is the plain weight the pass computes anyway times 1 / E (one lg2 and one rcp per score instead of
  //    two lg2 and a second ex2), and the perturbed sum shares the plain softmax's running maximum
  constexpr bool kHasPV = (MODE != 1);                 // P, v and O exist
  constexpr bool kPert = (MODE == 1 || MODE == 2);     // perturbed log-sum-exp through its own online state
  constexpr bool kPertT1 = (MODE == 4);                // perturbed sum as p / E beside the plain row sum
  constexpr bool kDump = (MODE == 3);                  // plain scores written out
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + SM::kBarOff;
  // barriers: q_full, k_full[KS], v_full[KS], kv_empty[KS], s_full[2], pv_done[2], p_ready[2 tiles][2 halves]
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (1 + KS + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (1 + 2 * KS + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (1 + 3 * KS + t); };
  auto pv_done = [&](int t) { return bar_base + 8u * (3 + 3 * KS + t); };
  // P of a block becomes ready in two halves (keys 0..63, 64..127) so that P v starts on the first half
  // while the softmax threads still work on the second
  auto p_ready = [&](int t, int half) { return bar_base + 8u * (5 + 3 * KS + 2 * t + half); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + SM::kBarOff + 8 * (9 + 3 * KS));
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
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_ready(t, 0), 128);
      mbar_init(p_ready(t, 1), 128);
      mbar_init(pv_done(t), 1);
    }
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
  // everything above overlapped the previous kernel's tail (the projection that writes q / k / v); from here on its
  // results are read.  The next kernel (merge, statistics) may start its own prologue.
  griddep_wait();
  griddep_launch();

  // ---- which two tiles: heavy (late) query blocks first so the causal tail is short
  const int split = static_cast<int>(blockIdx.x) / p.ctas_per_split;
  const int cta = static_cast<int>(blockIdx.x) - split * p.ctas_per_split;
  const int row_blk = cta / p.units;
  const int unit = cta % p.units;
  int b, kvh;
  TileInfo tile[2];
  if (p.pair_heads) {
    const int pairs_per_group = (p.group + 1) >> 1;
    const int pi = unit % pairs_per_group;
    const int bk = unit / pairs_per_group;
    kvh = bk % p.Hkv;
    b = bk / p.Hkv;
    const int qb = p.n_qblocks - 1 - row_blk;
    tile[0].h = kvh * p.group + 2 * pi;
    tile[1].h = tile[0].h + 1;
    tile[0].q0 = tile[1].q0 = qb * BQ;
    tile[0].n_blocks = 1;
    tile[1].n_blocks = (2 * pi + 1 < p.group) ? 1 : 0;
  } else {
    const int n_qb2 = (p.n_qblocks + 1) >> 1;
    const int qb2 = n_qb2 - 1 - row_blk;
    b = unit / p.Hq;
    const int h = unit - b * p.Hq;
    kvh = h / p.group;
    tile[0].h = tile[1].h = h;
    tile[0].q0 = qb2 * 2 * BQ;
    tile[1].q0 = tile[0].q0 + BQ;
    tile[0].n_blocks = 1;
    tile[1].n_blocks = (tile[1].q0 < p.M) ? 1 : 0;
  }
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    if (tile[t].n_blocks) {
      const int q_hi = min(tile[t].q0 + BQ, p.M);
      const int kv_end = p.causal ? min(p.L, p.P + q_hi) : p.L;
      tile[t].n_blocks = (kv_end + BKV - 1) / BKV;
    }
  }
  tile[0].present = tile[0].n_blocks > 0;
  tile[1].present = tile[1].n_blocks > 0;
  int j0 = 0;           // first key block of this CTA
  if (p.n_splits > 1) {
    const int n_full = max(tile[0].n_blocks, tile[1].n_blocks);
    j0 = (n_full * split) / p.n_splits;
    const int j1 = (n_full * (split + 1)) / p.n_splits;
    tile[0].n_blocks = max(0, min(j1, tile[0].n_blocks) - j0);
    tile[1].n_blocks = max(0, min(j1, tile[1].n_blocks) - j0);
  }
  const int n_max = max(tile[0].n_blocks, tile[1].n_blocks);

  auto q_s = [&](int t) { return smem_base + SM::kQOff + t * SM::kTileBytes; };
  auto k_s = [&](int s) { return smem_base + SM::kKVOff + s * 2 * SM::kTileBytes; };
  auto v_s = [&](int s) { return k_s(s) + SM::kTileBytes; };

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      if (kHasPV) tma_prefetch_desc(&tm_v);
      const int n_tiles = (tile[0].n_blocks ? 1 : 0) + (tile[1].n_blocks ? 1 : 0);
      mbar_expect_tx(q_full, n_tiles * SM::kTileBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (tile[t].n_blocks) {
#pragma unroll
          for (int c = 0; c < SM::kChunks; ++c) {
            if constexpr (DUP) {
              // the descriptor's box is 32 rows: the same queries land in each quarter of the tile
#pragma unroll
              for (int rep = 0; rep < kDup; ++rep)
                tma_load_head_tile(q_s(t) + c * SM::kChunkBytes + rep * kDupRows * 128, &tm_q, q_full, p.qi, c * 64,
                                   tile[t].q0, tile[t].h, b);
            } else {
              tma_load_head_tile(q_s(t) + c * SM::kChunkBytes, &tm_q, q_full, p.qi, c * 64, tile[t].q0, tile[t].h, b);
            }
          }
        }
      }
    }
    for (int j = 0; j < n_max; ++j) {
      const int st = j % KS;
      const uint32_t ph = (j / KS) & 1;
      bool ok = mbar_wait(kv_empty(st), ph ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(k_full(st), SM::kTileBytes);
#pragma unroll
        for (int c = 0; c < SM::kChunks; ++c)
          tma_load_head_tile(k_s(st) + c * SM::kChunkBytes, &tm_k, k_full(st), p.ki, c * 64, (j0 + j) * BKV, kvh, b);
        if (kHasPV) {
          mbar_expect_tx(v_full(st), SM::kTileBytes);
#pragma unroll
          for (int c = 0; c < SM::kChunks; ++c)
            tma_load_head_tile(v_s(st) + c * SM::kChunkBytes, &tm_v, v_full(st), p.vi, c * 64, (j0 + j) * BKV, kvh, b);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    constexpr uint32_t idesc_qk = make_idesc_f16(Io<T>::kFmt, 0, 0, BQ, BKV);   // q, k both K-major
    constexpr uint32_t idesc_pv = make_idesc_f16(Io<T>::kFmt, 0, 1, BQ, D);     // P (TMEM) K-major, v MN-major
    bool ok = mbar_wait(q_full, 0, ctl, KST_TIMEOUT_MMA);
    ok = __all_sync(0xffffffffu, ok);
    // S_t = q_t k_j^T   (k_full(j) must have been waited for)
    auto issue_qk = [&](int t, int j) {
      if (lane == 0) {
        const int st = j % KS;
        const uint32_t d_tmem = tmem_base + t * BKV;
        // descriptors are built once per block and advanced by constants (the address field counts 16 bytes)
        const uint64_t qd = make_smem_desc(q_s(t), 0, 1024);
        const uint64_t kd = make_smem_desc(k_s(st), 0, 1024);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * SM::kChunkBytes + (kk & 3) * 32) >> 4);
          umma_ss(d_tmem, qd + off, kd + off, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full(t));
      }
      __syncwarp();
    };
    if (ok && n_max > 0) {
      ok = mbar_wait(k_full(0), 0, ctl, KST_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && n_max > 0) {
      tc_fence_after();
      for (int t = 0; t < 2; ++t)
        if (tile[t].n_blocks) issue_qk(t, 0);
    }
    for (int j = 0; j < n_max && ok; ++j) {
      const int st = j % KS;
      const uint32_t ph = (j / KS) & 1;
      bool k_next_ready = false;
      for (int t = 0; t < 2 && ok; ++t) {
        if (j >= tile[t].n_blocks) continue;
        if (kHasPV) {
          bool w = mbar_wait(v_full(st), ph, ctl, KST_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, w);
          if (!ok) break;
          const uint32_t o_tmem = tmem_base + 2 * BKV + t * BKV;
          const uint32_t p_tmem = tmem_base + t * BKV;
          const uint64_t vd = make_smem_desc(v_s(st), SM::kChunkBytes, 1024);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            // first / second 64 keys of P_t(j) are in TMEM
            ok = mbar_wait(p_ready(t, half), j & 1, ctl, KST_TIMEOUT_MMA);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
              // P_t sits over S_t, per 32 score columns c: [hi of keys 32c..32c+31 | lo of the same keys],
              // 16 columns (32 packed values) each.  One MMA consumes 16 keys = 8 columns.
#pragma unroll
              for (int k4 = 0; k4 < BKV / 32; ++k4) {
                const int kk = half * (BKV / 32) + k4;
                const uint32_t a_col = (kk >> 1) * 32 + (kk & 1) * 8;
                const uint64_t bdesc = vd + static_cast<uint64_t>((kk * 2048) >> 4);
                umma_ts(o_tmem, p_tmem + a_col, bdesc, idesc_pv, (j | kk) != 0 ? 1u : 0u);
                if constexpr (SPLIT) umma_ts(o_tmem, p_tmem + a_col + 16, bdesc, idesc_pv, 1u);
              }
              if (half == 1) umma_commit(pv_done(t));
            }
            __syncwarp();
          }
          if (!ok) break;
        } else {
          // the softmax warpgroup of tile t has consumed S_t(j)
          ok = mbar_wait(p_ready(t, 1), j & 1, ctl, KST_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        if (j + 1 < tile[t].n_blocks) {
          if (!k_next_ready) {
            const int st1 = (j + 1) % KS;
            const uint32_t ph1 = ((j + 1) / KS) & 1;
            ok = mbar_wait(k_full(st1), ph1, ctl, KST_TIMEOUT_MMA);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            k_next_ready = true;
          }
          issue_qk(t, j + 1);
        }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(kv_empty(st));   // every MMA that read stage st has been issued
      __syncwarp();
    }
  } else {
    // ------------------------------- softmax / epilogue (warps 2..9) -------------------------------
    const int t = (warp - 2) >> 2;                 // which tile this warpgroup owns
    const int quad = warp & 3;                     // TMEM lane quarter of this warp
    const int row = quad * 32 + lane;
    const int q_abs = tile[t].q0 + (DUP ? (row & (kDupRows - 1)) : row);
    const int h = tile[t].h;
    const int n_blocks = tile[t].n_blocks;
    const bool row_valid = q_abs < p.M;
    // a warp whose 32 rows all lie past the last query (M = 16 new tokens fill half of one warp) only keeps
    // the barrier protocol going: its rows of S / P / O are never stored and feed no other row
    const bool warp_active = DUP || tile[t].q0 + quad * 32 < p.M;
    auto my_chunk = [&](int c) { return !DUP || c == quad; };      // DUP: replica `quad` owns chunk `quad`
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const int limit = p.causal ? min(p.P + q_abs, p.L - 1) : p.L - 1;               // last visible key of this row
    const int limit_min = p.causal ? min(p.P + tile[t].q0, p.L - 1) : p.L - 1;     // ... of the tile's first row
    const uint32_t s_tmem = tmem_base + t * BKV + lane_addr;
    const uint32_t o_tmem = tmem_base + 2 * BKV + t * BKV + lane_addr;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    uint32_t r[32];
    const uint32_t rowhash =
        (kPert || kPertT1) ? noise_rowhash(noise_headkey(p.noise.seed, static_cast<uint32_t>(b * p.noise.Hq + h + p.noise.bh0)),
                              static_cast<uint32_t>(q_abs))
              : 0u;
    // state of the perturbed log-sum-exp, and where this row's scores go when they are kept
    float m2_run = -INFINITY, l2_run = 0.f;
    float* score_row = (p.scores != nullptr && row_valid)
                           ? p.scores + ((static_cast<long long>(b) * p.Hq + h) * p.M + q_abs) * p.score_pitch
                           : nullptr;
    // DUP + noise tensor: the 32 noise values of the replica's chunk are requested before the wait for S, so that
    // their latency (HBM, when the projection's weights have just swept the L2) overlaps that wait
    uint4 noise_pre[4];
    bool noise_pre_ok = false;
    // Perturbed scores of chunk c of block kv0 (S values in r[]): online log-sum-exp update, optional write-out.
    // t = (s * scale + g) * log2(e) / tau; with generated noise g = -ln2 * log2(E):  t = s * c_s + log2(E) * c_g
    //
    // The exponentials of a chunk are DEFERRED to the next call: tv[] keeps the chunk's perturbed scores and
    // pend_m the maximum they are to be taken against, and the next chunk's generator (integer and lg2 work)
    // runs between them, so that the XU pipe and the other pipes stay busy together instead of in turns.
    // l2_run is relative to m_l, the maximum of the last chunk folded in; pert_flush() folds the last one.
    float tv[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) tv[i] = -INFINITY;
    float pend_m = -INFINITY, m_l = -INFINITY;
    auto pert_fold = [&](float accp) {
      if (pend_m != -INFINITY) {
        l2_run = l2_run * ex2_approx(m_l - pend_m) + accp;      // m_l = -inf, l2_run = 0 on the first fold
        m_l = pend_m;
      }
    };
    auto pert_flush = [&]() {
      const float sub = (pend_m == -INFINITY) ? 0.f : pend_m;
      float accp = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) accp += ex2_approx(tv[i] - sub);
      pert_fold(accp);
      pend_m = -INFINITY;
      m2_run = m_l;
    };
    auto pert_chunk = [&](int kv0, int c, bool masked) {
      const bool fast = p.noise.mode == TRN_NOISE_GUMBEL;
      const float sub = (pend_m == -INFINITY) ? 0.f : pend_m;     // tv[] = -inf then: every term is 0
      float accp = 0.f;
      // 128-bit loads need the noise rows 16-byte aligned (checked once on the host)
      const bool fast_tensor = !masked && p.noise.mode == TRN_NOISE_TENSOR && p.noise_vec_ok;
      const float c_s = p.scale * p.pert_log2;
      const float c_g = -0.6931471805599453f * p.pert_log2;
      float cm = -INFINITY;
      if (fast) {
        // generated noise, no per-element compare.  Written stage by stage over groups of eight keys: with two
        // arithmetic warps per scheduler the order of independent instructions decides how well the XU pipe
        // (two lg2 per key) overlaps the integer and fp32 work, and this order measured 16 % faster than one
        // key after the other
        constexpr int G = 8;
        const uint32_t jbase = static_cast<uint32_t>(kv0 + c * 32) * 0x85ebca6bu;
#pragma unroll
        for (int i0 = 0; i0 < 32; i0 += G) {
          uint32_t x[G];
          float u[G], w[G];
#pragma unroll
          for (int i = 0; i < G; ++i) x[i] = rowhash ^ (jbase + static_cast<uint32_t>(i0 + i) * 0x85ebca6bu);
#pragma unroll
          for (int i = 0; i < G; ++i) x[i] ^= x[i] >> 16;
#pragma unroll
          for (int i = 0; i < G; ++i) x[i] *= 0x7feb352du;
#pragma unroll
          for (int i = 0; i < G; ++i) x[i] = (x[i] ^ (x[i] >> 15)) >> 9;
#pragma unroll
          for (int i = 0; i < G; ++i) accp += ex2_approx(tv[i0 + i] - sub);      // the previous chunk's
#pragma unroll
          for (int i = 0; i < G; ++i) u[i] = lg2_approx(unit_from_23bits(x[i]));
#pragma unroll
          for (int i = 0; i < G; ++i) {
            const float v = unit_from_23bits(x[i] ^ 0x7fffffu);                 // 1 - u, exact
            const float w_ser = fmaf(0.5f * v, v, v);
            w[i] = (v < kGumbelSeriesBelow) ? w_ser : -0.6931471805599453f * u[i];
          }
#pragma unroll
          for (int i = 0; i < G; ++i) w[i] = lg2_approx(w[i]);
#pragma unroll
          for (int i = 0; i < G; ++i) {
            const float v = fmaf(w[i], c_g, __uint_as_float(r[i0 + i]) * c_s);
            tv[i0 + i] = v;
            cm = fmaxf(cm, v);
          }
        }
        if (masked) {
          // block on the causal diagonal or past the last key: drop the invisible keys afterwards, so that
          // the loop above stays the only copy of the generator
          cm = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (kv0 + c * 32 + i > limit) tv[i] = -INFINITY;
            cm = fmaxf(cm, tv[i]);
          }
        }
      } else if (fast_tensor) {
#pragma unroll
        for (int i = 0; i < 32; ++i) accp += ex2_approx(tv[i] - sub);
        // interior block, noise tensor: this row's 32 values come in as four 128-bit loads
        const T* nrow = static_cast<const T*>(p.noise.ptr) + b * p.noise.sb + h * p.noise.sh +
                        static_cast<long long>(row_valid ? q_abs : 0) * p.noise.si + kv0 + c * 32;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          const uint4 nv = (DUP && noise_pre_ok) ? noise_pre[i >> 3] : __ldg(reinterpret_cast<const uint4*>(nrow + i));
          const uint32_t w4[4] = {nv.x, nv.y, nv.z, nv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 g2 = Io<T>::unpack2(w4[e]);
            const float v0 = (__uint_as_float(r[i + 2 * e]) * p.scale + g2.x) * p.pert_log2;
            const float v1 = (__uint_as_float(r[i + 2 * e + 1]) * p.scale + g2.y) * p.pert_log2;
            tv[i + 2 * e] = v0;
            tv[i + 2 * e + 1] = v1;
            cm = fmax3(cm, v0, v1);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) accp += ex2_approx(tv[i] - sub);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = kv0 + c * 32 + i;
          float v = -INFINITY;
          if (col <= limit) {
            const float g = row_valid ? noise_at<T>(p.noise, rowhash, b, h, q_abs, col) : 0.f;
            v = (__uint_as_float(r[i]) * p.scale + g) * p.pert_log2;
          }
          tv[i] = v;
          cm = fmaxf(cm, v);
        }
      }
      pert_fold(accp);
      m2_run = fmaxf(m2_run, cm);
      pend_m = m2_run;            // -inf while the row has seen no visible key: tv[] is all -inf then
      if (score_row != nullptr && kv0 + c * 32 < p.score_pitch) {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(score_row + kv0 + c * 32 + i) = make_float4(tv[i], tv[i + 1], tv[i + 2], tv[i + 3]);
      }
    };
    // plain scores of chunk c (S values in r[]) written out in the log2 domain; keys past a row's limit as -inf
    auto dump_chunk = [&](int kv0, int c, bool masked) {
      if (score_row == nullptr || kv0 + c * 32 >= p.score_pitch) return;
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 v = make_float4(__uint_as_float(r[i]) * p.scale_log2, __uint_as_float(r[i + 1]) * p.scale_log2,
                               __uint_as_float(r[i + 2]) * p.scale_log2, __uint_as_float(r[i + 3]) * p.scale_log2);
        if (masked) {
          const int col = kv0 + c * 32 + i;
          if (col > limit) v.x = -INFINITY;
          if (col + 1 > limit) v.y = -INFINITY;
          if (col + 2 > limit) v.z = -INFINITY;
          if (col + 3 > limit) v.w = -INFINITY;
        }
        *reinterpret_cast<float4*>(score_row + kv0 + c * 32 + i) = v;
      }
    };

    for (int j = 0; j < n_blocks; ++j) {
      const int kv0 = (j0 + j) * BKV;
      if constexpr (DUP && kPert) {
        noise_pre_ok = p.noise.mode == TRN_NOISE_TENSOR && p.noise_vec_ok && (kv0 + BKV - 1) <= limit_min;
        if (noise_pre_ok) {
          const T* nrow = static_cast<const T*>(p.noise.ptr) + b * p.noise.sb + h * p.noise.sh +
                          static_cast<long long>(row_valid ? q_abs : 0) * p.noise.si + kv0 + quad * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) noise_pre[i] = __ldg(reinterpret_cast<const uint4*>(nrow + 8 * i));
        }
      }
      ok = mbar_wait(s_full(t), j & 1, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (!warp_active) {
        if (kHasPV) mbar_arrive(p_ready(t, 0));
        mbar_arrive(p_ready(t, 1));
        continue;
      }
      const bool masked = (kv0 + BKV - 1) > limit_min;

      if (MODE == 1) {
        // one pass, chunk-wise online log-sum-exp of the perturbed scores
#pragma unroll 1
        for (int c = 0; c < BKV / 32; ++c) {
          if (!my_chunk(c)) continue;
          tmem_ld32(s_tmem + c * 32, r);
          tmem_wait_ld();
          pert_chunk(kv0, c, masked);
        }
        tc_fence_before();
        mbar_arrive(p_ready(t, 1));
        continue;
      }

      // ---- pass 1: block maximum of this row
      float mb = -INFINITY;
      if constexpr (kPert || kDump) {
        // one loop with one call site of the perturbed-score code: this variant's instruction footprint matters
        // when the projection's weights have just swept the L2 (the reference's M = 16 shapes)
#pragma unroll 1
        for (int c = 0; c < BKV / 32; ++c) {
          if (!my_chunk(c)) continue;
          tmem_ld32(s_tmem + c * 32, r);
          tmem_wait_ld();
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kv0 + c * 32 + i <= limit) mb = fmaxf(mb, __uint_as_float(r[i]));
          } else {
            float m0 = fmaxf(__uint_as_float(r[0]), __uint_as_float(r[1]));
            float m1 = fmaxf(__uint_as_float(r[2]), __uint_as_float(r[3]));
#pragma unroll
            for (int i = 4; i < 32; i += 4) {
              m0 = fmax3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
              m1 = fmax3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
            }
            mb = fmax3(mb, m0, m1);
          }
          if constexpr (kPert) pert_chunk(kv0, c, masked);
          else dump_chunk(kv0, c, masked);
        }
      } else if (masked) {
        for (int c = 0; c < BKV / 32; ++c) {
          if (!my_chunk(c)) continue;
          tmem_ld32(s_tmem + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (kv0 + c * 32 + i <= limit) mb = fmaxf(mb, __uint_as_float(r[i]));
        }
      } else {
        for (int c = 0; c < BKV / 32; ++c) {
          if (!my_chunk(c)) continue;
          tmem_ld32(s_tmem + c * 32, r);
          tmem_wait_ld();
          float m0 = fmaxf(__uint_as_float(r[0]), __uint_as_float(r[1]));
          float m1 = fmaxf(__uint_as_float(r[2]), __uint_as_float(r[3]));
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            m0 = fmax3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            m1 = fmax3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          }
          mb = fmax3(mb, m0, m1);
        }
      }
      mb *= p.scale_log2;                         // scale > 0, so max commutes with it
      // m_run is the exponent offset in use: (row max seen at the last rescale) - kPBias.  fp16 has few
      // exponent bits, so its p values are biased up by 2^4 to keep the low-order part of p out of
      // the subnormal range; bf16 needs no bias.
      constexpr float kPBias = (Io<PT>::kFmt == 0) ? 4.0f : 0.0f;
      const float m_target = mb - kPBias;
      const bool grow = (m_target - m_run) > kRescaleThreshold;   // first block: m_run = -inf -> true
      float alpha = 1.0f;
      if (grow) {
        alpha = ex2_approx(m_run - m_target);     // 0 on the first block
        m_run = m_target;
      }
      // S_t(j) was produced after P_t(j-1) v (MMAs run in issue order), so O_t is quiescent here
      bool r_holds_s = DUP;          // DUP: r[] still holds the replica's chunk of S from pass 1 ...
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        r_holds_s = false;           // ... unless it is used as scratch here
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld32(o_tmem + c * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(o_tmem + c * 32, r);
        }
        l_run *= alpha;
        if constexpr (kPertT1) l2_run *= alpha;
      }
      // ---- pass 2: p = 2^(s * c - m), row sum, P written over S (hi | lo per 32 score columns).
      //      Arithmetic on pairs of columns uses the packed fp32x2 instructions of sm_100.
      float2 lsum = make_float2(0.f, 0.f);
      float2 lsum2 = make_float2(0.f, 0.f);            // MODE 4: sum of p / E
      const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
      const float2 neg_m2 = make_float2(-m_run, -m_run);
      const float2 minus1 = make_float2(-1.f, -1.f);
      // compiled twice: the unmasked version carries no per-element compare / select
      auto pass2 = [&](auto masked_tag) {
        constexpr bool kMasked = decltype(masked_tag)::value;
        // p of the 32 score columns of chunk c held in src[] -> pk[] (hi parts, then lo parts), row sum
        auto chunk_p = [&](const uint32_t (&src)[32], int c, uint32_t (&pk)[SPLIT ? 32 : 16]) {
          // stage by stage over groups of eight column pairs: one softmax warp per scheduler is active at a
          // time, so the order of independent instructions decides how much of each result's latency is hidden
          constexpr int G = 8;
#pragma unroll
          for (int i0 = 0; i0 < 16; i0 += G) {
            float2 pp[G];
#pragma unroll
            for (int i = 0; i < G; ++i)
              pp[i] = __ffma2_rn(make_float2(__uint_as_float(src[2 * (i0 + i)]), __uint_as_float(src[2 * (i0 + i) + 1])),
                                 c2, neg_m2);
#pragma unroll
            for (int i = 0; i < G; ++i) pp[i] = make_float2(ex2_approx(pp[i].x), ex2_approx(pp[i].y));
            if constexpr (kMasked) {
#pragma unroll
              for (int i = 0; i < G; ++i) {
                if (kv0 + c * 32 + 2 * (i0 + i) > limit) pp[i].x = 0.f;
                if (kv0 + c * 32 + 2 * (i0 + i) + 1 > limit) pp[i].y = 0.f;
              }
            }
#pragma unroll
            for (int i = 0; i < G; ++i) pk[i0 + i] = Io<PT>::pack2(pp[i].x, pp[i].y);
#pragma unroll
            for (int i = 0; i < G; ++i) lsum = __fadd2_rn(lsum, pp[i]);
            if constexpr (kPertT1) {
              // 1 / E of the same 16 keys (E = -ln u from the counter-based bits), stage by stage over four pairs
              // at a time; masked keys have p = 0 and add nothing
              constexpr int H = 4;
#pragma unroll
              for (int h0 = 0; h0 < G; h0 += H) {
                const uint32_t jb = static_cast<uint32_t>(kv0 + c * 32 + 2 * (i0 + h0)) * 0x85ebca6bu;
                uint32_t xa[H], xb[H];
                float2 e2[H];
#pragma unroll
                for (int i = 0; i < H; ++i) {
                  xa[i] = rowhash ^ (jb + static_cast<uint32_t>(2 * i) * 0x85ebca6bu);
                  xb[i] = rowhash ^ (jb + static_cast<uint32_t>(2 * i + 1) * 0x85ebca6bu);
                }
#pragma unroll
                for (int i = 0; i < H; ++i) { xa[i] ^= xa[i] >> 16; xb[i] ^= xb[i] >> 16; }
#pragma unroll
                for (int i = 0; i < H; ++i) { xa[i] *= 0x7feb352du; xb[i] *= 0x7feb352du; }
#pragma unroll
                for (int i = 0; i < H; ++i) { xa[i] = (xa[i] ^ (xa[i] >> 15)) >> 9; xb[i] = (xb[i] ^ (xb[i] >> 15)) >> 9; }
#pragma unroll
                for (int i = 0; i < H; ++i)
                  e2[i] = make_float2(lg2_approx(unit_from_23bits(xa[i])), lg2_approx(unit_from_23bits(xb[i])));
#pragma unroll
                for (int i = 0; i < H; ++i) {
                  const float va = unit_from_23bits(xa[i] ^ 0x7fffffu), vb = unit_from_23bits(xb[i] ^ 0x7fffffu);   // 1 - u
                  const float sa = fmaf(0.5f * va, va, va), sb = fmaf(0.5f * vb, vb, vb);
                  e2[i].x = (va < kGumbelSeriesBelow) ? sa : -0.6931471805599453f * e2[i].x;
                  e2[i].y = (vb < kGumbelSeriesBelow) ? sb : -0.6931471805599453f * e2[i].y;
                }
#pragma unroll
                for (int i = 0; i < H; ++i) e2[i] = make_float2(rcp_approx(e2[i].x), rcp_approx(e2[i].y));
#pragma unroll
                for (int i = 0; i < H; ++i) lsum2 = __ffma2_rn(pp[h0 + i], e2[i], lsum2);
              }
            }
            if constexpr (SPLIT) {
              // p = hi + lo with both parts 16-bit: the P v product keeps ~16 mantissa bits of p
#pragma unroll
              for (int i = 0; i < G; ++i) pp[i] = __ffma2_rn(Io<PT>::unpack2(pk[i0 + i]), minus1, pp[i]);   // p - hi, exact
#pragma unroll
              for (int i = 0; i < G; ++i) pk[16 + i0 + i] = Io<PT>::pack2(pp[i].x, pp[i].y);
            }
          }
        };
        auto store_p = [&](int c, uint32_t (&pk)[SPLIT ? 32 : 16]) {
          if constexpr (SPLIT) {
            tmem_st32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(pk));
          } else {
            tmem_st16(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[16]>(pk));
          }
        };
        auto first_half_ready = [&]() {        // keys 0..63 of P are written: let P v begin
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(p_ready(t, 0));
        };
        if constexpr (DUP) {
#pragma unroll 1
          for (int c = 0; c < BKV / 32; ++c) {
            uint32_t pk[SPLIT ? 32 : 16];
            if (my_chunk(c)) {
              if (!r_holds_s) {          // warp-uniform
                tmem_ld32(s_tmem + c * 32, r);
                tmem_wait_ld();
              }
              chunk_p(r, c, pk);
            } else {
              // another replica's columns: this replica's p is zero there
#pragma unroll
              for (int i = 0; i < (SPLIT ? 32 : 16); ++i) pk[i] = 0u;
            }
            store_p(c, pk);
            if (c == 1) first_half_ready();
          }
        } else {
          // two register buffers: the tensor-memory load of the next chunk is in flight while this one is worked on
          uint32_t rb[32];
          tmem_ld32(s_tmem, r);
          tmem_wait_ld();
#pragma unroll 1
          for (int c = 0; c < BKV / 32; c += 2) {
            uint32_t pk[SPLIT ? 32 : 16];
            tmem_ld32(s_tmem + (c + 1) * 32, rb);
            chunk_p(r, c, pk);
            store_p(c, pk);
            tmem_wait_ld();
            if (c + 2 < BKV / 32) tmem_ld32(s_tmem + (c + 2) * 32, r);
            chunk_p(rb, c + 1, pk);
            store_p(c + 1, pk);
            if (c == 0) first_half_ready();
            tmem_wait_ld();
          }
        }
      };
      if (masked) pass2(std::true_type{});
      else pass2(std::false_type{});
      l_run += lsum.x + lsum.y;
      if constexpr (kPertT1) l2_run += lsum2.x + lsum2.y;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_ready(t, 1));
    }

    const bool split_out = p.n_splits > 1;
    const long long part_row =
        ((static_cast<long long>(split) * p.B + b) * p.Hq + h) * p.M + q_abs;   // row of the partial results
    if constexpr (kPert) pert_flush();
    if constexpr (kPertT1) m2_run = m_run;                    // p / E sums are relative to the plain offset
    constexpr bool kTwoLse = (MODE == 2 || MODE == 4);       // a second (perturbed) log-sum-exp is reported
    if (MODE == 1) { m_run = m2_run; l_run = l2_run; }        // MODE 1 reports the perturbed value as its lse
    if constexpr (DUP) {
      // ---- merge the four replicas of this tile inside the CTA.  The k / v stages and the q tiles are free once
      //      the last MMAs of BOTH tiles have run (they share the k / v stream): o goes through the stage area as
      //      [replica][column][row] fp32 (conflict-free both ways), the log-sum-exps through the tile's q area.
      if (tile[t].present && n_blocks > 0) {          // uniform over the warpgroup
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (ok && tile[u].n_blocks > 0) {
            ok = kHasPV ? mbar_wait(pv_done(u), (tile[u].n_blocks - 1) & 1, ctl, KST_TIMEOUT_CONSUMER)
                        : mbar_wait(s_full(u), (tile[u].n_blocks - 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
            ok = __all_sync(0xffffffffu, ok);
          }
        }
        float* xo = reinterpret_cast<float*>(smem_gen + SM::kKVOff) + t * (kDup * D * kDupRows);
        float* xl = reinterpret_cast<float*>(smem_gen + SM::kQOff + t * SM::kTileBytes);     // [2][replica][row]
        const float lse1 = m_run + log2f(l_run);            // -inf when this replica saw no visible key
        const float lse2v = kTwoLse ? m2_run + log2f(l2_run) : 0.f;
        if (ok && kHasPV) {
          tc_fence_after();
          const float inv_l = (l_run > 0.f) ? 1.0f / l_run : 0.f;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld32(o_tmem + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) xo[(quad * D + c * 32 + i) * kDupRows + lane] = __uint_as_float(r[i]) * inv_l;
          }
          tc_fence_before();
        }
        xl[quad * kDupRows + lane] = lse1;
        if (kTwoLse) xl[(kDup + quad) * kDupRows + lane] = lse2v;
        // every warp of the warpgroup gets here (all waits above are bounded): named barrier 1 + t, 128 threads
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");
        // weights of the four replicas for row `lane`
        float w[kDup], mx = -INFINITY, tot = 0.f;
#pragma unroll
        for (int rp = 0; rp < kDup; ++rp) { w[rp] = xl[rp * kDupRows + lane]; mx = fmaxf(mx, w[rp]); }
#pragma unroll
        for (int rp = 0; rp < kDup; ++rp) { w[rp] = (w[rp] == -INFINITY) ? 0.f : ex2_approx(w[rp] - mx); tot += w[rp]; }
        const float inv_tot = 1.0f / tot;
        const int qrow = tile[t].q0 + lane;                 // this warp writes columns [quad * D/4, (quad+1) * D/4) of row `lane`
        const bool out_valid = qrow < p.M;
        const long long prow_idx = ((static_cast<long long>(split) * p.B + b) * p.Hq + h) * p.M + qrow;
        if (ok && kHasPV && out_valid) {
          constexpr int CW = D / kDup;                      // columns per warp: 32 or 16
          float acc[CW];
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            float v = 0.f;
#pragma unroll
            for (int rp = 0; rp < kDup; ++rp) v = fmaf(w[rp], xo[(rp * D + quad * CW + i) * kDupRows + lane], v);
            acc[i] = v * inv_tot;
          }
          if (split_out) {
            float* dst = p.part_o + prow_idx * D + quad * CW;
#pragma unroll
            for (int i = 0; i < CW; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
          } else {
            T* dst = static_cast<T*>(p.o) + static_cast<long long>(b) * p.o_sb + static_cast<long long>(qrow) * p.o_ss +
                     static_cast<long long>(h) * p.o_sh + quad * CW;
#pragma unroll
            for (int i = 0; i < CW; i += 8) {
              uint4 v;
              v.x = Io<T>::pack2(acc[i], acc[i + 1]); v.y = Io<T>::pack2(acc[i + 2], acc[i + 3]);
              v.z = Io<T>::pack2(acc[i + 4], acc[i + 5]); v.w = Io<T>::pack2(acc[i + 6], acc[i + 7]);
              *reinterpret_cast<uint4*>(dst + i) = v;
            }
          }
        }
        if (ok && out_valid && quad == 0) {
          const float lse_m = mx + log2f(tot);
          float lse2_m = 0.f;
          if (kTwoLse) {
            float m2 = -INFINITY, t2 = 0.f;
#pragma unroll
            for (int rp = 0; rp < kDup; ++rp) m2 = fmaxf(m2, xl[(kDup + rp) * kDupRows + lane]);
#pragma unroll
            for (int rp = 0; rp < kDup; ++rp) {
              const float v = xl[(kDup + rp) * kDupRows + lane];
              if (v != -INFINITY) t2 += ex2_approx(v - m2);
            }
            lse2_m = m2 + log2f(t2);
          }
          const long long li = (static_cast<long long>(b) * p.Hq + h) * p.M + qrow;
          if (split_out) {
            p.part_lse[prow_idx] = lse_m;
            if (kTwoLse) p.part_lse2[prow_idx] = lse2_m;
          } else {
            if (p.lse != nullptr) p.lse[li] = lse_m;
            if (kTwoLse) p.lse_pert[li] = lse2_m;
          }
        }
      } else if (split_out && tile[t].present && quad == 0 && tile[t].q0 + lane < p.M) {
        // this CTA's key range misses the tile: weight 0 in the merge kernel
        const long long prow_idx = ((static_cast<long long>(split) * p.B + b) * p.Hq + h) * p.M + tile[t].q0 + lane;
        p.part_lse[prow_idx] = -INFINITY;
        if (kTwoLse) p.part_lse2[prow_idx] = -INFINITY;
      }
    } else {
    if (ok && kHasPV && n_blocks > 0 && warp_active) {
      ok = mbar_wait(pv_done(t), (n_blocks - 1) & 1, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const float inv_l = 1.0f / l_run;
        T* orow = static_cast<T*>(p.o) + static_cast<long long>(b) * p.o_sb + static_cast<long long>(q_abs) * p.o_ss +
                  static_cast<long long>(h) * p.o_sh;
        float* prow = p.part_o + part_row * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld32(o_tmem + c * 32, r);
          tmem_wait_ld();
          if (row_valid && split_out) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(prow + c * 32 + i) =
                  make_float4(__uint_as_float(r[i]) * inv_l, __uint_as_float(r[i + 1]) * inv_l,
                              __uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l);
          } else if (row_valid) {
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
    if (split_out) {
      // a CTA whose key range misses this tile contributes weight 0
      if (ok && tile[t].present && row_valid) {
        p.part_lse[part_row] = (n_blocks > 0) ? m_run + log2f(l_run) : -INFINITY;
        if (kTwoLse) p.part_lse2[part_row] = (n_blocks > 0) ? m2_run + log2f(l2_run) : -INFINITY;
      }
    } else if (ok && n_blocks > 0 && row_valid) {
      const long long li = (static_cast<long long>(b) * p.Hq + h) * p.M + q_abs;
      if (p.lse != nullptr) p.lse[li] = m_run + log2f(l_run);
      if (kTwoLse) p.lse_pert[li] = m2_run + log2f(l2_run);
    }
    }   // !DUP
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

// Merges the partial results of a split-KV launch: one warp per (b, h, query) row.
//   w_s = 2^(lse_s - max_s lse_s);  o = sum_s w_s o_s / sum_s w_s;  lse = max + log2(sum_s w_s)
template <typename T, int D>
__global__ void __launch_bounds__(256)
attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, T* __restrict__ o,
                    long long o_sb, long long o_ss, long long o_sh, float* __restrict__ lse_out,
                    const float* __restrict__ part_lse2, float* __restrict__ lse2_out, int n_splits, int B,
                    int Hq, int M, const int* __restrict__ status) {
  griddep_wait();
  griddep_launch();
  if (*reinterpret_cast<const volatile int*>(status) != 0) return;
  constexpr int VPL = D / 32;
  const long long rows = static_cast<long long>(B) * Hq * M;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_lse[s * rows + row]);
  float tot = 0.f;
  float acc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ls = part_lse[s * rows + row];
    if (ls == -INFINITY) continue;             // this split saw no key of the row: its o was not written
    const float w = ex2_approx(ls - m);
    tot += w;
    if (part_o != nullptr) {
      const float* src = part_o + (s * rows + row) * D + lane * VPL;
      if constexpr (VPL == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
        acc[2] = fmaf(w, v.z, acc[2]); acc[3] = fmaf(w, v.w, acc[3]);
      } else {
        const float2 v = *reinterpret_cast<const float2*>(src);
        acc[0] = fmaf(w, v.x, acc[0]); acc[1] = fmaf(w, v.y, acc[1]);
      }
    }
  }
  const int q = static_cast<int>(row % M);
  const int h = static_cast<int>((row / M) % Hq);
  const int b = static_cast<int>(row / (static_cast<long long>(M) * Hq));
  if (part_o != nullptr) {
    const float inv = 1.0f / tot;
    T* dst = o + b * o_sb + q * o_ss + h * o_sh + lane * VPL;
    if constexpr (VPL == 4) {
      uint2 v;
      v.x = Io<T>::pack2(acc[0] * inv, acc[1] * inv);
      v.y = Io<T>::pack2(acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<uint2*>(dst) = v;
    } else {
      *reinterpret_cast<uint32_t*>(dst) = Io<T>::pack2(acc[0] * inv, acc[1] * inv);
    }
  }
  if (lse_out != nullptr && lane == 0) lse_out[row] = m + log2f(tot);
  if (part_lse2 != nullptr && lane == 0) {       // the perturbed scores' log-sum-exp merges the same way
    float m2 = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m2 = fmaxf(m2, part_lse2[s * rows + row]);
    float t2 = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ls = part_lse2[s * rows + row];
      if (ls != -INFINITY) t2 += ex2_approx(ls - m2);
    }
    lse2_out[row] = m2 + log2f(t2);
  }
}

// layout: lse partials, second lse partials (always reserved, used by MODE 2), then o partials
size_t split_lse_bytes(int n_splits, long long rows) {
  return (static_cast<size_t>(n_splits) * rows * sizeof(float) + 255) / 256 * 256;
}
size_t split_bytes(int n_splits, long long rows, int D, bool with_o) {
  const size_t o_b = with_o ? (static_cast<size_t>(n_splits) * rows * D * sizeof(float) + 255) / 256 * 256 : 0;
  return o_b + 2 * split_lse_bytes(n_splits, rows);
}

template <typename T, int D, int MODE, int PF, bool DUP>
int launch_inst(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  using SM = AttnSmem<D>;
  AttnParams p{};
  const int L = a.P + a.M;
  CUtensorMap tm_q, tm_k, tm_v;
  int rc = make_head_tmap(&tm_q, &p.qi, a.q, a.M, a.Hq, a.B, D, DUP ? kDupRows : BQ);
  if (rc != TRN_OK) return rc;
  rc = make_head_tmap(&tm_k, &p.ki, a.k_cache, L, a.Hkv, a.B, D, BKV);
  if (rc != TRN_OK) return rc;
  if (MODE != 1) {
    rc = make_head_tmap(&tm_v, &p.vi, a.v_cache, L, a.Hkv, a.B, D, BKV);
    if (rc != TRN_OK) return rc;
  } else {
    tm_v = tm_k;
    p.vi = p.ki;
  }
  p.o = a.o.ptr;
  p.o_sb = a.o.stride_b; p.o_ss = a.o.stride_s; p.o_sh = a.o.stride_h;
  p.lse = a.lse;
  p.lse_pert = a.lse_pert;
  p.scores = a.scores;
  p.score_pitch = static_cast<int>(a.score_pitch);
  p.B = a.B; p.M = a.M; p.P = a.P; p.L = L; p.Hq = a.Hq; p.Hkv = a.Hkv; p.group = a.Hq / a.Hkv;
  p.n_qblocks = (a.M + BQ - 1) / BQ;
  p.pair_heads = p.group >= 2 ? 1 : 0;
  long long rows_of_ctas;
  if (p.pair_heads) {
    p.units = a.B * a.Hkv * ((p.group + 1) / 2);
    rows_of_ctas = p.n_qblocks;
  } else {
    p.units = a.B * a.Hq;
    rows_of_ctas = (p.n_qblocks + 1) / 2;
  }
  p.causal = a.causal;
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
  p.noise_vec_ok = (a.noise != nullptr && aligned16(a.noise) && (a.noise_stride_b & 7) == 0 &&
                    (a.noise_stride_h & 7) == 0 && (a.noise_stride_i & 7) == 0)
                       ? 1
                       : 0;
  p.status = ds.status;
  auto kern = attn_fwd_kernel<T, D, MODE, PF, DUP>;
  rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), SM::kTotal, ds.device);
  if (rc != TRN_OK) return rc;
  const long long ctas = rows_of_ctas * p.units;
  if (ctas > 0x7fffffffLL) return TRN_E_SHAPE;
  // split-KV when the launch would leave most SMs idle and the caller lent scratch for the partials
  const long long rows = static_cast<long long>(a.B) * a.Hq * a.M;
  // under a causal mask a tile sees on average the prefix plus half of the new keys
  const int l_eff = a.causal ? a.P + (a.M + 1) / 2 : L;
  int n_splits = tls_attn_split_override > 0 ? tls_attn_split_override
                                             : attn_split_count(static_cast<int>(ctas), l_eff, ds.sm_count);
  if (n_splits > (L + BKV - 1) / BKV) n_splits = 1;
  const bool ws_ok = a.workspace != nullptr && (reinterpret_cast<uintptr_t>(a.workspace) & 255u) == 0;
  if (!ws_ok) n_splits = 1;
  while (n_splits > 1 && split_bytes(n_splits, rows, D, MODE != 1) > a.workspace_bytes) --n_splits;
  p.n_splits = n_splits;
  p.ctas_per_split = static_cast<int>(ctas);
  const int n_parts = n_splits;
  if (n_parts > 1) {
    uint8_t* ws = static_cast<uint8_t*>(a.workspace);
    const size_t l_b = split_lse_bytes(n_parts, rows);
    p.part_lse = reinterpret_cast<float*>(ws);
    p.part_lse2 = reinterpret_cast<float*>(ws + l_b);
    p.part_o = (MODE != 1) ? reinterpret_cast<float*>(ws + 2 * l_b) : nullptr;
  }
  TRN_CUDA_TRY(launch_pdl(kern, dim3(static_cast<unsigned>(ctas * n_splits)), dim3(kAttnThreads), SM::kTotal, st, tm_q, tm_k,
                          tm_v, p));
  if (n_parts > 1) {
    const int warps_per_cta = 8;
    const long long cgrid = (rows + warps_per_cta - 1) / warps_per_cta;
    TRN_CUDA_TRY(launch_pdl(attn_combine_kernel<T, D>, dim3(static_cast<unsigned>(cgrid)), dim3(warps_per_cta * 32), 0, st,
                            p.part_o, p.part_lse, static_cast<T*>(a.o.ptr), a.o.stride_b, a.o.stride_s, a.o.stride_h, a.lse,
                            (MODE == 2 || MODE == 4) ? p.part_lse2 : nullptr, a.lse_pert, n_parts, a.B, a.Hq, a.M,
                            ds.status));
  }
  return TRN_OK;
}

// few queries per head: the row-replicated variant
template <typename T, int D, int MODE, int PF>
int launch_variant(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  if constexpr (PF == 0 || MODE == 1) {
    if (a.M <= kDupRows) return launch_inst<T, D, MODE, PF, true>(a, st, ds);
  }
  return launch_inst<T, D, MODE, PF, false>(a, st, ds);
}

// single_p of the arguments -> PF of the kernel: 0 hi + lo, otherwise one part of the io type
template <typename T, int D, int MODE>
int launch_pf(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.single_p == 0) return launch_variant<T, D, MODE, 0>(a, st, ds);
  return launch_variant<T, D, MODE, 1>(a, st, ds);
}

template <typename T>
int launch_typed(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds) {
  const bool pert = a.noise_mode != TRN_NOISE_NONE;
  const bool fused = pert && a.lse_pert != nullptr;     // attention and the perturbed log-sum-exp in one pass
  // generated Gumbel noise at tau = 1 with no scores to keep: exp(s + g) = exp(s) / E
  const bool fused_t1 = fused && a.noise_mode == TRN_NOISE_GUMBEL && a.tau == 1.0f && a.scores == nullptr;
  if (a.D == 128) {
    if (fused_t1) return launch_pf<T, 128, 4>(a, st, ds);
    if (fused) return launch_pf<T, 128, 2>(a, st, ds);
    if (pert) return launch_variant<T, 128, 1, 1>(a, st, ds);
    if (a.scores != nullptr) return launch_pf<T, 128, 3>(a, st, ds);
    return launch_pf<T, 128, 0>(a, st, ds);
  }
  if (a.D == 64) {
    if (fused_t1) return launch_pf<T, 64, 4>(a, st, ds);
    if (fused) return launch_pf<T, 64, 2>(a, st, ds);
    if (pert) return launch_variant<T, 64, 1, 1>(a, st, ds);
    if (a.scores != nullptr) return launch_pf<T, 64, 3>(a, st, ds);
    return launch_pf<T, 64, 0>(a, st, ds);
  }
  return TRN_E_SHAPE;
}

bool ht_ok(const TrnHeadTensor& t) {
  return t.ptr != nullptr && aligned16(t.ptr) && (t.stride_b & 7) == 0 && (t.stride_s & 7) == 0 &&
         (t.stride_h & 7) == 0;
}

}  // namespace


int attn_split_count(int ctas, int L, int sm_count) {
  const int n_blocks = (L + BKV - 1) / BKV;
  if (ctas <= 0) return 1;
  const int want = min(min(sm_count / ctas, n_blocks / 2), kAttnMaxSplits);
  return want >= 2 ? want : 1;
}

thread_local int tls_attn_split_override = 0;

int attn_planned_splits(int B, int M, int P, int Hq, int Hkv, int D, int causal, int sm_count) {
  if (B <= 0 || M <= 0 || P < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || (D != 64 && D != 128)) return 1;
  const int group = Hq / Hkv;
  const long long n_qb = (M + BQ - 1) / BQ;
  const long long ctas = group >= 2 ? n_qb * B * Hkv * ((group + 1) / 2) : ((n_qb + 1) / 2) * B * Hq;
  if (ctas > sm_count) return 1;
  return attn_split_count(static_cast<int>(ctas), causal ? P + (M + 1) / 2 : P + M, sm_count);
}

size_t attn_split_workspace(int B, int M, int P, int Hq, int Hkv, int D, int sm_count) {
  const int n = attn_planned_splits(B, M, P, Hq, Hkv, D, /*causal=*/0, sm_count);     // the larger of the two cases
  if (n <= 1) return 0;
  return split_bytes(n, static_cast<long long>(B) * Hq * M, D, true);
}

int launch_attention(const TrnAttnArgs& a, cudaStream_t st, const DeviceState& ds, AttnFusedStats* fstats) {
  if (a.B <= 0 || a.M <= 0 || a.P < 0 || a.Hq <= 0 || a.Hkv <= 0 || a.Hq % a.Hkv != 0) return TRN_E_SHAPE;
  if (a.D != 64 && a.D != 128) return TRN_E_SHAPE;
  if (!(a.scale > 0.f)) return TRN_E_SHAPE;
  if (a.single_p < 0 || a.single_p > 1) return TRN_E_VARIANT;
  const bool pert = a.noise_mode != TRN_NOISE_NONE;
  if (a.noise_mode < TRN_NOISE_NONE || a.noise_mode > TRN_NOISE_GUMBEL) return TRN_E_VARIANT;
  if (a.q.ptr == nullptr || a.k_cache.ptr == nullptr) return TRN_E_NULL;
  if (!ht_ok(a.q) || !ht_ok(a.k_cache)) return TRN_E_ALIGN;
  const bool fused = pert && a.lse_pert != nullptr;
  if (!pert || fused) {
    if (a.v_cache.ptr == nullptr || a.o.ptr == nullptr) return TRN_E_NULL;
    if (!ht_ok(a.v_cache) || !ht_ok(a.o)) return TRN_E_ALIGN;
  }
  if (pert) {
    if (!fused && a.lse == nullptr) return TRN_E_NULL;
    if (!(a.tau > 0.f)) return TRN_E_SHAPE;
    if (a.noise_mode == TRN_NOISE_TENSOR && a.noise == nullptr) return TRN_E_NULL;
  }
  if (a.scores != nullptr) {
    if (a.score_pitch < a.P + a.M || (a.score_pitch & 31) != 0 || !aligned16(a.scores)) return TRN_E_SHAPE;
  }
  if (a.dtype != TRN_BF16 && a.dtype != TRN_FP16) return TRN_E_DTYPE;
  if (fstats != nullptr) fstats->done = 0;
  if (attn_small_applies(a)) {
    if (fstats != nullptr && fstats->sum_p != nullptr && attn_small_stats_applies(a, ds.sm_count)) {
      const int rc = launch_attn_small(a, st, ds, fstats);
      if (rc == TRN_OK) fstats->done = 1;
      return rc;
    }
    return launch_attn_small(a, st, ds);
  }
  if (a.dtype == TRN_BF16) return launch_typed<__nv_bfloat16>(a, st, ds);
  return launch_typed<__half>(a, st, ds);
}

}  // namespace trn
