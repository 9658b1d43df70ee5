// QKV projection on the 5th-gen tensor cores:  [q | k | v] = rowscale * (x @ [wq | wk | wv])
// with the epilogues the attention block needs fused in (ref_rms.py:47-56, 102-103, 217-220, 72-73):
//   * PreNorm's per-row rsqrt(mean x^2 + eps) applied to the accumulator row,
//   * QKNorm's per-(token, head) RMS norm over head_dim (+ gamma) on q and k,
//   * head-split scatter: q to the caller's q tensor, k / v appended at rows [P, P+M) of the caches.
//
// Shape of the kernel: persistent, one CTA per SM, 128 x 256 output tile (128 x 128 for problems of less
// than one wave), K step 64.
//   warp 0     TMA producer: x tile [128 x 64] (K-major) and w tile [64 x 256] (four 64-column
//              blocks, MN-major: w is used as x @ w so N is its contiguous dim) into a 4-stage ring
//   warp 1     allocates TMEM, one lane issues tcgen05.mma 128x256x16 (fp32 accumulators in TMEM,
//              two accumulator buffers of 256 columns so the epilogue overlaps the next tile)
//   warps 2-5  epilogue: tcgen05.ld the accumulator rows, scale / normalise, pack to 16-bit and
//              store 64-byte runs per thread
// The three weight matrices are separate tensors, so the tile space is three "segments", each with
// its own TMA descriptor and output addressing.
//
// Algorithmic work per launch: 2 * rows * N * (Hq + 2 Hkv) * D flops;
// compulsory bytes: x + wq + wk + wv + q + k + v once each.
#include "common.cuh"
#include "host.h"
#include "small_mma.cuh"

namespace trn {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kABytes = BM * BK * 2;          // 16 KiB
constexpr int kBBlockBytes = BK * 64 * 2;     // one 64-column block of w: 64 rows x 128 B = 8 KiB
constexpr int kThreads = 192;
constexpr int kBarBytes = 256;
#ifndef TRN_GEMM_GROUP_M
#define TRN_GEMM_GROUP_M 8
#endif
constexpr int kGroupM = TRN_GEMM_GROUP_M;     // m-tiles per raster group (L2 reuse of the w columns)

// Tile width BN: 256 columns for large problems; 128 when the 256-wide tiling would leave SMs idle (the
// reference's M = 16 shapes stream ~100 MB of weights through only 48 tiles otherwise).
template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kBBytes = kBBlockBytes * (BN / 64);
  static constexpr int kStageBytes = kABytes + kBBytes;        // 48 / 32 KiB
  static constexpr int kTmemCols = 2 * BN;                     // two accumulators of BN fp32 columns
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;   // +1024: manual 1 KiB alignment
};

struct Seg {
  void* out;
  const void* gamma;
  long long stride_b, stride_s, stride_h;
  int n;         // columns of this weight matrix (heads * D)
  int n_tiles;   // ceil(n / tile width)
  int tile0;     // first n-tile index of this segment in the concatenated tile space
  int row_off;   // position offset of row 0 inside the output (P for the caches, 0 for q)
  int norm;      // per-head RMS norm in the epilogue
};

struct GemmParams {
  Seg seg[3];
  const float* row_scale;
  int rows;            // B * M
  int rows_per_batch;  // M
  int K;               // hidden size N of the block
  int D;               // head_dim
  int m_tiles, n_tiles_total, total_tiles;
  float qk_eps;
  int K2;              // KCAT kernels: length of the second contraction phase (0 otherwise)
  int gate;            // GATED kernels: 0 = c1 * sigmoid(c1), 1 = sigmoid(c1)
  int* status;
};

struct TileCoord {
  int m_tile, seg, n_tile;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int t) {
  const int per_group = kGroupM * p.n_tiles_total;
  const int grp = t / per_group;
  const int r = t - grp * per_group;
  const int m0 = grp * kGroupM;
  const int gsz = min(kGroupM, p.m_tiles - m0);
  const int nt = r / gsz;
  TileCoord c;
  c.m_tile = m0 + (r - nt * gsz);
  c.seg = (nt >= p.seg[2].tile0) ? 2 : (nt >= p.seg[1].tile0 ? 1 : 0);
  c.n_tile = nt - p.seg[c.seg].tile0;
  return c;
}

// KCAT (LoRA, lora_benchmark.py:41-64: o = x @ w + d @ b with d = x @ a): a single output segment whose
// accumulator runs over two contraction phases, [x | d] @ [w ; b].  The descriptor slots are reused: tm_w0 = w,
// tm_w1 = b, tm_w2 = d (an activation like x).  Both products meet in fp32 in tensor memory.
//
// GATED (gated MLP, gmlp_benchmark.py:53-74: o = gate(x @ w1) * (x @ w2)): one output segment whose tile is BN / 2
// columns wide; the accumulator's first half holds x @ w1 and its second half x @ w2 for the SAME output columns
// (tm_w0 = w1, tm_w1 = w2, each feeding half of the stage's weight blocks), and the epilogue multiplies them.
//   FORM 0: plain projection, 1: KCAT, 2: GATED
template <typename T, int BN, int FORM>
__global__ void __launch_bounds__(kThreads, 1)
qkv_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w0,
                const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_w2,
                const __grid_constant__ GemmParams p) {
  // an earlier CTA / kernel gave up: leave before touching barriers or TMEM (decision is CTA-uniform)
  __shared__ int s_skip;
  if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;

  constexpr bool KCAT = (FORM == 1);
  constexpr bool GATED = (FORM == 2);
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr int kTmemCols = Cfg::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  // barrier layout (8 bytes each): full[4], empty[4], tmem_full[2], tmem_empty[2], then tmem ptr, abort
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * kStageBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Ctl ctl{p.status, abort_flag};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // the set-up above overlapped the previous kernel's tail (PreNorm's row statistics / X_norm); the next kernel
  // (attention) may begin its own set-up
  griddep_wait();
  griddep_launch();

  const int k_steps = (p.K + BK - 1) / BK;
  const int k_steps2 = KCAT ? (p.K2 + BK - 1) / BK : 0;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w0);
      tma_prefetch_desc(&tm_w1);
      tma_prefetch_desc(&tm_w2);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
      const TileCoord tc = decode_tile(p, t);
      const CUtensorMap* tm_w = tc.seg == 0 ? &tm_w0 : (tc.seg == 1 ? &tm_w1 : &tm_w2);
      for (int ks = 0; ks < k_steps; ++ks) {
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          mbar_expect_tx(full_bar(stage), kStageBytes);
          tma_load_2d(sa, &tm_x, full_bar(stage), ks * BK, tc.m_tile * BM);
          if constexpr (GATED) {
            constexpr int HB = BN / 128;           // 64-column blocks per half
#pragma unroll
            for (int c = 0; c < HB; ++c) {
              tma_load_2d(sb + c * kBBlockBytes, &tm_w0, full_bar(stage), tc.n_tile * (BN / 2) + c * 64, ks * BK);
              tma_load_2d(sb + (HB + c) * kBBlockBytes, &tm_w1, full_bar(stage), tc.n_tile * (BN / 2) + c * 64, ks * BK);
            }
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * kBBlockBytes, tm_w, full_bar(stage), tc.n_tile * BN + c * 64, ks * BK);
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if constexpr (KCAT) {
        // second phase: rows of d against the rows of b that belong to the same output columns
        for (int ks = 0; ks < k_steps2 && ok; ++ks) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1u, ctl, KST_TIMEOUT_PRODUCER);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (lane == 0) {
            const uint32_t sa = smem_base + stage * kStageBytes;
            const uint32_t sb = sa + kABytes;
            mbar_expect_tx(full_bar(stage), kStageBytes);
            tma_load_2d(sa, &tm_w2, full_bar(stage), ks * BK, tc.m_tile * BM);
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * kBBlockBytes, &tm_w1, full_bar(stage), tc.n_tile * BN + c * 64, ks * BK);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    constexpr uint32_t idesc = make_idesc_f16(Io<T>::kFmt, /*a_mn=*/0, /*b_mn=*/1, BM, BN);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      // A segment's last tile may hold fewer than BN columns (an MQA k / v head: 64 of 256): its MMAs are issued
      // only as wide as the columns that exist (rounded up to 64; an instruction's cost grows with its N), the
      // accumulator columns past them are never read
      uint32_t idesc_t = idesc;
      if constexpr (FORM == 0) {
        const TileCoord tcm = decode_tile(p, t);
        const int n_valid = p.seg[tcm.seg].n - tcm.n_tile * BN;
        if (n_valid < BN) idesc_t = make_idesc_f16(Io<T>::kFmt, /*a_mn=*/0, /*b_mn=*/1, BM, (n_valid + 63) & ~63);
      }
      ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, ctl, KST_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int ks = 0; ks < k_steps + k_steps2; ++ks) {
        ok = mbar_wait(full_bar(stage), phase, ctl, KST_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // x tile: K-major, 16 K-elements = 32 bytes inside the 128-byte swizzled row
            const uint64_t adesc = make_smem_desc(sa + kk * 32, 0, 1024);
            // w tile: MN-major, 16 K-rows = 2 KiB; 64-column blocks 8 KiB apart
            const uint64_t bdesc = make_smem_desc(sb + kk * 2048, kBBlockBytes, 1024);
            umma_ss(d_tmem, adesc, bdesc, idesc_t, (ks | kk) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));   // frees the stage when these MMAs have read it
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(tfull_bar(acc));
      __syncwarp();
    }
  } else {
    // ------------------------------- epilogue (warps 2..5) -------------------------------
    const int quad = warp & 3;                   // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const int r_in_tile = quad * 32 + lane;
    const int heads_per_tile = BN / p.D;
    const int chunks_per_head = p.D / 32;
    const float inv_d = 1.0f / static_cast<float>(p.D);
    bool ok = true;
    int it = 0;
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++it) {
      const TileCoord tc = decode_tile(p, t);
      const Seg& sg = p.seg[tc.seg];
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ok = mbar_wait(tfull_bar(acc), acc_phase, ctl, KST_TIMEOUT_CONSUMER);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();

      const int row = tc.m_tile * BM + r_in_tile;
      const bool valid_row = row < p.rows;
      const int b = valid_row ? row / p.rows_per_batch : 0;
      const int s = valid_row ? row - b * p.rows_per_batch : 0;
      const float rscale = (valid_row && p.row_scale != nullptr) ? __ldg(p.row_scale + row) : 1.0f;
      T* out_row = static_cast<T*>(sg.out) + static_cast<long long>(b) * sg.stride_b +
                   static_cast<long long>(sg.row_off + s) * sg.stride_s;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);

      if constexpr (GATED) {
        // o = gate(c1) * c2 on 32 columns at a time; gate = c1 * sigmoid(c1) (p.gate == 0) or sigmoid(c1)
        T* out_cols = out_row + tc.n_tile * (BN / 2);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          if (tc.n_tile * (BN / 2) + c * 32 >= sg.n) break;
          uint32_t r1[32], r2[32];
          tmem_ld32(t_row + c * 32, r1);
          tmem_ld32(t_row + BN / 2 + c * 32, r2);
          tmem_wait_ld();
          if (valid_row) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float c1 = __uint_as_float(r1[i + j]);
                const float sg1 = __fdividef(1.0f, 1.0f + __expf(-c1));
                f[j] = (p.gate == 0 ? c1 * sg1 : sg1) * __uint_as_float(r2[i + j]);
              }
              uint4 o;
              o.x = Io<T>::pack2(f[0], f[1]); o.y = Io<T>::pack2(f[2], f[3]);
              o.z = Io<T>::pack2(f[4], f[5]); o.w = Io<T>::pack2(f[6], f[7]);
              *reinterpret_cast<uint4*>(out_cols + c * 32 + i) = o;
            }
          }
        }
      } else
      for (int hh = 0; hh < heads_per_tile; ++hh) {
        const int col0 = tc.n_tile * BN + hh * p.D;
        if (col0 >= sg.n) break;
        const int h = col0 / p.D;
        float rs = rscale;
        uint32_t r[32];
        if (sg.norm) {
          float ss = 0.f;
          for (int c = 0; c < chunks_per_head; ++c) {
            tmem_ld32(t_row + hh * p.D + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float v = __uint_as_float(r[i]) * rscale;
              ss = fmaf(v, v, ss);
            }
          }
          rs = rscale * rsqrtf(ss * inv_d + p.qk_eps);
        }
        T* out_head = out_row + static_cast<long long>(h) * sg.stride_h;
        for (int c = 0; c < chunks_per_head; ++c) {
          tmem_ld32(t_row + hh * p.D + c * 32, r);
          tmem_wait_ld();
          if (valid_row) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[i + j]) * rs;
              if (sg.gamma != nullptr) {
                const uint4 g = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(sg.gamma) + c * 32 + i));
                const float2 g0 = Io<T>::unpack2(g.x), g1 = Io<T>::unpack2(g.y);
                const float2 g2 = Io<T>::unpack2(g.z), g3 = Io<T>::unpack2(g.w);
                f[0] *= g0.x; f[1] *= g0.y; f[2] *= g1.x; f[3] *= g1.y;
                f[4] *= g2.x; f[5] *= g2.y; f[6] *= g3.x; f[7] *= g3.y;
              }
              uint4 o;
              o.x = Io<T>::pack2(f[0], f[1]); o.y = Io<T>::pack2(f[2], f[3]);
              o.z = Io<T>::pack2(f[4], f[5]); o.w = Io<T>::pack2(f[6], f[7]);
              *reinterpret_cast<uint4*>(out_head + c * 32 + i) = o;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
    }
  }

  // ------------------------------- teardown -------------------------------
  __syncthreads();
  if (*abort_flag) {
    // a wait ran out: give copies / MMAs in flight time to land before the CTA's memory is reused
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

#include "qkv_splitk.cuh"
#include "qkv_gemm2.cuh"

// Extra operands of the LoRA form: o = x @ wq + d @ b (wk, wv unused).
struct KcatOperands {
  const void* d;   // [rows, K2]
  const void* b;   // [K2, heads_q * D]
  int K2;
};

template <typename T, int BN, int FORM>
int launch_tiled(const TrnProjArgs& a, cudaStream_t st, const DeviceState& ds, const KcatOperands* kc = nullptr,
                 int gate = 0, int n_split = 1, int rows_pad = 0, bool pairs = false) {
  constexpr bool KCAT = (FORM == 1);
  constexpr bool GATED = (FORM == 2);
  GemmParams p{};
  p.gate = gate;
  const int rows = a.B * a.M;
  p.rows = rows;
  p.rows_per_batch = a.M;
  p.K = a.N;
  p.D = a.D;
  p.row_scale = a.row_scale;
  p.qk_eps = a.qk_eps;
  p.status = ds.status;
  p.m_tiles = (rows + BM - 1) / BM;

  const void* w[3] = {a.wq, a.wk, a.wv};
  const TrnHeadTensor* outs[3] = {&a.q, &a.k_cache, &a.v_cache};
  const int heads[3] = {a.Hq, a.Hkv, a.Hkv};
  const void* gam[3] = {a.gamma_q, a.gamma_k, nullptr};
  CUtensorMap tm_w[3];
  int tile0 = 0;
  for (int i = 0; i < 3; ++i) {
    Seg& s = p.seg[i];
    s.out = outs[i]->ptr;
    s.stride_b = outs[i]->stride_b;
    s.stride_s = outs[i]->stride_s;
    s.stride_h = outs[i]->stride_h;
    s.n = heads[i] * a.D;
    s.n_tiles = GATED ? (i == 0 ? (s.n + BN / 2 - 1) / (BN / 2) : 0) : (s.n + BN - 1) / BN;
    s.tile0 = tile0;
    tile0 += s.n_tiles;
    s.row_off = (i == 0) ? 0 : a.P;
    s.norm = (a.qk_norm && i < 2) ? 1 : 0;
    s.gamma = s.norm ? gam[i] : nullptr;
    if (s.n == 0 || (GATED && i == 2)) {  // segment not present (single-output forms): placeholder descriptor
      tm_w[i] = tm_w[0];
      continue;
    }
    const uint64_t dims[2] = {static_cast<uint64_t>(s.n), static_cast<uint64_t>(a.N)};
    const uint64_t strides[2] = {1, static_cast<uint64_t>(s.n)};
    const uint32_t box[2] = {64, BK};
    int rc = make_tmap_16bit(&tm_w[i], w[i], 2, dims, strides, box);
    if (rc != TRN_OK) return rc;
  }
  if (KCAT) {
    // slot 1 = b [K2, n0], slot 2 = d [rows, K2]
    p.K2 = kc->K2;
    {
      const uint64_t dims[2] = {static_cast<uint64_t>(p.seg[0].n), static_cast<uint64_t>(kc->K2)};
      const uint64_t strides[2] = {1, static_cast<uint64_t>(p.seg[0].n)};
      const uint32_t box[2] = {64, BK};
      int rc = make_tmap_16bit(&tm_w[1], kc->b, 2, dims, strides, box);
      if (rc != TRN_OK) return rc;
    }
    {
      const uint64_t dims[2] = {static_cast<uint64_t>(kc->K2), static_cast<uint64_t>(rows)};
      const uint64_t strides[2] = {1, static_cast<uint64_t>(kc->K2)};
      const uint32_t box[2] = {BK, BM};
      int rc = make_tmap_16bit(&tm_w[2], kc->d, 2, dims, strides, box);
      if (rc != TRN_OK) return rc;
    }
  }
  p.n_tiles_total = tile0;
  p.total_tiles = p.m_tiles * p.n_tiles_total;

  CUtensorMap tm_x;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(rows)};
    const uint64_t strides[2] = {1, static_cast<uint64_t>(a.N)};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(n_split > 1 ? kSkARows : BM)};
    int rc = make_tmap_16bit(&tm_x, a.x, 2, dims, strides, box);
    if (rc != TRN_OK) return rc;
  }

  if constexpr (BN == 256 && FORM == 0) {
    if (pairs) {
      // CTA pairs (qkv_gemm2.cuh): 256 x 256 tiles, one pair of SMs each, persistent over the tiles
      p.m_tiles = (rows + 2 * BM - 1) / (2 * BM);
      p.total_tiles = p.m_tiles * p.n_tiles_total;
      auto pk = qkv_gemm2_kernel<T>;
      int rc = ensure_dyn_smem(reinterpret_cast<const void*>(pk), kG2SmemBytes, ds.device);
      if (rc != TRN_OK) return rc;
      const int max_pairs = ds.sm_count / 2;
      const int n_pairs = p.total_tiles < max_pairs ? p.total_tiles : max_pairs;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(static_cast<unsigned>(2 * n_pairs), 1, 1);
      cfg.blockDim = dim3(kG2Threads, 1, 1);
      cfg.dynamicSmemBytes = kG2SmemBytes;
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = pdl_enabled() ? 2 : 1;
      TRN_CUDA_TRY(cudaLaunchKernelEx(&cfg, pk, tm_x, tm_w[0], tm_w[1], tm_w[2], p));
      return TRN_OK;
    }
  }
  if constexpr ((BN == 256 || BN == 384) && FORM == 0) {
    if (n_split > 1 || BN == 384) {
      // at most 32 rows: the contraction of every tile split over a cluster of n_split CTAs (qkv_splitk.cuh)
      auto sk = qkv_splitk_kernel<T, BN>;
      int rc = ensure_dyn_smem(reinterpret_cast<const void*>(sk), SkCfg<BN>::kSmemBytes, ds.device);
      if (rc != TRN_OK) return rc;
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(static_cast<unsigned>(p.n_tiles_total * n_split), 1, 1);
      cfg.blockDim = dim3(kSkThreads, 1, 1);
      cfg.dynamicSmemBytes = SkCfg<BN>::kSmemBytes;
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(n_split);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = pdl_enabled() ? 2 : 1;
      TRN_CUDA_TRY(cudaLaunchKernelEx(&cfg, sk, tm_x, tm_w[0], tm_w[1], tm_w[2], p, n_split, rows_pad));
      return TRN_OK;
    }
  }
  if constexpr (BN != 384) {
    using Cfg = GemmCfg<BN>;
    auto kern = qkv_gemm_kernel<T, BN, FORM>;
    {
      int rc = ensure_dyn_smem(reinterpret_cast<const void*>(kern), Cfg::kSmemBytes, ds.device);
      if (rc != TRN_OK) return rc;
    }
    const int grid = p.total_tiles < ds.sm_count ? p.total_tiles : ds.sm_count;
    TRN_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, st, tm_x, tm_w[0], tm_w[1], tm_w[2], p));
  }
  return TRN_OK;
}

// Tile width and split of the contraction for at most 32 rows (split 1: the persistent kernel serves the shape): the
// pair that puts the most CTAs on the device while every tile's cluster is resident at once.  What the device can hold
// is asked once per tile width and cluster size (cudaOccupancyMaxActiveClusters: B200's GPCs do not all hold a
// multiple of every size).
template <typename T, int BN>
void splitk_plan_bn(const TrnProjArgs& a, const DeviceState& ds, int* best_bn, int* best_split, int* best_ctas, int* rows_pad) {
  int tiles = 0, max_split = 1, rp = 0;
  if (!splitk_shape_ok<BN>(a, &rp, &tiles, &max_split)) return;
  *rows_pad = rp;
  constexpr int kMaxDev = 64;
  static int resident[kMaxDev][kSkMaxSplit + 1];      // 0: not asked yet; -1: the query failed
  if (ds.device < 0 || ds.device >= kMaxDev) return;
  auto sk = qkv_splitk_kernel<T, BN>;
  if (ensure_dyn_smem(reinterpret_cast<const void*>(sk), SkCfg<BN>::kSmemBytes, ds.device) != TRN_OK) return;
  for (int ns = 2; ns <= max_split; ++ns) {
    int& r = resident[ds.device][ns];
    if (r == 0) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(static_cast<unsigned>(ns * 64), 1, 1);
      cfg.blockDim = dim3(kSkThreads, 1, 1);
      cfg.dynamicSmemBytes = SkCfg<BN>::kSmemBytes;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(ns);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      r = (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(sk), &cfg) == cudaSuccess && n > 0) ? n : -1;
      if (r < 0) (void)cudaGetLastError();
    }
    if (r >= tiles && tiles * ns > *best_ctas) { *best_bn = BN; *best_split = ns; *best_ctas = tiles * ns; }
  }
}

template <typename T>
int launch_typed(const TrnProjArgs& a, cudaStream_t st, const DeviceState& ds) {
  // A single row tile (M <= 128 tokens: decode / chunked prefill, the reference's own M = 16 shapes) streams
  // the weights once and is HBM-bound; 256-wide tiles would put that stream on too few SMs, so the narrower
  // tile is used when it fits in one wave.  Measured with the weights coming from HBM (L2 flushed between
  // calls), M = 16, N = 4096: 32.9 us against 41.0 us; with several row tiles the wide tile wins (M = 512:
  // 37.3 us against 49.6 us).
  // At most 32 rows: the contraction is split as well (qkv_splitk.cuh), which puts the stream on every SM.
  const long long m_tiles = (static_cast<long long>(a.B) * a.M + BM - 1) / BM;
  const long long n128 = (a.Hq * a.D + 127) / 128 + 2LL * ((a.Hkv * a.D + 127) / 128);
  int rows_pad = 0, bn = 0, n_split = 1, ctas = 0;
  // 256-column tiles where the device can hold a cluster per tile; 384-column tiles only for projections too wide for
  // that (measured, weights from HBM: Llama M16 32.5 us with 256 x 2 on 96 CTAs against 37.0 with 384 x 4 on 132 —
  // more SMs do not help once the stream is DRAM-bound, the larger exchange costs — but N 8192, 3 x 8192 columns:
  // 86.8 us with 384 x 2 against 105.3 for the persistent kernel, where 96 tiles of 256 find no resident split)
  splitk_plan_bn<T, 256>(a, ds, &bn, &n_split, &ctas, &rows_pad);
  if (n_split == 1) splitk_plan_bn<T, 384>(a, ds, &bn, &n_split, &ctas, &rows_pad);
  if (n_split > 1 && bn == 384) return launch_tiled<T, 384, 0>(a, st, ds, nullptr, 0, n_split, rows_pad);
  if (n_split > 1) return launch_tiled<T, 256, 0>(a, st, ds, nullptr, 0, n_split, rows_pad);
  if (m_tiles == 1 && n128 <= 2LL * ds.sm_count) return launch_tiled<T, 128, 0>(a, st, ds);
  // several row tiles: CTA pairs (qkv_gemm2.cuh) once there is a wave of 256 x 256 tiles for the pairs of SMs
  const long long n256 = (a.Hq * a.D + 255) / 256 + 2LL * ((a.Hkv * a.D + 255) / 256);
  const bool pairs = ((m_tiles + 1) / 2) * n256 >= ds.sm_count / 2;
  return launch_tiled<T, 256, 0>(a, st, ds, nullptr, 0, 1, 0, pairs);
}

bool head_tensor_ok(const TrnHeadTensor& t) {
  return t.ptr != nullptr && aligned16(t.ptr) && (t.stride_b & 7) == 0 && (t.stride_s & 7) == 0 &&
         (t.stride_h & 7) == 0;
}

// o[M, P] = x[M, N] @ w[N, P] + (x @ a[N, R]) @ b[R, P]: two launches of the projection kernel.  The first writes
// d = x @ a (16-bit, as the reference's programs keep it); the second runs both contraction phases into one
// accumulator.  Outputs are addressed as "heads" of 64 columns.
template <typename T>
int launch_lora_typed(const TrnLoraArgs& a, cudaStream_t st, const DeviceState& ds) {
  auto plain = [&](const void* x, const void* w, void* out, int n_out) {
    TrnProjArgs pj{};
    pj.x = x;
    pj.wq = w; pj.wk = w; pj.wv = w;          // only the first segment exists (Hkv = 0)
    pj.B = 1; pj.M = a.M; pj.P = 0; pj.N = a.N;
    pj.Hq = n_out / 64; pj.Hkv = 0; pj.D = 64;
    pj.dtype = a.dtype;
    pj.q.ptr = out;
    pj.q.stride_b = static_cast<int64_t>(a.M) * n_out;
    pj.q.stride_s = n_out;
    pj.q.stride_h = 64;
    pj.k_cache = pj.q;
    pj.v_cache = pj.q;
    return pj;
  };
  const TrnProjArgs p1 = plain(a.x, a.a, a.d, a.R);
  int rc = launch_typed<T>(p1, st, ds);
  if (rc != TRN_OK) return rc;
  const TrnProjArgs p2 = plain(a.x, a.w, a.o, a.P);
  const KcatOperands kc{a.d, a.b, a.R};
  const long long m_tiles = (static_cast<long long>(a.M) + BM - 1) / BM;
  const long long n128 = (a.P + 127) / 128;
  if (m_tiles == 1 && n128 <= 2LL * ds.sm_count) return launch_tiled<T, 128, 1>(p2, st, ds, &kc);
  return launch_tiled<T, 256, 1>(p2, st, ds, &kc);
}

// o[M, N] = gate(x[M, K] @ w1[K, N]) * (x @ w2[K, N]): one launch; outputs addressed as "heads" of 64 columns.
// The second weight rides in the k slot: its segment has the same column count, but GATED kernels tile segment 0 only.
template <typename T>
int launch_gmlp_typed(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds) {
  TrnProjArgs pj{};
  pj.x = a.x;
  pj.wq = a.w1; pj.wk = a.w2; pj.wv = a.w1;
  pj.B = 1; pj.M = a.M; pj.P = 0; pj.N = a.K;
  pj.Hq = a.N / 64; pj.Hkv = a.N / 64; pj.D = 64;
  pj.dtype = a.dtype;
  pj.q.ptr = a.o;
  pj.q.stride_b = static_cast<int64_t>(a.M) * a.N;
  pj.q.stride_s = a.N;
  pj.q.stride_h = 64;
  pj.k_cache = pj.q;
  pj.v_cache = pj.q;
  const long long m_tiles = (static_cast<long long>(a.M) + BM - 1) / BM;
  const long long n64 = (a.N + 63) / 64;
  // a single row tile streams the weights once: narrow tiles (64 output columns) put that stream on more SMs
  if (m_tiles == 1 && n64 <= 2LL * ds.sm_count) return launch_tiled<T, 128, 2>(pj, st, ds, nullptr, a.gate);
  return launch_tiled<T, 256, 2>(pj, st, ds, nullptr, a.gate);
}

}  // namespace

int launch_gmlp(const TrnGmlpArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.x == nullptr || a.w1 == nullptr || a.w2 == nullptr || a.o == nullptr) return TRN_E_NULL;
  if (a.M <= 0 || a.K <= 0 || a.N <= 0) return TRN_E_SHAPE;
  if ((a.K & 7) != 0 || (a.N & 31) != 0) return TRN_E_SHAPE;
  if (!aligned16(a.x) || !aligned16(a.w1) || !aligned16(a.w2) || !aligned16(a.o)) return TRN_E_ALIGN;
  if (a.gate != TRN_GATE_SILU && a.gate != TRN_GATE_SIGMOID) return TRN_E_VARIANT;
  if (a.dtype != TRN_BF16 && a.dtype != TRN_FP16) return TRN_E_DTYPE;
  if (gmlp_small_applies(a)) return launch_gmlp_small(a, st, ds);
  if ((a.N & 63) != 0) return TRN_E_SHAPE;       // the tensor-memory kernel stores 64-column blocks
  if (a.dtype == TRN_BF16) return launch_gmlp_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_gmlp_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

int launch_lora(const TrnLoraArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.x == nullptr || a.w == nullptr || a.a == nullptr || a.b == nullptr || a.o == nullptr || a.d == nullptr)
    return TRN_E_NULL;
  if (a.M <= 0 || a.N <= 0 || a.P <= 0 || a.R <= 0) return TRN_E_SHAPE;
  if ((a.N & 7) != 0 || (a.P & 63) != 0 || (a.R & 63) != 0) return TRN_E_SHAPE;
  if (!aligned16(a.x) || !aligned16(a.w) || !aligned16(a.a) || !aligned16(a.b) || !aligned16(a.o) || !aligned16(a.d))
    return TRN_E_ALIGN;
  if (a.dtype != TRN_BF16 && a.dtype != TRN_FP16) return TRN_E_DTYPE;
  if (lora_small_applies(a)) return launch_lora_small(a, st, ds);
  if (a.dtype == TRN_BF16) return launch_lora_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_lora_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

int launch_qkv_project(const TrnProjArgs& a, cudaStream_t st, const DeviceState& ds) {
  if (a.x == nullptr || a.wq == nullptr || a.wk == nullptr || a.wv == nullptr) return TRN_E_NULL;
  if (a.q.ptr == nullptr || a.k_cache.ptr == nullptr || a.v_cache.ptr == nullptr) return TRN_E_NULL;
  if (a.B <= 0 || a.M <= 0 || a.P < 0 || a.N <= 0 || a.Hq <= 0 || a.Hkv <= 0) return TRN_E_SHAPE;
  if (a.D != 64 && a.D != 128) return TRN_E_SHAPE;
  if ((a.N & 7) != 0) return TRN_E_SHAPE;
  if (static_cast<long long>(a.B) * a.M > 0x7fffffffLL) return TRN_E_SHAPE;
  if (!aligned16(a.x) || !aligned16(a.wq) || !aligned16(a.wk) || !aligned16(a.wv)) return TRN_E_ALIGN;
  if (!aligned16(a.gamma_q) || !aligned16(a.gamma_k)) return TRN_E_ALIGN;
  if (!head_tensor_ok(a.q) || !head_tensor_ok(a.k_cache) || !head_tensor_ok(a.v_cache)) return TRN_E_ALIGN;
  if (a.dtype == TRN_BF16) return launch_typed<__nv_bfloat16>(a, st, ds);
  if (a.dtype == TRN_FP16) return launch_typed<__half>(a, st, ds);
  return TRN_E_DTYPE;
}

}  // namespace trn
