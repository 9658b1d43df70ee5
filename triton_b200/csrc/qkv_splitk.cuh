// QKV projection for at most 32 rows (decode, the reference's M = 16 shapes): the weight stream split over the whole
// GPU.  Included by qkv_gemm.cu (shares its tile constants, Seg / GemmParams and tensor maps).
//
// With one row tile the persistent kernel has (Hq + 2 Hkv) D / 128 tiles — 96 CTAs for Llama's 4096 x 12288 weights —
// and each CTA's ring holds 96 KiB of weights in flight (a third of every stage is the 128-row x tile, all but 16 rows
// of it padding): the 100 MB weight read runs at about half of the HBM rate.  Here
//   * a stage holds only 32 rows of x (4 KiB) beside its 64 x 256 weight block, so six stages fit: 192 KiB of weights
//     in flight per CTA.  The 128-row MMA reads the 96 rows past the x tile from the weight block that follows it in
//     the stage; those accumulator rows are never looked at;
//   * a tile's contraction is cut into n_split ranges, one CTA each, the CTAs of a tile forming a thread-block
//     cluster.  The device holds only so many clusters of a size at once (B200: 74 of 2, 45 of 3, 33 of 4), so the
//     split is the largest with a resident cluster per 256-column tile (Llama's 48 tiles: 2); projections with more
//     than 74 such tiles use 384-column tiles (two MMAs per k step, four stages).
// Every CTA accumulates its range in tensor memory like the persistent kernel (TMA ring -> tcgen05.mma), then hands
// its first rows_pad accumulator rows as fp32 to rank 0's shared memory (st.shared::cluster between two cluster
// barriers; the operand ring is dead by then and is reused).  Rank 0 adds the parts in rank order — bitwise reproducible — and runs the usual epilogue (row
// scale, per-head RMS norm, gamma, head-split scatter / cache append) from shared memory with all of its threads.
// The weight loads of the first ring fill are issued BEFORE the wait on the previous kernel (programmatic dependent
// launch): weights are never written by the stream's kernels; x, the row scales and the outputs are touched after it.

constexpr int kSkThreads = 128;
constexpr int kSkARows = 32;                 // rows of x per stage (the TMA box; rows past the last one are zero-filled)
constexpr int kSkABytes = kSkARows * BK * 2; // 4 KiB
constexpr int kSkMaxSplit = 8;

template <int BN>
struct SkCfg {
  static constexpr int kStages = (BN == 256) ? 6 : 4;
  static constexpr int kStageBytes = kSkABytes + (BN / 64) * kBBlockBytes;   // 36 / 52 KiB
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kSmemBytes = kRingBytes + kBarBytes + 1024;
  static constexpr int kPitch = BN + 4;      // fp32 words per partial row: 16-byte stores of a warp spread over all banks
  static constexpr int kTmemCols = (BN == 256) ? 256 : 512;
};

template <typename T, int BN>
__global__ void __launch_bounds__(kSkThreads, 1)
qkv_splitk_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w0,
                  const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_w2,
                  const __grid_constant__ GemmParams p, const int n_split, const int rows_pad) {
  using Cfg = SkCfg<BN>;
  constexpr int kSkBN = BN, kSkStages = Cfg::kStages, kStageBytes = Cfg::kStageBytes, kSkPitch = Cfg::kPitch;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kSkStages * kStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kSkStages + s); };
  const uint32_t tfull_bar = bar_base + 8u * (2 * kSkStages);
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_gen + kSkStages * kStageBytes + 8 * (2 * kSkStages + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* skip_flag = abort_flag + 1;
  const uint32_t flags_base = bar_base + 128;        // kSkMaxSplit words: which ranks delivered their part

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  Ctl ctl{p.status, abort_flag};

  // this CTA's tile and contraction range
  const int tile = static_cast<int>(blockIdx.x) / n_split;
  const int seg = (tile >= p.seg[2].tile0) ? 2 : (tile >= p.seg[1].tile0 ? 1 : 0);
  const int n_tile = tile - p.seg[seg].tile0;
  const CUtensorMap* tm_w = seg == 0 ? &tm_w0 : (seg == 1 ? &tm_w1 : &tm_w2);
  const int k_steps_all = (p.K + BK - 1) / BK;
  const int k_lo = k_steps_all * static_cast<int>(rank) / n_split;
  const int k_hi = k_steps_all * (static_cast<int>(rank) + 1) / n_split;
  const int nk = k_hi - k_lo;
  const int first = nk < kSkStages ? nk : kSkStages;      // stages of the first ring fill
  auto load_w = [&](int i) {
    const uint32_t sb = smem_base + (i % kSkStages) * kStageBytes + kSkABytes;
#pragma unroll
    for (int c = 0; c < kSkBN / 64; ++c)
      tma_load_2d(sb + c * kBBlockBytes, tm_w, full_bar(i % kSkStages), n_tile * kSkBN + c * 64, (k_lo + i) * BK);
  };
  auto load_x = [&](int i) {
    tma_load_2d(smem_base + (i % kSkStages) * kStageBytes, &tm_x, full_bar(i % kSkStages), (k_lo + i) * BK, 0);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSkStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    // an earlier kernel gave up: do no work, but keep every cluster barrier below (the CTAs of a cluster may read
    // different values of the word; none of them may wait for one that left)
    const int skip = *reinterpret_cast<volatile int*>(p.status);
    *skip_flag = skip;
    fence_mbar_init();
    // The first ring fill's WEIGHT loads go out here, by the thread that has just initialised the barriers: before
    // the CTA meets (tensor-memory allocation is still under way) and before the wait on the previous kernel.
    if (skip == 0) {
      tma_prefetch_desc(tm_w);
      for (int i = 0; i < first; ++i) {
        mbar_expect_tx(full_bar(i), kStageBytes);
        load_w(i);
      }
      tma_prefetch_desc(&tm_x);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const bool active = *skip_flag == 0;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0 && active) {
      // x once the previous kernel of the stream has finished
      griddep_wait();
      for (int i = 0; i < first; ++i) load_x(i);
      uint32_t phase = 0;                       // parity of the ring pass being waited for
      for (int i = kSkStages; i < nk; ++i) {
        const int stage = i % kSkStages;
        if (stage == 0) phase ^= 1u;
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, ctl, KST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(full_bar(stage), kStageBytes);
        load_x(i);
        load_w(i);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && active) {
      constexpr uint32_t idesc = make_idesc_f16(Io<T>::kFmt, /*a_mn=*/0, /*b_mn=*/1, BM, 256);
      constexpr uint32_t idesc_tail = make_idesc_f16(Io<T>::kFmt, /*a_mn=*/0, /*b_mn=*/1, BM, 128);
      uint32_t phase = 0;
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int stage = i % kSkStages;
        if (i != 0 && stage == 0) phase ^= 1u;
        ok = mbar_wait(full_bar(stage), phase, ctl, KST_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_base + stage * kStageBytes;
        const uint32_t sb = sa + kSkABytes;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
          const uint64_t adesc = make_smem_desc(sa + kk * 32, 0, 1024);
          const uint64_t bdesc = make_smem_desc(sb + kk * 2048, kBBlockBytes, 1024);
          umma_ss(tmem_base, adesc, bdesc, idesc, (i | kk) != 0 ? 1u : 0u);
          if constexpr (BN == 384) {           // columns 256-383: the stage's fifth and sixth weight blocks
            const uint64_t bdesc2 = make_smem_desc(sb + 4 * kBBlockBytes + kk * 2048, kBBlockBytes, 1024);
            umma_ss(tmem_base + 256, adesc, bdesc2, idesc_tail, (i | kk) != 0 ? 1u : 0u);
          }
        }
        umma_commit(empty_bar(stage));
      }
      if (ok) umma_commit(tfull_bar);
    }
    __syncwarp();
  }
  griddep_wait();                 // every thread: the row scales are read and the outputs written after this point
  griddep_launch();

  // ------------------------------- accumulator complete -------------------------------
  bool done = active;
  if (done) done = mbar_wait(tfull_bar, 0, ctl, KST_TIMEOUT_CONSUMER);
  tc_fence_after();
  __syncthreads();                // the ring of this CTA is dead (all copies landed, all MMAs read them) or abandoned
  if (*abort_flag) {
    // a wait ran out: give copies / MMAs in flight time to land before the ring is reused
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (n_split > 1) cluster_sync_all_relaxed();          // ... and so is every other rank's, rank 0's included

  // ------------------------------- parts -> rank 0's shared memory -------------------------------
  // slot [rank][row][kSkPitch] fp32 at the start of rank 0's ring
  if (warp == 0 && done) {             // warp 0 owns tensor-memory lanes 0-31 = accumulator rows 0-31
    const uint32_t base0 = n_split > 1 ? map_to_rank(smem_base, 0) : smem_base;
    const uint32_t slot = base0 + (rank * rows_pad + lane) * (kSkPitch * 4);
#pragma unroll 1
    for (int c = 0; c < kSkBN / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_base + c * 32, r);          // warp-wide: lanes without a row take part and store nothing
      tmem_wait_ld();
      if (lane < rows_pad) {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          st_cluster_f4(slot + (c * 32 + i) * 4, __uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                        __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
      }
    }
  }
  // every rank tells rank 0 whether its part is there (a rank whose wait ran out has none)
  if (threadIdx.x == 0)
    st_cluster_u32((n_split > 1 ? map_to_rank(flags_base, 0) : flags_base) + rank * 4, done ? 1u : 0u);
  tc_fence_before();
  if (n_split > 1) cluster_sync_all(); else __syncthreads();

  // ------------------------------- rank 0: sum the parts, epilogue -------------------------------
  bool all_parts = done;
  for (int r = 0; r < n_split; ++r)
    all_parts = all_parts && reinterpret_cast<volatile uint32_t*>(smem_gen + kSkStages * kStageBytes + 128)[r] != 0u;
  if (rank == 0 && all_parts) {
    // a task = 64 columns of one row (a head of 64, or half a head of 128: the two halves sit in neighbouring lanes)
    const Seg& sg = p.seg[seg];
    constexpr int kUnits = kSkBN / 64;
    const int n_tasks = rows_pad * kUnits;
#pragma unroll 1
    for (int task = threadIdx.x; task < ((n_tasks + 31) & ~31); task += kSkThreads) {
      const int row = task / kUnits, unit = task - row * kUnits;
      const int col0 = n_tile * kSkBN + unit * 64;         // first of the task's columns within the segment
      const bool live = task < n_tasks && row < p.rows && col0 < sg.n;
      float v[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = 0.f;
      if (live) {
        const float* part = reinterpret_cast<const float*>(smem_gen) + row * kSkPitch + unit * 64;
        for (int r = 0; r < n_split; ++r) {
#pragma unroll
          for (int i = 0; i < 64; i += 4) {
            const float4 f = *reinterpret_cast<const float4*>(part + r * rows_pad * kSkPitch + i);
            v[i] += f.x; v[i + 1] += f.y; v[i + 2] += f.z; v[i + 3] += f.w;
          }
        }
      }
      const float rscale = (live && p.row_scale != nullptr) ? __ldg(p.row_scale + row) : 1.0f;
      float rs = rscale;
      if (sg.norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float x = v[i] * rscale;
          ss = fmaf(x, x, ss);
        }
        if (p.D == 128) ss += __shfl_xor_sync(0xffffffffu, ss, 1);       // the head's other 64 columns
        rs = rscale * rsqrtf(ss / static_cast<float>(p.D) + p.qk_eps);
      }
      if (live) {
        const int b = row / p.rows_per_batch, s = row - b * p.rows_per_batch;
        const int h = col0 / p.D, d0 = col0 - h * p.D;
        T* out = static_cast<T*>(sg.out) + static_cast<long long>(b) * sg.stride_b +
                 static_cast<long long>(sg.row_off + s) * sg.stride_s + static_cast<long long>(h) * sg.stride_h + d0;
#pragma unroll
        for (int i = 0; i < 64; i += 8) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = v[i + j] * rs;
          if (sg.gamma != nullptr) {
            const uint4 g = __ldg(reinterpret_cast<const uint4*>(static_cast<const T*>(sg.gamma) + d0 + i));
            const float2 g0 = Io<T>::unpack2(g.x), g1 = Io<T>::unpack2(g.y);
            const float2 g2 = Io<T>::unpack2(g.z), g3 = Io<T>::unpack2(g.w);
            f[0] *= g0.x; f[1] *= g0.y; f[2] *= g1.x; f[3] *= g1.y;
            f[4] *= g2.x; f[5] *= g2.y; f[6] *= g3.x; f[7] *= g3.y;
          }
          uint4 o;
          o.x = Io<T>::pack2(f[0], f[1]); o.y = Io<T>::pack2(f[2], f[3]);
          o.z = Io<T>::pack2(f[4], f[5]); o.w = Io<T>::pack2(f[6], f[7]);
          *reinterpret_cast<uint4*>(out + i) = o;
        }
      }
    }
  }

  // ------------------------------- teardown -------------------------------
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// rows of x a launch of this kernel can take; for a tile width, the tiles of the three segments and the largest split
// the shape allows (the launcher asks the device how many clusters of each size it can hold at once)
template <int BN>
inline bool splitk_shape_ok(const TrnProjArgs& a, int* rows_pad_out, int* tiles_out, int* max_split_out) {
  using Cfg = SkCfg<BN>;
  const long long rows = static_cast<long long>(a.B) * a.M;
  if (rows > kSkARows || (a.D != 64 && a.D != 128)) return false;
  const int rows_pad = rows <= 16 ? 16 : 32;
  const int k_steps = (a.N + BK - 1) / BK;
  int ns = kSkMaxSplit;
  // at least one ring pass of contraction per CTA, parts that fit in rank 0's ring
  while (ns > 1 && (k_steps < Cfg::kStages * ns || ns * rows_pad * Cfg::kPitch * 4 > Cfg::kRingBytes)) --ns;
  *rows_pad_out = rows_pad;
  *tiles_out = (a.Hq * a.D + BN - 1) / BN + 2 * ((a.Hkv * a.D + BN - 1) / BN);
  *max_split_out = ns;
  return ns > 1;
}
